// Flash-attention forward for sm_100a (head dim up to 128, f16 / bf16, f32 accumulate).  The tiles are
// 128 head dims wide; a narrower head (a multiple of 8: 32, 64, 96 ...) is the same computation with
// the missing columns read as zeros and never written, which the tensor maps do by themselves: their
// innermost extent is the head dim, loads past it fill zeros, stores past it are clipped.
//
// Persistent blocks, one per SM.  A block takes query tiles (128 query rows of one (batch,
// head)) from a static list and, for each, walks over the key/value tiles of 128 rows that
// the mask lets it see.  A work item is one (batch, head) and a pair of query tiles, the t-th
// longest and the t-th shortest, so that under a causal mask all items cost the same; items
// go round-robin over the blocks, consecutive items share K and V in L2.  Every barrier keeps
// counting across query tiles, so the loads and the first S of the next query tile overlap
// the epilogue of the current one.  Warp roles (three warpgroups):
//   warp 0        TMA producer of Q (per query tile) and of the K tiles (2-stage ring)
//   warp 2        TMA producer of the V tiles (2-stage ring)
//   warp 1        issuer of S = Q K^T  (tcgen05.mma; all lanes run the loop and the waits,
//   warp 3        issuer of O += P V    one elected lane executes the tcgen05 instructions)
//   warps 4..7    softmax group 0: key tiles 0, 2, 4, ...
//   warps 8..11   softmax group 1: key tiles 1, 3, 5, ...
// Tensor memory (all 512 columns): S 0,128 | P 256,320 | O 384.  Each group has its own S
// tile and its own P tile, so the next S of a group is computed while the group still works
// on its current tile and nothing waits for a buffer; the one O accumulator takes P V of all
// tiles in order.  Inside a group thread t owns query row t: it reads its row of S, finds
// the row maximum, writes P (16-bit) to tensor memory, where it is the A operand of P V
// (tcgen05.mma with A in tensor memory), and keeps a partial row sum.
//
// One accumulator for two groups needs one reference maximum per row that both threads of the
// row agree on.  It is the running maximum of the sequential algorithm: every thread replays
// the same steps over ALL key tiles (ref_step), its own tiles from its own maxima, the other
// group's tiles from the maxima that group publishes in shared memory right after finding
// them (long before they are needed, so the wait is a formality).  The step of tile j belongs
// to the group of tile j: if the reference moved, that thread multiplies the row of O by
// 2^(old - new) after P V of tile j - 1 has completed and before it hands over P of tile j;
// the P V issuer takes the tiles in order, so no product ever sees a half-rescaled row.  Both
// threads scale their partial sums by every step's factor.  The reference only moves when a
// row of the warp grew by more than 2^8, so rescaling is rare after the first tiles.
// At the end the two partial sums are added (the thread that is one step behind scales
// its sum by the last factor), each thread finishes 64 head-dim columns of its row.
// The control warps give most of their registers to the softmax warps (setmaxnreg).
//
// Numerics follow the reference kernel (external_libs/runtime/flash_attn/lib/
// softmax.h:129-178, flash_fwd_kernel.h:276-453): exp2 domain with the scale
// folded in, row sum from the unrounded f32 probabilities, P rounded to the
// storage type before P V, LSE = max * scale + ln(sum), +inf for a fully masked
// row.  One deviation that stays inside the rounding of P: the stale reference
// (at most 2^8 below the true running maximum) is used consistently for P, the
// row sum and the LSE.
#include <cuda.h>

#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace b200 {
namespace {

constexpr int kBM = 128;        // query rows per block
constexpr int kBN = 128;        // key rows per tile
constexpr int kD = 128;         // head dim
constexpr uint32_t kTileBytes = kBN * kD * 2;  // 32 KiB: two 64-column blocks of 128 x 128 B
constexpr uint32_t kHalfTile = kTileBytes / 2; // one 64-column block
constexpr int kThreads = 384;    // four control warps, two groups of four softmax / elementwise warps
constexpr uint32_t kTmemCols = 512;
// forward: two S tiles, two P tiles and one O accumulator fill the 512 columns of tensor memory
constexpr int kFwdKStages = 2, kFwdVStages = 2; // K / V ring depths of the forward kernel
constexpr uint32_t kColS0 = 0, kColS1 = 128, kColP0 = 256, kColP1 = 320, kColO = 384;
constexpr int kCtrlRegs = 56, kSoftmaxRegs = 224; // 128 * 56 + 256 * 224 <= 64 Ki registers
constexpr float kRescaleThreshold = 8.0f; // log2 units

// Sticky status of the attention kernels on this device: 0, or the code of the last kernel whose
// bounded wait ran out (2 forward, 3 backward).  Device code names it directly; the host reads and
// clears it with b200_flash_attn_take_status.
static __device__ int g_attn_status;

// Host-side test hook (b200_flash_attn_debug): polls per bounded wait, and whether the elementwise
// warps leave out the arrival that hands P (forward) or P / dS (backward) to the MMA issuer, so
// that a wait runs out without anything faulting.
uint32_t g_wait_polls = 100000u;
int g_debug_skip_arrive = 0;

struct FwdParams {
  float *lse;
  int *status;
  uint32_t wait_polls;
  int debug_skip_arrive;
  int d; // head dim, <= 128
  int64_t H, Hk, Sq, Sk;
  int n_q_tiles, pairs; // query tiles per (batch, head); pairs of them per work item
  int64_t total_items;  // pairs * H * B
  float scale_log2;
  int64_t window_left, window_right; // < 0: unbounded
};

// Two f32 in one 64-bit register for the packed FMA / ADD of sm_100 (one issue slot for two
// results); the softmax loop is bound by instruction issue, not by any one pipe.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Named barrier 1 over the N worker threads of a block that also ORs a predicate, so that a
// decision to give up is taken by all of them together (nobody is left waiting at a barrier).
template <int N> __device__ __forceinline__ bool named_bar_or_n(bool pred) {
  uint32_t out;
  asm volatile("{\n"
               ".reg .pred p, q;\n"
               "setp.ne.u32 q, %1, 0;\n"
               "bar.red.or.pred p, 1, %2, q;\n"
               "selp.u32 %0, 1, 0, p;\n"
               "}\n"
               : "=r"(out)
               : "r"((uint32_t)pred), "n"(N)
               : "memory");
  return out != 0;
}

// the same over 128 threads with the barrier number chosen at run time
__device__ __forceinline__ bool named_bar_or_id(int id, bool pred) {
  uint32_t out;
  asm volatile("{\n"
               ".reg .pred p, q;\n"
               "setp.ne.u32 q, %1, 0;\n"
               "bar.red.or.pred p, %2, 128, q;\n"
               "selp.u32 %0, 1, 0, p;\n"
               "}\n"
               : "=r"(out)
               : "r"((uint32_t)pred), "r"(id)
               : "memory");
  return out != 0;
}

// Registers move from the control warps to the softmax warps at run time (all four warps
// of a warpgroup execute the instruction).
template <int N> __device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

struct SharedStorage {
  uint64_t bar_q, q_empty; // Q of a query tile has arrived / is no longer read
  uint64_t k_full[kFwdKStages], k_empty[kFwdKStages], v_full[kFwdVStages], v_empty[kFwdVStages];
  uint64_t s_full[2], s_empty[2]; // per softmax group: S of its tile is in tensor memory / in registers
  uint64_t p_full[2];             // per softmax group: P of its tile is in tensor memory, O is rescaled
  uint64_t pv_done[2];            // per softmax group: the P V of its tile has completed
  // per softmax group and tile parity: the row maxima of the group's tile are in `rowmax`.
  // One barrier per tile parity, so that a reader never has to tell apart two phases of the
  // same parity even if the publisher is a tile ahead of it.
  uint64_t mx_ready[2][2];
  uint32_t tmem_base;
  int failed;
  alignas(16) float rowmax[2][2][kBM]; // [group][tile parity][row]: scaled row maximum of the group's tile
  float2 xch[2][kBM];      // (reference max, row sum) of each group, for the final merge
};

__device__ __forceinline__ bool wait_or_flag(uint64_t *bar, uint32_t parity, SharedStorage *ss, uint32_t polls) {
  if (mbar_wait(bar, parity, polls))
    return true;
  ss->failed = 1; // some arrival never came: every role gives up at its next wait
  return false;
}

// The MMA-issuing warps run their loops with all 32 lanes (waits included) and only the
// tcgen05 instructions themselves are executed by one elected lane: descriptors and
// addresses then live in uniform registers, which is what the instruction takes, and
// an issue costs ~10 cycles instead of ~55 from inside a single-lane branch.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n"
               ".reg .pred P;\n"
               "elect.sync _|P, 0xffffffff;\n"
               "selp.u32 %0, 1, 0, P;\n"
               "}\n"
               : "=r"(pred));
  return pred != 0;
}
// all 32 lanes wait; the verdict is the same in every lane, so a warp gives up as a whole and
// the warp-wide votes and tensor-memory instructions that follow a wait stay convergent
__device__ __forceinline__ bool warp_wait_or_flag(uint64_t *bar, uint32_t parity, SharedStorage *ss, uint32_t polls) {
  const bool ok = __all_sync(0xffffffffu, mbar_wait(bar, parity, polls));
  if (!ok)
    ss->failed = 1;
  return ok;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, bool bf16) {
  if (bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

// One step of the running reference maximum of the rows of a warp: `m` are the rows' (scaled)
// maxima of key tile `tile`.  The reference only moves when some row of the warp grew by more
// than 2^8 (then every row of the warp takes its new maximum), so that O is rescaled rarely.
// Returns whether it moved; alpha = 2^(old - new) is the factor for everything accumulated so far.
__device__ __forceinline__ bool ref_step(int tile, float m, float &ref, float &alpha) {
  const float m_new = fmaxf(ref, m);
  const bool grew = m_new - ref > kRescaleThreshold; // also true for -inf -> finite
  const bool moved = tile > 0 && __any_sync(0xffffffffu, grew);
  alpha = 1.f;
  if (tile == 0) {
    ref = m_new;
  } else if (moved) {
    alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(ref - m_new);
    ref = m_new;
  }
  return moved;
}

template <bool kBF16>
__global__ void __launch_bounds__(kThreads, 1)
    flash_fwd_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                     const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap o_map,
                     const FwdParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *smem =
      reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *sQ = smem;              // Q of the current query tile
  unsigned char *sO = sQ + kTileBytes;   // the finished O tile on its way out
  unsigned char *sK = sO + kTileBytes;
  unsigned char *sV = sK + kFwdKStages * kTileBytes;
  SharedStorage *ss = reinterpret_cast<SharedStorage *>(sV + kFwdVStages * kTileBytes);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31; // warp: known uniform
  const int64_t shift = p.Sk - p.Sq;
  const bool right_bounded = p.window_right >= 0;
  const bool left_bounded = p.window_left >= 0;
  const int kv_group = (int)(p.H / p.Hk);

  // The block's work list.  The blocks are persistent (one per SM).  An item is one (batch, head)
  // and a pair of query tiles, the t-th longest and the t-th shortest, so that under a causal
  // mask every item costs the same; items go round-robin over the blocks, consecutive items
  // share K and V.  Every role walks the same list of query tiles, two per item, and every
  // barrier keeps counting across query tiles, so loads and the first products of the next
  // query tile overlap the epilogue of the current one.
  struct Work {
    int h, b, hk, n; // n: key tiles (128 keys each) this query tile visits, [0, n)
    int64_t q0;
  };
  auto work_at = [&](int idx, Work &w) -> int { // 1: work, 0: nothing at idx (odd middle tile), -1: list ended
    const int64_t item = (int64_t)blockIdx.x + (int64_t)(idx >> 1) * gridDim.x;
    if (item >= p.total_items)
      return -1;
    const int pr = (int)(item % p.pairs);
    const int64_t bh = item / p.pairs;
    const int hi = p.n_q_tiles - 1 - pr;
    if ((idx & 1) && pr == hi)
      return 0;
    const int q_tile = (idx & 1) ? pr : hi;
    w.h = (int)(bh % p.H);
    w.b = (int)(bh / p.H);
    w.hk = w.h / kv_group;
    w.q0 = (int64_t)q_tile * kBM;
    int n = (int)((p.Sk + kBN - 1) / kBN);
    if (right_bounded) {
      const int64_t last_visible = w.q0 + kBM - 1 + shift + p.window_right;
      n = last_visible < 0 ? 0 : (int)min((int64_t)n, last_visible / kBN + 1);
    }
    w.n = n;
    return 1;
  };
  auto next_work = [&](int &idx, Work &w) -> bool { // advances idx to the next query tile of the list
    for (;;) {
      const int r = work_at(idx, w);
      if (r < 0)
        return false;
      ++idx;
      if (r > 0)
        return true;
    }
  };

  if (threadIdx.x == 0) {
    mbar_init(&ss->bar_q, 1);
    mbar_init(&ss->q_empty, 1);
    for (int s = 0; s < kFwdKStages; ++s) {
      mbar_init(&ss->k_full[s], 1);
      mbar_init(&ss->k_empty[s], 1);
    }
    for (int s = 0; s < kFwdVStages; ++s) {
      mbar_init(&ss->v_full[s], 1);
      mbar_init(&ss->v_empty[s], 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&ss->s_full[g], 1);
      mbar_init(&ss->s_empty[g], 4);
      mbar_init(&ss->p_full[g], 4);
      mbar_init(&ss->pv_done[g], 1);
      mbar_init(&ss->mx_ready[g][0], 4);
      mbar_init(&ss->mx_ready[g][1], 4);
    }
    ss->failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ss->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ss->tmem_base;

  if (warp < 4)
    reg_dec<kCtrlRegs>(); // the four control warps hand registers to the softmax warps
  if (warp == 0) {
    // ----------------------------------------------------------- producer of Q and K
    if (lane == 0) {
      prefetch_tensormap(&q_map);
      prefetch_tensormap(&k_map);
      uint32_t kc = 0, qc = 0; // K tiles and Q tiles loaded so far
      int idx = 0;
      Work w;
      bool ok = true;
      while (ok && next_work(idx, w)) {
        if (w.n == 0)
          continue;
        // Q's buffer is free once the last Q K^T of the previous query tile has completed
        if (qc > 0 && !wait_or_flag(&ss->q_empty, (qc - 1) & 1, ss, p.wait_polls))
          break;
        mbar_arrive_expect_tx(&ss->bar_q, kTileBytes);
        tma_load_4d(sQ, &q_map, 0, w.h, (int)w.q0, w.b, &ss->bar_q);
        tma_load_4d(sQ + kHalfTile, &q_map, 64, w.h, (int)w.q0, w.b, &ss->bar_q);
        ++qc;
        for (int j = 0; j < w.n; ++j, ++kc) {
          const int st = kc % kFwdKStages;
          if (!wait_or_flag(&ss->k_empty[st], ((kc / kFwdKStages) & 1) ^ 1, ss, p.wait_polls)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&ss->k_full[st], kTileBytes);
          tma_load_4d(sK + st * kTileBytes, &k_map, 0, w.hk, j * kBN, w.b, &ss->k_full[st]);
          tma_load_4d(sK + st * kTileBytes + kHalfTile, &k_map, 64, w.hk, j * kBN, w.b, &ss->k_full[st]);
        }
      }
    }
  } else if (warp == 2) {
    // ----------------------------------------------------------- producer of V
    if (lane == 0) {
      prefetch_tensormap(&v_map);
      uint32_t vc = 0;
      int idx = 0;
      Work w;
      bool ok = true;
      while (ok && next_work(idx, w)) {
        for (int j = 0; j < w.n; ++j, ++vc) {
          const int st = vc % kFwdVStages;
          if (!wait_or_flag(&ss->v_empty[st], ((vc / kFwdVStages) & 1) ^ 1, ss, p.wait_polls)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&ss->v_full[st], kTileBytes);
          tma_load_4d(sV + st * kTileBytes, &v_map, 0, w.hk, j * kBN, w.b, &ss->v_full[st]);
          tma_load_4d(sV + st * kTileBytes + kHalfTile, &v_map, 64, w.hk, j * kBN, w.b, &ss->v_full[st]);
        }
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------------------- issuer of S = Q K^T
    // S of a group is free as soon as the group has its previous tile in registers, so the
    // next S is normally ready before the group asks for it, across query tiles as well.
    constexpr uint32_t idesc_qk = umma_idesc_f16(kBF16, kBM, kBN, false, false);
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t q_addr = smem_addr(sQ), k_addr = smem_addr(sK);
    uint32_t kc = 0, qc = 0, tc[2] = {0, 0}; // K tiles, Q tiles, tiles per softmax group so far
    int idx = 0;
    Work w;
    bool ok = true;
    while (ok && next_work(idx, w)) {
      if (w.n == 0)
        continue;
      ok = warp_wait_or_flag(&ss->bar_q, qc & 1, ss, p.wait_polls);
      ++qc;
      for (int j = 0; ok && j < w.n; ++j, ++kc) {
        const int g = j & 1, st = kc % kFwdKStages;
        ok = warp_wait_or_flag(&ss->k_full[st], (kc / kFwdKStages) & 1, ss, p.wait_polls) &&
             warp_wait_or_flag(&ss->s_empty[g], (tc[g] & 1) ^ 1, ss, p.wait_polls);
        if (!ok)
          break;
        ++tc[g];
        tc_fence_after_sync();
        const uint32_t d_tmem = tm + (g ? kColS1 : kColS0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) { // 8 steps of 16 head dims
          const uint32_t off = (kk >> 2) * kHalfTile + (kk & 3) * 32;
          const uint64_t adesc = umma_smem_desc(q_addr + off, 16, 1024);
          const uint64_t bdesc = umma_smem_desc(k_addr + st * kTileBytes + off, 16, 1024);
          if (elect_one())
            umma_ss(d_tmem, adesc, bdesc, idesc_qk, kk != 0);
        }
        if (elect_one()) {
          umma_commit(&ss->s_full[g]);
          umma_commit(&ss->k_empty[st]);
          if (j + 1 == w.n)
            umma_commit(&ss->q_empty); // the query tile's last product: Q may be replaced
        }
      }
    }
  } else if (warp == 3) {
    // ----------------------------------------------------------- issuer of O += P V
    constexpr uint32_t idesc_pv = umma_idesc_f16(kBF16, kBM, kD, false, true);
    const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
    const uint32_t v_addr = smem_addr(sV);
    uint32_t vc = 0, tc[2] = {0, 0};
    int idx = 0;
    Work w;
    bool ok = true;
    while (ok && next_work(idx, w)) {
      for (int j = 0; ok && j < w.n; ++j, ++vc) {
        const int g = j & 1, st = vc % kFwdVStages;
        ok = warp_wait_or_flag(&ss->v_full[st], (vc / kFwdVStages) & 1, ss, p.wait_polls) &&
             warp_wait_or_flag(&ss->p_full[g], tc[g] & 1, ss, p.wait_polls);
        if (!ok)
          break;
        ++tc[g];
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) { // 8 steps of 16 keys
          // A: P[:, 16 keys] in tensor memory; B: V[16 keys, 128 dims] (dims contiguous = MN-major)
          const uint64_t bdesc = umma_smem_desc(v_addr + st * kTileBytes + kk * 16 * 128, kHalfTile, 1024);
          if (elect_one())
            umma_ts(tm + kColO, tm + (g ? kColP1 : kColP0) + kk * 8, bdesc, idesc_pv, (j | kk) != 0);
        }
        if (elect_one()) {
          umma_commit(&ss->pv_done[g]);
          umma_commit(&ss->v_empty[st]);
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------- softmax
    reg_inc<kSoftmaxRegs>();
    const int g = (warp - 4) >> 2;           // group: key tiles g, g + 2, g + 4, ... of a query tile
    const int quarter = warp & 3;            // tensor-memory lanes 32 * quarter .. + 31
    const int row = quarter * 32 + lane;     // query row inside the tile
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t col_s = g ? kColS1 : kColS0, col_p = g ? kColP1 : kColP0;
    uint32_t tc[2] = {0, 0}; // key tiles of [this group, the other group] over all query tiles so far
    bool ok = true;
    int idx = 0;
    Work w;
    while (next_work(idx, w)) {
      const int n = w.n;
      const int64_t q0 = w.q0, qrow = q0 + row;
      const int n_mine = (n + 1 - g) >> 1, n_other = (n + g) >> 1;
      // `ref` is the reference maximum of the row after the last tile this thread knows about:
      // both threads of a row replay the same sequence of steps (ref_step) over all key tiles,
      // the other group's tiles from the maxima it publishes.
      float ref = -INFINITY, l = 0.f;
      for (int i = 0; ok && i < n_mine; ++i) {
        const int j = 2 * i + g;
        const uint32_t ti = tc[0] + i; // this tile's number among the group's tiles of the whole list
        // The other group's maxima of the tile before: it published them early in its tile, half
        // a period ago, so this wait is a formality; it is taken here, where the thread would
        // otherwise idle until its S arrives, and not between the maximum and the exponentials.
        float m_other = -INFINITY;
        if (j > 0) {
          const uint32_t to = tc[1] + ((j - 1) >> 1); // tile j - 1 among the other group's tiles
          if (!warp_wait_or_flag(&ss->mx_ready[g ^ 1][to & 1], (to >> 1) & 1, ss, p.wait_polls)) {
            ok = false;
            break;
          }
          m_other = ss->rowmax[g ^ 1][to & 1][row];
        }
        if (!warp_wait_or_flag(&ss->s_full[g], ti & 1, ss, p.wait_polls)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        // the whole row of S into registers; S may then be overwritten by the group's next Q K^T
        uint32_t s[kBN];
        {
          const uint32_t base = tmem + lane_base + col_s;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            tmem_ld32(base + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
          tmem_wait_ld();
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&ss->s_empty[g]);

        const int64_t kv0 = (int64_t)j * kBN;
        const bool need_mask = (right_bounded && kv0 + kBN - 1 > q0 + shift + p.window_right) ||
                               (kv0 + kBN > p.Sk) || left_bounded;
        if (need_mask) { // visible columns of this tile for this row: [lo, hi]
          const int64_t hi64 = (right_bounded ? min(p.Sk - 1, qrow + shift + p.window_right) : p.Sk - 1) - kv0;
          const int64_t lo64 = (left_bounded ? qrow + shift - p.window_left : 0) - kv0;
          const int hi = (int)max((int64_t)-1, min((int64_t)kBN - 1, hi64));
          const int lo = (int)max((int64_t)0, min((int64_t)kBN, lo64));
#pragma unroll
          for (int c = 0; c < kBN; ++c)
            if (c > hi || c < lo)
              s[c] = 0xff800000u; // -inf
        }
        // row maximum: eight independent chains of 3-input max
        float mx8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e)
          mx8[e] = fmaxf(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1]));
#pragma unroll
        for (int c = 16; c < kBN; c += 16) {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            mx8[e] = fmax3(mx8[e], __uint_as_float(s[c + 2 * e]), __uint_as_float(s[c + 2 * e + 1]));
        }
        const float m_mine =
            fmax3(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])) * p.scale_log2;
        // publish this tile's maxima for the other group
        ss->rowmax[g][ti & 1][row] = m_mine;
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&ss->mx_ready[g][ti & 1]);
        float alpha, a_step;
        bool rescale = false;
        alpha = 1.f;
        if (j > 0) {
          ref_step(j - 1, m_other, ref, a_step); // the other group rescaled O for this step
          alpha = a_step;
        }
        rescale = ref_step(j, m_mine, ref, a_step); // this thread rescales O for this step
        alpha *= a_step;
        l *= alpha; // this group's partial row sum follows every move of the reference
        const float m_safe = (ref == -INFINITY) ? 0.f : ref;
        // probabilities: x = s * scale - m for two columns per packed FMA, 2^x on the MUFU unit,
        // four independent packed partial sums; the 16-bit P reuses the front of the row's registers
        const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2), negm2 = f2_pack(-m_safe, -m_safe);
        uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
        uint32_t(&packed)[kBN] = s;
#pragma unroll
        for (int c = 0; c < kBN; c += 2) {
          const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), scale2, negm2);
          float x0, x1;
          f2_unpack(x2, x0, x1);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
          sum2[(c >> 1) & 3] = f2_add(sum2[(c >> 1) & 3], f2_pack(p0, p1));
          packed[c >> 1] = pack2(p0, p1, kBF16);
        }
        {
          float a0, a1, b0, b1;
          f2_unpack(f2_add(sum2[0], sum2[1]), a0, a1);
          f2_unpack(f2_add(sum2[2], sum2[3]), b0, b1);
          l += (a0 + a1) + (b0 + b1);
        }

        // P V of the tile before (the other group's) has completed: then so has this group's
        // previous one, which read the P columns, and O holds every tile up to j - 1
        if (j > 0) {
          const uint32_t to = tc[1] + ((j - 1) >> 1);
          if (!warp_wait_or_flag(&ss->pv_done[g ^ 1], to & 1, ss, p.wait_polls)) {
            ok = false;
            break;
          }
        }
        tc_fence_after_sync();
        // P row -> tensor memory: 128 keys = 64 columns of two 16-bit values
        tmem_st32(tmem + lane_base + col_p, *reinterpret_cast<uint32_t(*)[32]>(&packed[0]));
        tmem_st32(tmem + lane_base + col_p + 32, *reinterpret_cast<uint32_t(*)[32]>(&packed[32]));
        if (rescale) {
          const uint32_t base = tmem + lane_base + kColO;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32(base + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int q = 0; q < 32; ++q)
              r[q] = __float_as_uint(__uint_as_float(r[q]) * a_step);
            tmem_st32(base + c * 32, r);
          }
        }
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0 && !p.debug_skip_arrive)
          mbar_arrive(&ss->p_full[g]);
      }

      // ---- epilogue of the query tile: O / l -> 16 bit -> shared -> TMA store; LSE
      // the last P V: products complete in issue order, so it is the only one to wait for
      if (ok && n > 0) {
        const int gl = (n - 1) & 1; // group of the last key tile
        const uint32_t tl = (gl == g ? tc[0] : tc[1]) + ((n - 1) >> 1);
        ok = warp_wait_or_flag(&ss->pv_done[gl], tl & 1, ss, p.wait_polls);
      }
      tc[0] += n_mine;
      tc[1] += n_other;
      if (warp == 4 && lane == 0)
        bulk_wait_read<0>(); // the previous query tile's store has read the staging buffer
      ss->xch[g][row] = make_float2(ref, l);
      tc_fence_before_sync();
      const bool give_up = named_bar_or_n<256>(!ok); // both groups
      tc_fence_after_sync();
      // the two threads of a row may be one step apart: the later reference is the one O is scaled with
      const float2 other = ss->xch[g ^ 1][row];
      const float m_tot = fmaxf(ref, other.x);
      const float a_mine = (ref == -INFINITY) ? 0.f : fast_exp2(ref - m_tot);
      const float a_other = (other.x == -INFINITY) ? 0.f : fast_exp2(other.x - m_tot);
      const float l_tot = l * a_mine + other.y * a_other;
      const float inv_l = (l_tot > 0.f) ? 1.f / l_tot : 0.f;
      const bool have = !give_up && n > 0;
      // this thread finishes head-dim columns [64 g, 64 g + 64) of its row
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        if (have) {
          tmem_ld32(tmem + lane_base + kColO + g * 64 + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int q = 0; q < 32; ++q)
            r[q] = 0u;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) { // 8 columns = one 16-byte chunk
          uint4 v;
          v.x = pack2(__uint_as_float(r[q * 8 + 0]) * inv_l, __uint_as_float(r[q * 8 + 1]) * inv_l, kBF16);
          v.y = pack2(__uint_as_float(r[q * 8 + 2]) * inv_l, __uint_as_float(r[q * 8 + 3]) * inv_l, kBF16);
          v.z = pack2(__uint_as_float(r[q * 8 + 4]) * inv_l, __uint_as_float(r[q * 8 + 5]) * inv_l, kBF16);
          v.w = pack2(__uint_as_float(r[q * 8 + 6]) * inv_l, __uint_as_float(r[q * 8 + 7]) * inv_l, kBF16);
          const int chunk = c * 4 + q;
          *reinterpret_cast<uint4 *>(sO + g * kHalfTile + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
        }
      }
      fence_proxy_async_smem();
      if (g == 0 && qrow < p.Sq)
        p.lse[((int64_t)w.b * p.H + w.h) * p.Sq + qrow] =
            (l_tot > 0.f) ? (m_tot + log2f(l_tot)) * 0.6931471805599453f : INFINITY;
      // both groups: O is staged and read out of tensor memory, the next query tile may overwrite it
      tc_fence_before_sync();
      asm volatile("bar.sync 2, 256;" ::: "memory");
      tc_fence_after_sync();
      if (warp == 4 && lane == 0 && !give_up) {
        tma_store_4d(&o_map, sO, 0, w.h, (int)q0, w.b);
        if (p.d > 64) // a store that would start past the end of the head is left out
          tma_store_4d(&o_map, sO + kHalfTile, 64, w.h, (int)q0, w.b);
        bulk_commit();
      }
      if (give_up)
        break;
    }
    if (warp == 4 && lane == 0)
      bulk_wait_read<0>(); // shared memory must outlive the last store's reads
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ss->failed) {
    g_attn_status = 2;
    if (p.status)
      *p.status = 2;
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

int make_qkv_map(CUtensorMap *map, bool bf16, const void *base, int64_t d, int64_t heads, int64_t seq,
                 int64_t batch, int64_t head_stride, int64_t row_stride, int64_t batch_stride,
                 uint32_t box_rows = 128) {
  const uint64_t dims[4] = {(uint64_t)d, (uint64_t)heads, (uint64_t)seq, (uint64_t)batch};
  const uint64_t strides[3] = {(uint64_t)head_stride * 2, (uint64_t)row_stride * 2, (uint64_t)batch_stride * 2};
  const uint32_t box[4] = {64, 1, box_rows, 1};
  return make_tensor_map(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                         const_cast<void *>(base), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}


// =============================================================================
// backward
// =============================================================================
// Three kernels, no atomics, so the result is a function of the inputs alone
// (the reference adds dQ partials with atomicAdd, flash_bwd_kernel.h:663):
//   1. bwd_dot_do_o_kernel   D[b,h,i] = sum_d dO * O  (f32)
//   2. bwd_dkdv_kernel       one block per 128 keys; walks over the query tiles
//                            that see them; dK, dV accumulate in tensor memory
//   3. bwd_dq_kernel         one block per 128 queries; walks over the key tiles;
//                            dQ accumulates in tensor memory
// Kernels 2 and 3 both recompute P = exp2(S * scale * log2e - LSE * log2e) and
// dS = P o (dP - D) from the saved LSE, as the reference does
// (flash_bwd_kernel.h:472-580); P and dS are rounded to the storage type before
// the following products.  Kernel 2 works on transposed tiles (S^T = K Q^T), so
// that the thread that owns a key row writes rows of P^T and dS^T, which are the
// K-major A operands of dV += P^T dO and dK += dS^T Q.

// Tensor-memory columns.  S / dP tiles are 128 x 64 (64 streamed rows per step) and
// double-buffered, one buffer per elementwise group; P and dS (16 bit) overwrite the
// front of the S / dP buffer they were computed from.
//   dK/dV kernel: S^T 0,64 | dP^T 128,192 | dV 256 | dK 384
//   dQ kernel:    Q 0 | dO 64 (A operands) | S 128,192 | dP 256,320 | dQ 384
constexpr int kBwdBN = 64;       // streamed rows per step
constexpr int kBwdStages = 4;    // ring depth of the streamed (row tile, row tile) pairs
constexpr uint32_t kStrTileBytes = kBwdBN * kD * 2; // 16 KiB: [2 column blocks][64 rows][128 B]
constexpr uint32_t kStrHalf = kStrTileBytes / 2;

struct BwdParams {
  const float *lse;   // [B, H, Sq]
  const float *dsum;  // [B, H, Sq_rounded]
  int64_t H, Hk, Sq, Sk, Sq_rounded;
  float scale, scale_log2;
  int64_t window_left, window_right;
  uint32_t wait_polls;
  int debug_skip_arrive;
  int d; // head dim, <= 128
};

struct BwdShared {
  uint64_t bar_resident;                          // the block's own tiles (K,V or Q,dO) in shared memory
  uint64_t res_ready;                             // ... and, dQ kernel, copied to tensor memory
  uint64_t full[kBwdStages], empty[kBwdStages];   // streamed tile pairs
  uint64_t sdp_full[2];                           // S / dP of a group's tile are in tensor memory
  uint64_t pds_full[2];                           // the group has written P / dS
  uint64_t all_done;                              // every MMA of the block has completed
  uint32_t tmem_base;
  int failed;
  // dK/dV kernel: -lse * log2e and -dsum of the streamed queries [group][parity][row], negated
  // so that pairs of them are addends of packed FMAs / ADDs (read four at a time: 16-byte aligned)
  alignas(16) float neg_lse2[2][2][kBwdBN];
  alignas(16) float neg_dsum[2][2][kBwdBN];
};

__device__ __forceinline__ bool bwd_wait(uint64_t *bar, uint32_t parity, BwdShared *ss, uint32_t polls) {
  if (mbar_wait(bar, parity, polls))
    return true;
  ss->failed = 1;
  return false;
}
__device__ __forceinline__ bool bwd_warp_wait(uint64_t *bar, uint32_t parity, BwdShared *ss, uint32_t polls) {
  const bool ok = __all_sync(0xffffffffu, mbar_wait(bar, parity, polls));
  if (!ok)
    ss->failed = 1;
  return ok;
}

// 16-byte chunk `chunk16` (0..15: 8 columns each) of row `row` of a 128 x 128 16-bit
// tile stored as [2 column blocks][128 rows][128 B] with the 128-byte swizzle
__device__ __forceinline__ void store_tile_chunk(unsigned char *tile, int row, int chunk16, uint4 v) {
  const int blk = chunk16 >> 3, chunk = chunk16 & 7;
  *reinterpret_cast<uint4 *>(tile + blk * kHalfTile + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
}
__device__ __forceinline__ uint4 load_tile_chunk(const unsigned char *tile, int row, int chunk16) {
  const int blk = chunk16 >> 3, chunk = chunk16 & 7;
  return *reinterpret_cast<const uint4 *>(tile + blk * kHalfTile + row * 128 + ((chunk ^ (row & 7)) << 4));
}

__global__ void __launch_bounds__(256)
    bwd_dot_do_o_kernel(const void *__restrict__ dout, const void *__restrict__ out, float *__restrict__ dsum,
                        int64_t B, int64_t H, int64_t Sq, int64_t Sq_rounded, int64_t o_batch_stride,
                        int64_t o_row_stride, int64_t o_head_stride, int d, bool bf16) {
  // 16 threads per (b, h, row): 8 elements each of the row of d <= 128 elements
  const int64_t gid = (int64_t)blockIdx.x * 16 + (threadIdx.x >> 4);
  const int sub = threadIdx.x & 15;
  const int64_t total = B * H * Sq;
  float acc = 0.f;
  if (gid < total && sub * 8 < d) {
    const int64_t row = gid % Sq, h = (gid / Sq) % H, b = gid / (Sq * H);
    const int64_t off = b * o_batch_stride + row * o_row_stride + h * o_head_stride + sub * 8;
    const uint4 a = ld_nc_v4(static_cast<const uint16_t *>(dout) + off);
    const uint4 c = ld_nc_v4(static_cast<const uint16_t *>(out) + off);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 x, y;
      if (bf16) {
        x = make_float2(__uint_as_float(aw[k] << 16), __uint_as_float(aw[k] & 0xffff0000u));
        y = make_float2(__uint_as_float(cw[k] << 16), __uint_as_float(cw[k] & 0xffff0000u));
      } else {
        x = __half22float2(*reinterpret_cast<const __half2 *>(&aw[k]));
        y = __half22float2(*reinterpret_cast<const __half2 *>(&cw[k]));
      }
      acc = fmaf(x.x, y.x, acc);
      acc = fmaf(x.y, y.y, acc);
    }
  }
  for (int off = 8; off > 0; off >>= 1)
    acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (gid < total && sub == 0) {
    const int64_t row = gid % Sq, bh = gid / Sq;
    dsum[bh * Sq_rounded + row] = acc;
  }
}

// kDKDV = true : block owns keys [own0, own0+128) (rows of the transposed tiles) and streams
//                (Q, dO) tiles of 64 queries:  S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q
// kDKDV = false: block owns queries [own0, own0+128) and streams (K, V) tiles of 64 keys:
//                S = Q K^T, dP = dO V^T, dQ += dS K
// Warp roles: 0 TMA producer, 1 MMA issuer (all lanes run the loop, one elected lane issues),
// 4..7 and 8..11 two elementwise groups that take the streamed tiles alternately, so that the
// tensor core works on one group's products while the other group computes P and dS.
// P^T / dS^T (dS) go back to tensor memory and are the A operands of the accumulating
// products; in the dQ kernel Q and dO are A operands from tensor memory as well.
template <bool kBF16, bool kDKDV>
__global__ void __launch_bounds__(kThreads, 1)
    flash_bwd_kernel(const __grid_constant__ CUtensorMap res0_map, // K (kDKDV) or Q, 128-row boxes
                     const __grid_constant__ CUtensorMap res1_map, // V (kDKDV) or dO
                     const __grid_constant__ CUtensorMap str0_map, // Q (kDKDV) or K, 64-row boxes
                     const __grid_constant__ CUtensorMap str1_map, // dO (kDKDV) or V
                     const __grid_constant__ CUtensorMap out0_map, // dK (kDKDV) or dQ
                     const __grid_constant__ CUtensorMap out1_map, // dV (kDKDV), unused otherwise
                     const BwdParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *smem =
      reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *sRes0 = smem;                     // K (kDKDV) / Q; at the end dK / dQ on its way out
  unsigned char *sRes1 = sRes0 + kTileBytes;       // V (kDKDV) / dO; at the end dV
  unsigned char *sStr = sRes1 + kTileBytes;        // [stage][2 tiles of 64 rows]
  BwdShared *ss = reinterpret_cast<BwdShared *>(sStr + kBwdStages * 2 * kStrTileBytes);

  constexpr uint32_t kColA0 = 0, kColA1 = 64;                    // dQ kernel: Q, dO
  constexpr uint32_t kColS = kDKDV ? 0 : 128;                    // + 64 * group
  constexpr uint32_t kColDP = kDKDV ? 128 : 256;                 // + 64 * group
  constexpr uint32_t kColAcc0 = kDKDV ? 256 : 384, kColAcc1 = 384; // dV | dK, or dQ

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31; // warp: known uniform
  const int b = blockIdx.z;
  const int64_t shift = p.Sk - p.Sq;
  const bool right_bounded = p.window_right >= 0;
  const bool left_bounded = p.window_left >= 0;
  const int group = (int)(p.H / p.Hk);
  const int n_q_tiles = (int)((p.Sq + kBM - 1) / kBM);

  // the tile this block owns, and the range of streamed 64-row tiles [t_begin, t_end)
  int own_tile, head, t_begin, t_end, heads_in_loop;
  if (kDKDV) {
    own_tile = blockIdx.x;
    head = blockIdx.y; // key/value head
    heads_in_loop = group;
    t_begin = 0;
    t_end = (int)((p.Sq + kBwdBN - 1) / kBwdBN);
    if (right_bounded) { // queries that can see key own0: q >= own0 - shift - window_right
      const int64_t first_q = (int64_t)own_tile * 128 - shift - p.window_right;
      t_begin = first_q <= 0 ? 0 : (int)min((int64_t)t_end, first_q / kBwdBN);
    }
  } else {
    own_tile = n_q_tiles - 1 - (int)blockIdx.x;
    head = blockIdx.y; // query head
    heads_in_loop = 1;
    t_begin = 0;
    t_end = (int)((p.Sk + kBwdBN - 1) / kBwdBN);
    if (right_bounded) {
      const int64_t last_visible = (int64_t)own_tile * kBM + kBM - 1 + shift + p.window_right;
      t_end = last_visible < 0 ? 0 : (int)min((int64_t)t_end, last_visible / kBwdBN + 1);
    }
  }
  const int tiles_per_head = max(0, t_end - t_begin);
  const int T = tiles_per_head * heads_in_loop;
  const int64_t own0 = (int64_t)own_tile * 128;

  if (threadIdx.x == 0) {
    mbar_init(&ss->bar_resident, 1);
    mbar_init(&ss->res_ready, 8);
    for (int s = 0; s < kBwdStages; ++s) {
      mbar_init(&ss->full[s], 1);
      mbar_init(&ss->empty[s], 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&ss->sdp_full[g], 1);
      mbar_init(&ss->pds_full[g], 4);
    }
    mbar_init(&ss->all_done, 1);
    ss->failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ss->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = ss->tmem_base;

  // streamed iteration -> (query head, streamed tile index)
  auto iter_head = [&](int it) { return kDKDV ? head * group + it / tiles_per_head : head; };
  auto iter_tile = [&](int it) { return t_begin + (kDKDV ? it % tiles_per_head : it); };
  const int kv_head = kDKDV ? head : head / group;

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0 && T > 0) {
      prefetch_tensormap(&res0_map);
      prefetch_tensormap(&res1_map);
      prefetch_tensormap(&str0_map);
      prefetch_tensormap(&str1_map);
      const int res_head = kDKDV ? kv_head : head;
      mbar_arrive_expect_tx(&ss->bar_resident, 2 * kTileBytes);
      tma_load_4d(sRes0, &res0_map, 0, res_head, (int)own0, b, &ss->bar_resident);
      tma_load_4d(sRes0 + kHalfTile, &res0_map, 64, res_head, (int)own0, b, &ss->bar_resident);
      tma_load_4d(sRes1, &res1_map, 0, res_head, (int)own0, b, &ss->bar_resident);
      tma_load_4d(sRes1 + kHalfTile, &res1_map, 64, res_head, (int)own0, b, &ss->bar_resident);
      for (int it = 0; it < T; ++it) {
        const int st = it % kBwdStages;
        if (!bwd_wait(&ss->empty[st], (uint32_t)(((it / kBwdStages) & 1) ^ 1), ss, p.wait_polls))
          break;
        mbar_arrive_expect_tx(&ss->full[st], 2 * kStrTileBytes);
        unsigned char *t0 = sStr + st * 2 * kStrTileBytes, *t1 = t0 + kStrTileBytes;
        const int row0 = iter_tile(it) * kBwdBN;
        const int hh = kDKDV ? iter_head(it) : kv_head;
        tma_load_4d(t0, &str0_map, 0, hh, row0, b, &ss->full[st]);
        tma_load_4d(t0 + kStrHalf, &str0_map, 64, hh, row0, b, &ss->full[st]);
        tma_load_4d(t1, &str1_map, 0, hh, row0, b, &ss->full[st]);
        tma_load_4d(t1 + kStrHalf, &str1_map, 64, hh, row0, b, &ss->full[st]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (T > 0) {
      constexpr uint32_t idesc_sdp = umma_idesc_f16(kBF16, 128, kBwdBN, false, false); // B K-major, N = 64
      constexpr uint32_t idesc_acc = umma_idesc_f16(kBF16, 128, 128, false, true);     // B rows = K index
      const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
      const uint32_t res0 = smem_addr(sRes0), res1 = smem_addr(sRes1), str = smem_addr(sStr);
      // S (S^T) and dP (dP^T) of streamed tile `it` into the buffers of group it & 1:
      // contraction over the 128 head dims, 8 steps of 16
      auto issue_sdp = [&](int it) {
        const int st = it % kBwdStages, g = it & 1;
        const uint32_t t0 = str + st * 2 * kStrTileBytes, t1 = t0 + kStrTileBytes;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t a_off = (kk >> 2) * kHalfTile + (kk & 3) * 32;
          const uint32_t b_off = (kk >> 2) * kStrHalf + (kk & 3) * 32;
          const uint64_t b0 = umma_smem_desc(t0 + b_off, 16, 1024), b1 = umma_smem_desc(t1 + b_off, 16, 1024);
          if (kDKDV) {
            const uint64_t a0 = umma_smem_desc(res0 + a_off, 16, 1024), a1 = umma_smem_desc(res1 + a_off, 16, 1024);
            if (elect_one()) {
              umma_ss(tm + kColS + g * 64, a0, b0, idesc_sdp, kk != 0);
              umma_ss(tm + kColDP + g * 64, a1, b1, idesc_sdp, kk != 0);
            }
          } else if (elect_one()) {
            umma_ts(tm + kColS + g * 64, tm + kColA0 + kk * 8, b0, idesc_sdp, kk != 0);
            umma_ts(tm + kColDP + g * 64, tm + kColA1 + kk * 8, b1, idesc_sdp, kk != 0);
          }
        }
        if (elect_one())
          umma_commit(&ss->sdp_full[g]);
      };
      bool ok = kDKDV ? bwd_warp_wait(&ss->bar_resident, 0, ss, p.wait_polls) : bwd_warp_wait(&ss->res_ready, 0, ss, p.wait_polls);
      for (int it = 0; ok && it < 2 && it < T; ++it) {
        ok = bwd_warp_wait(&ss->full[it % kBwdStages], 0, ss, p.wait_polls);
        if (ok) {
          tc_fence_after_sync();
          issue_sdp(it);
        }
      }
      for (int it = 0; ok && it < T; ++it) {
        const int st = it % kBwdStages, g = it & 1;
        const uint32_t t0 = str + st * 2 * kStrTileBytes, t1 = t0 + kStrTileBytes;
        // the streamed tile after next arrived long ago (the ring is four deep): look at its
        // barrier while the group still computes, not between the two batches of products
        if (it + 2 < T)
          ok = bwd_warp_wait(&ss->full[(it + 2) % kBwdStages], (uint32_t)(((it + 2) / kBwdStages) & 1), ss, p.wait_polls);
        ok = ok && bwd_warp_wait(&ss->pds_full[g], (uint32_t)((it >> 1) & 1), ss, p.wait_polls);
        if (!ok)
          break;
        tc_fence_after_sync();
        // contraction over the 64 streamed rows: 4 steps of 16; B = streamed tile, rows = K index
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t b0 = umma_smem_desc(t0 + ks * 16 * 128, kStrHalf, 1024);
          const uint64_t b1 = umma_smem_desc(t1 + ks * 16 * 128, kStrHalf, 1024);
          if (elect_one()) {
            if (kDKDV) {
              // dV += P^T dO ; dK += dS^T Q
              umma_ts(tm + kColAcc0, tm + kColS + g * 64 + ks * 8, b1, idesc_acc, (it | ks) != 0);
              umma_ts(tm + kColAcc1, tm + kColDP + g * 64 + ks * 8, b0, idesc_acc, (it | ks) != 0);
            } else {
              // dQ += dS K
              umma_ts(tm + kColAcc0, tm + kColDP + g * 64 + ks * 8, b0, idesc_acc, (it | ks) != 0);
            }
          }
        }
        if (elect_one())
          umma_commit(&ss->empty[st]);
        // the group's buffers are free for its next tile as soon as the products above have
        // read P / dS: the tensor core runs what this lane issues in order
        if (it + 2 < T)
          issue_sdp(it + 2);
      }
      if (ok && elect_one())
        umma_commit(&ss->all_done);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------- elementwise groups
    const int g = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;       // owned-side row: a key (kDKDV) or a query
    const int64_t own_idx = own0 + row;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t col_s = kColS + g * 64, col_dp = kColDP + g * 64;
    const float kLog2e = 1.4426950408889634f;
    float my_lse2 = 0.f, my_dsum = 0.f;
    if (!kDKDV && own_idx < p.Sq) {
      my_lse2 = p.lse[((int64_t)b * p.H + head) * p.Sq + own_idx] * kLog2e;
      my_dsum = p.dsum[((int64_t)b * p.H + head) * p.Sq_rounded + own_idx];
    }
    bool ok = T > 0;
    if (!kDKDV && T > 0) {
      // own Q (group 0) / dO (group 1) row -> tensor memory, the A operands of S and dP
      ok = bwd_wait(&ss->bar_resident, 0, ss, p.wait_polls);
      const unsigned char *src = g == 0 ? sRes0 : sRes1;
#pragma unroll
      for (int db = 0; db < 2; ++db) {
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 v = load_tile_chunk(src, row, db * 8 + c);
          r[c * 4 + 0] = v.x;
          r[c * 4 + 1] = v.y;
          r[c * 4 + 2] = v.z;
          r[c * 4 + 3] = v.w;
        }
        tmem_st32(tmem + lane_base + (g == 0 ? kColA0 : kColA1) + db * 32, r);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0 && ok)
        mbar_arrive(&ss->res_ready);
    }
    const int n_mine = (T + 1 - g) >> 1;
    // dK/dV: statistics of the 64 streamed queries of a tile, one query per thread of the group's
    // first two warps.  They are fetched one tile ahead, so that the two dependent global loads
    // are not on the path between two tiles.
    const int stat_t = (warp & 3) * 32 + lane;
    auto load_stats = [&](int i, float &l2, float &dd) {
      l2 = INFINITY, dd = 0.f; // rows past the end: P = exp2(-inf) = 0
      if (kDKDV && stat_t < kBwdBN && i < n_mine) {
        const int it = 2 * i + g;
        const int64_t qi = (int64_t)iter_tile(it) * kBwdBN + stat_t;
        const int qh = iter_head(it);
        if (qi < p.Sq) {
          l2 = p.lse[((int64_t)b * p.H + qh) * p.Sq + qi] * kLog2e;
          dd = p.dsum[((int64_t)b * p.H + qh) * p.Sq_rounded + qi];
        }
      }
    };
    float next_l2, next_dd;
    load_stats(0, next_l2, next_dd);
    const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
    for (int i = 0; ok && i < n_mine; ++i) {
      const int it = 2 * i + g;
      const int64_t str0 = (int64_t)iter_tile(it) * kBwdBN;
      if (kDKDV) {
        if (stat_t < kBwdBN) {
          ss->neg_lse2[g][i & 1][stat_t] = -next_l2;
          ss->neg_dsum[g][i & 1][stat_t] = -next_dd;
        }
        load_stats(i + 1, next_l2, next_dd); // in flight during this tile
      }
      const bool waited = bwd_wait(&ss->sdp_full[g], (uint32_t)(i & 1), ss, p.wait_polls);
      // one barrier per tile and group: publishes the statistics and makes giving up unanimous
      if (named_bar_or_id(1 + g, !waited)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // visibility of (query, key): key <= query + shift + wr, key >= query + shift - wl, both in
      // range.  For this thread's row that is a column interval [lo, hi] of the tile; most tiles
      // are fully visible and skip the masking altogether.
      int lo, hi;
      {
        int64_t lo64, hi64;
        if (kDKDV) { // row = key own_idx, columns = queries str0 + c
          hi64 = (left_bounded ? min(p.Sq - 1, own_idx - shift + p.window_left) : p.Sq - 1) - str0;
          lo64 = (right_bounded ? own_idx - shift - p.window_right : 0) - str0;
          if (own_idx >= p.Sk)
            hi64 = -1;
        } else { // row = query own_idx, columns = keys str0 + c
          hi64 = (right_bounded ? min(p.Sk - 1, own_idx + shift + p.window_right) : p.Sk - 1) - str0;
          lo64 = (left_bounded ? own_idx + shift - p.window_left : 0) - str0;
          if (own_idx >= p.Sq)
            hi64 = -1;
        }
        hi = (int)max((int64_t)-1, min((int64_t)kBwdBN - 1, hi64));
        lo = (int)max((int64_t)0, min((int64_t)kBwdBN, lo64));
      }
      const bool need_mask = __any_sync(0xffffffffu, lo > 0 || hi < kBwdBN - 1);
      uint32_t pp[32], dd[32]; // the row's 64 values of P and dS, 16 bit
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sr[32], dr[32];
        tmem_ld32(tmem + lane_base + col_s + c * 32, sr);
        tmem_ld32(tmem + lane_base + col_dp + c * 32, dr);
        tmem_wait_ld();
        if (need_mask) {
#pragma unroll
          for (int q = 0; q < 32; ++q)
            if (c * 32 + q > hi || c * 32 + q < lo)
              sr[q] = 0xff800000u; // -inf: P = 0, dS = 0
        }
        // P = 2^(S * scale - lse), dS = P * (dP - dsum): four columns per step, two per packed op
#pragma unroll
        for (int q = 0; q < 32; q += 4) {
          uint64_t nl[2], nd[2];
          if (kDKDV) {
            const float4 l4 = *reinterpret_cast<const float4 *>(&ss->neg_lse2[g][i & 1][c * 32 + q]);
            const float4 d4 = *reinterpret_cast<const float4 *>(&ss->neg_dsum[g][i & 1][c * 32 + q]);
            nl[0] = f2_pack(l4.x, l4.y), nl[1] = f2_pack(l4.z, l4.w);
            nd[0] = f2_pack(d4.x, d4.y), nd[1] = f2_pack(d4.z, d4.w);
          } else {
            nl[0] = nl[1] = f2_pack(-my_lse2, -my_lse2);
            nd[0] = nd[1] = f2_pack(-my_dsum, -my_dsum);
          }
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int k = q + 2 * e;
            const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(sr[k]), __uint_as_float(sr[k + 1])), scale2, nl[e]);
            float x0, x1;
            f2_unpack(x2, x0, x1);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            const uint64_t t2 = f2_add(f2_pack(__uint_as_float(dr[k]), __uint_as_float(dr[k + 1])), nd[e]);
            float d0, d1;
            f2_unpack(f2_mul(f2_pack(p0, p1), t2), d0, d1);
            pp[c * 16 + k / 2] = pack2(p0, p1, kBF16);
            dd[c * 16 + k / 2] = pack2(d0, d1, kBF16);
          }
        }
      }
      // both tiles are in registers: P^T / dS^T (dS) take the place of the values they came from
      if (kDKDV)
        tmem_st32(tmem + lane_base + col_s, pp);
      tmem_st32(tmem + lane_base + col_dp, dd);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0 && !p.debug_skip_arrive)
        mbar_arrive(&ss->pds_full[g]);
    }

    // ---- epilogue: accumulators -> 16 bit -> shared -> TMA store
    if (ok && T > 0)
      ok = bwd_wait(&ss->all_done, 0, ss, p.wait_polls);
    tc_fence_after_sync();
    const bool have = ok && T > 0;
    // kDKDV: group 0 takes dV (unscaled) -> V's tile, group 1 dK (* scale) -> K's tile;
    // else both groups take half of dQ's columns each (* scale) -> Q's tile
    const uint32_t col0 = kDKDV ? (g == 0 ? kColAcc0 : kColAcc1) : kColAcc0 + g * 64;
    unsigned char *stage = (kDKDV && g == 0) ? sRes1 : sRes0;
    const float mul = (kDKDV && g == 0) ? 1.f : p.scale;
    constexpr int kChunks = kDKDV ? 4 : 2;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      uint32_t r[32];
      if (have) {
        tmem_ld32(tmem + lane_base + col0 + c * 32, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int q = 0; q < 32; ++q)
          r[q] = 0u;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 v;
        v.x = pack2(__uint_as_float(r[q * 8 + 0]) * mul, __uint_as_float(r[q * 8 + 1]) * mul, kBF16);
        v.y = pack2(__uint_as_float(r[q * 8 + 2]) * mul, __uint_as_float(r[q * 8 + 3]) * mul, kBF16);
        v.z = pack2(__uint_as_float(r[q * 8 + 4]) * mul, __uint_as_float(r[q * 8 + 5]) * mul, kBF16);
        v.w = pack2(__uint_as_float(r[q * 8 + 6]) * mul, __uint_as_float(r[q * 8 + 7]) * mul, kBF16);
        store_tile_chunk(stage, row, (kDKDV ? 0 : g * 8) + c * 4 + q, v);
      }
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync 3, 256;" ::: "memory"); // both groups
    if (warp == 4 && lane == 0 && ss->failed == 0) {
      if (kDKDV) {
        tma_store_4d(&out1_map, sRes1, 0, head, (int)own0, b);
        if (p.d > 64)
          tma_store_4d(&out1_map, sRes1 + kHalfTile, 64, head, (int)own0, b);
      }
      tma_store_4d(&out0_map, sRes0, 0, head, (int)own0, b);
      if (p.d > 64)
        tma_store_4d(&out0_map, sRes0 + kHalfTile, 64, head, (int)own0, b);
      bulk_commit();
      bulk_wait_all<0>();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ss->failed)
    g_attn_status = 3; // dq / dk / dv of this block were not stored
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <bool kBF16, bool kDKDV>
int launch_bwd(const CUtensorMap &res0, const CUtensorMap &res1, const CUtensorMap &str0, const CUtensorMap &str1,
               const CUtensorMap &out0, const CUtensorMap &out1, const BwdParams &p, dim3 grid,
               cudaStream_t stream) {
  const size_t smem = (size_t)2 * kTileBytes + (size_t)kBwdStages * 2 * kStrTileBytes + sizeof(BwdShared) + 1024;
  // the attribute belongs to the current device's context: set on every call (a host-side table write)
  if (int rc = check_cuda(cudaFuncSetAttribute(flash_bwd_kernel<kBF16, kDKDV>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)))
    return rc;
  flash_bwd_kernel<kBF16, kDKDV><<<grid, kThreads, smem, stream>>>(res0, res1, str0, str1, out0, out1, p);
  return check_launch();
}

} // namespace
} // namespace b200

using namespace b200;

extern "C" int b200_flash_attn_take_status(int *status) {
  int v = 0;
  if (int rc = check_cuda(cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int))))
    return rc;
  if (v != 0) {
    const int zero = 0;
    if (int rc = check_cuda(cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int))))
      return rc;
  }
  if (status)
    *status = v;
  return B200_OK;
}

extern "C" void b200_flash_attn_debug(int skip_arrive, unsigned wait_polls) {
  g_debug_skip_arrive = skip_arrive;
  g_wait_polls = wait_polls ? wait_polls : 100000u;
}

extern "C" int b200_flash_attn_fwd(int dtype, const void *q, const void *k, const void *v, void *out,
                                   float *softmax_lse, const b200_flash_attn_params *pp, cudaStream_t stream) {
  if (!pp || !q || !k || !v || !out || !softmax_lse)
    return B200_ERR_INVALID_ARG;
  const b200_flash_attn_params &a = *pp;
  if (dtype != B200_F16 && dtype != B200_BF16)
    return B200_ERR_UNSUPPORTED;
  if (a.d <= 0 || a.d > kD || a.d % 8 != 0 || a.p_dropout != 0.f || a.h_k <= 0 || a.h % a.h_k != 0 || a.b <= 0 || a.seqlen_q <= 0 ||
      a.seqlen_k <= 0)
    return B200_ERR_UNSUPPORTED; // head dim a multiple of 8 up to 128, no dropout
  const int64_t strides[] = {a.q_batch_stride, a.k_batch_stride, a.v_batch_stride, a.o_batch_stride,
                             a.q_row_stride,   a.k_row_stride,   a.v_row_stride,   a.o_row_stride,
                             a.q_head_stride,  a.k_head_stride,  a.v_head_stride,  a.o_head_stride};
  for (int64_t s : strides)
    if (s <= 0 || s % 8 != 0)
      return B200_ERR_ALIGNMENT; // TMA needs 16-byte multiples
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out))
    return B200_ERR_ALIGNMENT;
  const bool bf16 = dtype == B200_BF16;
  CUtensorMap q_map, k_map, v_map, o_map;
  if (int rc = make_qkv_map(&q_map, bf16, q, a.d, a.h, a.seqlen_q, a.b, a.q_head_stride, a.q_row_stride, a.q_batch_stride))
    return rc;
  if (int rc = make_qkv_map(&k_map, bf16, k, a.d, a.h_k, a.seqlen_k, a.b, a.k_head_stride, a.k_row_stride, a.k_batch_stride))
    return rc;
  if (int rc = make_qkv_map(&v_map, bf16, v, a.d, a.h_k, a.seqlen_k, a.b, a.v_head_stride, a.v_row_stride, a.v_batch_stride))
    return rc;
  if (int rc = make_qkv_map(&o_map, bf16, out, a.d, a.h, a.seqlen_q, a.b, a.o_head_stride, a.o_row_stride, a.o_batch_stride))
    return rc;
  FwdParams p;
  p.lse = softmax_lse;
  p.status = nullptr;
  p.wait_polls = g_wait_polls;
  p.debug_skip_arrive = g_debug_skip_arrive;
  p.d = (int)a.d;
  p.H = a.h;
  p.Hk = a.h_k;
  p.Sq = a.seqlen_q;
  p.Sk = a.seqlen_k;
  p.scale_log2 = a.softmax_scale * 1.4426950408889634f;
  p.window_left = a.window_size_left;
  p.window_right = a.window_size_right;
  p.n_q_tiles = (int)((a.seqlen_q + kBM - 1) / kBM);
  p.pairs = (p.n_q_tiles + 1) / 2;
  p.total_items = (int64_t)p.pairs * a.h * a.b;
  const size_t smem = (size_t)(2 + kFwdKStages + kFwdVStages) * kTileBytes + sizeof(SharedStorage) + 1024;
  { // the attribute belongs to the current device's context: set on every call (a host-side table write)
    cudaError_t e = bf16 ? cudaFuncSetAttribute(flash_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                         : cudaFuncSetAttribute(flash_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (int rc = check_cuda(e))
      return rc;
  }
  const dim3 grid((unsigned)(p.total_items < kNumSMs ? p.total_items : kNumSMs)); // persistent blocks, one per SM
  if (bf16)
    flash_fwd_kernel<true><<<grid, kThreads, smem, stream>>>(q_map, k_map, v_map, o_map, p);
  else
    flash_fwd_kernel<false><<<grid, kThreads, smem, stream>>>(q_map, k_map, v_map, o_map, p);
  return check_launch();
}

extern "C" int b200_flash_attn_bwd(int dtype, const void *dout, const void *q, const void *k, const void *v,
                                   const void *out, const float *softmax_lse, void *dq, void *dk, void *dv,
                                   float *d_softmax_sum, float *dq_accum, const b200_flash_attn_params *pp,
                                   cudaStream_t stream) {
  (void)dq_accum; // the reference's f32 dQ accumulator: not needed, dQ has its own pass
  if (!pp || !dout || !q || !k || !v || !out || !softmax_lse || !dq || !dk || !dv || !d_softmax_sum)
    return B200_ERR_INVALID_ARG;
  const b200_flash_attn_params &a = *pp;
  if (dtype != B200_F16 && dtype != B200_BF16)
    return B200_ERR_UNSUPPORTED;
  if (a.d <= 0 || a.d > kD || a.d % 8 != 0 || a.p_dropout != 0.f || a.h_k <= 0 || a.h % a.h_k != 0 || a.b <= 0 || a.seqlen_q <= 0 ||
      a.seqlen_k <= 0 || a.seqlen_q_rounded < a.seqlen_q)
    return B200_ERR_UNSUPPORTED;
  const int64_t strides[] = {a.q_batch_stride, a.k_batch_stride, a.v_batch_stride, a.o_batch_stride,
                             a.q_row_stride,   a.k_row_stride,   a.v_row_stride,   a.o_row_stride,
                             a.q_head_stride,  a.k_head_stride,  a.v_head_stride,  a.o_head_stride};
  for (int64_t s : strides)
    if (s <= 0 || s % 8 != 0)
      return B200_ERR_ALIGNMENT;
  const void *ptrs[] = {dout, q, k, v, out, dq, dk, dv};
  for (const void *ptr : ptrs)
    if (!aligned16(ptr))
      return B200_ERR_ALIGNMENT;
  const bool bf16 = dtype == B200_BF16;
  // dq / dk / dv use the strides of q / k / v and dout those of out, as in the
  // reference's custom call (flash_api.cu:370-381)
  // q / k / v / dout are read both as a block's own 128-row tile and as streamed 64-row tiles
  CUtensorMap q_map, k_map, v_map, do_map, q64_map, k64_map, v64_map, do64_map, dq_map, dk_map, dv_map;
  struct {
    CUtensorMap *m;
    const void *base;
    int64_t heads, seq, hs, rs, bs;
    uint32_t box_rows;
  } maps[] = {{&q_map, q, a.h, a.seqlen_q, a.q_head_stride, a.q_row_stride, a.q_batch_stride, 128},
              {&k_map, k, a.h_k, a.seqlen_k, a.k_head_stride, a.k_row_stride, a.k_batch_stride, 128},
              {&v_map, v, a.h_k, a.seqlen_k, a.v_head_stride, a.v_row_stride, a.v_batch_stride, 128},
              {&do_map, dout, a.h, a.seqlen_q, a.o_head_stride, a.o_row_stride, a.o_batch_stride, 128},
              {&q64_map, q, a.h, a.seqlen_q, a.q_head_stride, a.q_row_stride, a.q_batch_stride, kBwdBN},
              {&k64_map, k, a.h_k, a.seqlen_k, a.k_head_stride, a.k_row_stride, a.k_batch_stride, kBwdBN},
              {&v64_map, v, a.h_k, a.seqlen_k, a.v_head_stride, a.v_row_stride, a.v_batch_stride, kBwdBN},
              {&do64_map, dout, a.h, a.seqlen_q, a.o_head_stride, a.o_row_stride, a.o_batch_stride, kBwdBN},
              {&dq_map, dq, a.h, a.seqlen_q, a.q_head_stride, a.q_row_stride, a.q_batch_stride, 128},
              {&dk_map, dk, a.h_k, a.seqlen_k, a.k_head_stride, a.k_row_stride, a.k_batch_stride, 128},
              {&dv_map, dv, a.h_k, a.seqlen_k, a.v_head_stride, a.v_row_stride, a.v_batch_stride, 128}};
  for (auto &m : maps)
    if (int rc = make_qkv_map(m.m, bf16, m.base, a.d, m.heads, m.seq, a.b, m.hs, m.rs, m.bs, m.box_rows))
      return rc;

  const int64_t rows = a.b * a.h * a.seqlen_q;
  bwd_dot_do_o_kernel<<<(unsigned)ceil_div<int64_t>(rows, 16), 256, 0, stream>>>(
      dout, out, d_softmax_sum, a.b, a.h, a.seqlen_q, a.seqlen_q_rounded, a.o_batch_stride, a.o_row_stride,
      a.o_head_stride, (int)a.d, bf16);
  if (int rc = check_launch())
    return rc;

  BwdParams p;
  p.lse = softmax_lse;
  p.dsum = d_softmax_sum;
  p.H = a.h;
  p.Hk = a.h_k;
  p.Sq = a.seqlen_q;
  p.Sk = a.seqlen_k;
  p.Sq_rounded = a.seqlen_q_rounded;
  p.scale = a.softmax_scale;
  p.scale_log2 = a.softmax_scale * 1.4426950408889634f;
  p.window_left = a.window_size_left;
  p.window_right = a.window_size_right;
  p.wait_polls = g_wait_polls;
  p.debug_skip_arrive = g_debug_skip_arrive;
  p.d = (int)a.d;
  const dim3 grid_kv((unsigned)((a.seqlen_k + 127) / 128), (unsigned)a.h_k, (unsigned)a.b);
  const dim3 grid_q((unsigned)((a.seqlen_q + kBM - 1) / kBM), (unsigned)a.h, (unsigned)a.b);
  int rc = bf16 ? launch_bwd<true, true>(k_map, v_map, q64_map, do64_map, dk_map, dv_map, p, grid_kv, stream)
                : launch_bwd<false, true>(k_map, v_map, q64_map, do64_map, dk_map, dv_map, p, grid_kv, stream);
  if (rc)
    return rc;
  return bf16 ? launch_bwd<true, false>(q_map, do_map, k64_map, v64_map, dq_map, dq_map, p, grid_q, stream)
              : launch_bwd<false, false>(q_map, do_map, k64_map, v64_map, dq_map, dq_map, p, grid_q, stream);
}
