// Flash-attention forward for sm_100a (head dim 128, f16 / bf16, f32 accumulate).
//
// One block owns 128 query rows of one (batch, head) and walks over the key/value
// tiles of 128 rows that the mask lets it see.  Warp roles:
//   warp 0      TMA producer: Q once, then K and V tiles into 2-stage rings
//   warp 1      MMA issuer (one lane): S = Q K^T and O += P V with tcgen05.mma,
//               accumulators in tensor memory (S double-buffered, O resident)
//   warps 2..9  softmax: two threads per query row, 64 key columns each; a thread
//               reads its part of the row of S from tensor memory, keeps the
//               running max (agreed with its partner) and its part of the row sum,
//               writes P (16-bit) to shared memory as the A operand of P V,
//               rescales its half of O in tensor memory when the running max
//               moved, and writes O / LSE at the end
// While the softmax warps work on tile j the tensor core already computes
// S for tile j + 1.
//
// Numerics follow the reference kernel (external_libs/runtime/flash_attn/lib/
// softmax.h:129-178, flash_fwd_kernel.h:276-453): exp2 domain with the scale
// folded in, row sum from the unrounded f32 probabilities, P rounded to the
// storage type before P V, LSE = max * scale + ln(sum), +inf for a fully masked
// row.  One deviation that does not change the result: O is only rescaled when
// the running max grew by more than 2^8 (the stale max is used consistently for
// P, the row sum and the LSE).
#include <cuda.h>

#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace b200 {
namespace {

constexpr int kBM = 128;        // query rows per block
constexpr int kBN = 128;        // key rows per tile
constexpr int kD = 128;         // head dim
constexpr int kStages = 2;      // K / V ring depth
constexpr uint32_t kTileBytes = kBN * kD * 2;  // 32 KiB: two 64-column blocks of 128 x 128 B
constexpr uint32_t kHalfTile = kTileBytes / 2; // one 64-column block
constexpr int kThreads = 320;    // forward: producer, MMA issuer, eight softmax warps
constexpr int kBwdThreads = 192; // backward: producer, MMA issuer, one elementwise group
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO = 256;
constexpr float kRescaleThreshold = 8.0f; // log2 units
constexpr int kPolyEvery = 4; // forward softmax: one exponential in 4 is a polynomial (0 = none)

struct FwdParams {
  float *lse;
  int *status;
  int64_t H, Hk, Sq, Sk;
  float scale_log2;
  int64_t window_left, window_right; // < 0: unbounded
};

// 2^x for x <= 0 on the FMA/ALU pipes (the MUFU unit, 16 results per clock per SM, is the
// softmax bottleneck).  Round x to the nearest integer n with the 1.5 * 2^23 trick, evaluate
// 2^(x - n) on [-0.5, 0.5] with a degree-4 polynomial (relative error 4e-5, well below the
// 16-bit rounding P gets anyway) and add n to the exponent field.  Below 2^-125: exactly 0.
__device__ __forceinline__ float exp2_poly(float x) {
  const float xc = fmaxf(x, -125.f);
  const float r = xc + 12582912.f;
  const float f = xc - (r - 12582912.f);
  float y = fmaf(f, 0.009618129f, 0.05550411f);
  y = fmaf(y, f, 0.2402265f);
  y = fmaf(y, f, 0.6931472f);
  y = fmaf(y, f, 1.0f);
  const float v = __uint_as_float(__float_as_uint(y) + (__float_as_uint(r) << 23));
  return x < -125.f ? 0.f : v;
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

struct SharedStorage {
  uint64_t bar_q;
  uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, o_done;
  uint32_t tmem_base;
  int failed;
  float xch[2][2][128]; // per-row values the two column halves of the softmax exchange
};

__device__ __forceinline__ bool wait_or_flag(uint64_t *bar, uint32_t parity, SharedStorage *ss) {
  if (mbar_wait(bar, parity))
    return true;
  ss->failed = 1; // some arrival never came: every role gives up at its next wait
  return false;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, bool bf16) {
  if (bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

template <bool kBF16>
__global__ void __launch_bounds__(kThreads, 1)
    flash_fwd_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                     const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap o_map,
                     const FwdParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *smem =
      reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *sQ = smem;
  unsigned char *sK = sQ + kTileBytes;
  unsigned char *sV = sK + kStages * kTileBytes;
  unsigned char *sP = sV + kStages * kTileBytes;
  SharedStorage *ss = reinterpret_cast<SharedStorage *>(sP + kTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_q_tiles = (int)((p.Sq + kBM - 1) / kBM);
  const int q_tile = n_q_tiles - 1 - (int)blockIdx.x; // longest rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = (int)(h / (p.H / p.Hk));
  const int64_t q0 = (int64_t)q_tile * kBM;
  const int64_t shift = p.Sk - p.Sq;
  const bool right_bounded = p.window_right >= 0;
  const bool left_bounded = p.window_left >= 0;

  // key tiles this block visits: [0, n)
  int n = (int)((p.Sk + kBN - 1) / kBN);
  if (right_bounded) {
    const int64_t last_visible = q0 + kBM - 1 + shift + p.window_right;
    n = last_visible < 0 ? 0 : (int)min((int64_t)n, last_visible / kBN + 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(&ss->bar_q, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&ss->k_full[s], 1);
      mbar_init(&ss->k_empty[s], 1);
      mbar_init(&ss->v_full[s], 1);
      mbar_init(&ss->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ss->s_full[s], 1);
      mbar_init(&ss->s_empty[s], 8);
    }
    mbar_init(&ss->p_full, 8);
    mbar_init(&ss->o_done, 1);
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

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0 && n > 0) {
      prefetch_tensormap(&q_map);
      prefetch_tensormap(&k_map);
      prefetch_tensormap(&v_map);
      mbar_arrive_expect_tx(&ss->bar_q, kTileBytes);
      tma_load_4d(sQ, &q_map, 0, h, (int)q0, b, &ss->bar_q);
      tma_load_4d(sQ + kHalfTile, &q_map, 64, h, (int)q0, b, &ss->bar_q);
      for (int j = 0; j < n; ++j) {
        const int st = j % kStages;
        const uint32_t ph = (uint32_t)((j / kStages) & 1);
        if (!wait_or_flag(&ss->k_empty[st], ph ^ 1, ss))
          break;
        mbar_arrive_expect_tx(&ss->k_full[st], kTileBytes);
        tma_load_4d(sK + st * kTileBytes, &k_map, 0, hk, j * kBN, b, &ss->k_full[st]);
        tma_load_4d(sK + st * kTileBytes + kHalfTile, &k_map, 64, hk, j * kBN, b, &ss->k_full[st]);
        if (!wait_or_flag(&ss->v_empty[st], ph ^ 1, ss))
          break;
        mbar_arrive_expect_tx(&ss->v_full[st], kTileBytes);
        tma_load_4d(sV + st * kTileBytes, &v_map, 0, hk, j * kBN, b, &ss->v_full[st]);
        tma_load_4d(sV + st * kTileBytes + kHalfTile, &v_map, 64, hk, j * kBN, b, &ss->v_full[st]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_qk = umma_idesc_f16(kBF16, kBM, kBN, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_f16(kBF16, kBM, kD, false, true);
      const uint32_t q_addr = smem_addr(sQ), k_addr = smem_addr(sK), v_addr = smem_addr(sV), p_addr = smem_addr(sP);
      auto issue_qk = [&](int j) { // S[j & 1] = Q K_j^T
        const int st = j % kStages;
        const uint32_t d_tmem = tmem + ((j & 1) ? kColS1 : kColS0);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t off = kb * kHalfTile + ks * 32;
            umma_ss(d_tmem, umma_smem_desc(q_addr + off, 16, 1024),
                    umma_smem_desc(k_addr + st * kTileBytes + off, 16, 1024), idesc_qk, (kb | ks) != 0);
          }
        umma_commit(&ss->s_full[j & 1]);
        umma_commit(&ss->k_empty[st]);
      };
      bool ok = wait_or_flag(&ss->bar_q, 0, ss) && wait_or_flag(&ss->k_full[0], 0, ss);
      if (ok) {
        tc_fence_after_sync();
        issue_qk(0);
      }
      for (int j = 0; ok && j < n; ++j) {
        if (j + 1 < n) {
          const int st = (j + 1) % kStages;
          ok = wait_or_flag(&ss->k_full[st], (uint32_t)(((j + 1) / kStages) & 1), ss) &&
               wait_or_flag(&ss->s_empty[(j + 1) & 1], (uint32_t)((((j + 1) / 2) & 1) ^ 1), ss);
          if (!ok)
            break;
          tc_fence_after_sync();
          issue_qk(j + 1);
        }
        const int st = j % kStages;
        ok = wait_or_flag(&ss->p_full, (uint32_t)(j & 1), ss) &&
             wait_or_flag(&ss->v_full[st], (uint32_t)((j / kStages) & 1), ss);
        if (!ok)
          break;
        tc_fence_after_sync();
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            // A: P[:, 16 keys] (K-major); B: V[16 keys, 128 dims] (dims contiguous = MN-major)
            const uint64_t adesc = umma_smem_desc(p_addr + kb * kHalfTile + ks * 32, 16, 1024);
            const uint64_t bdesc =
                umma_smem_desc(v_addr + st * kTileBytes + (kb * 64 + ks * 16) * 128, kHalfTile, 1024);
            umma_ss(tmem + kColO, adesc, bdesc, idesc_pv, (j | kb | ks) != 0);
          }
        umma_commit(&ss->o_done);
        umma_commit(&ss->v_empty[st]);
      }
    }
  } else {
    // ------------------------------------------------------------- softmax
    // Eight warps: warps 2..5 take key columns 0..63 of the tile, warps 6..9 columns 64..127;
    // inside each half, thread t owns query row t.  The two threads of a row agree on the row
    // maximum through shared memory once per tile; their row sums only meet in the epilogue.
    const int half = (warp - 2) >> 2;          // which 64 key columns (and, for O, which 64 dims)
    const int quarter = warp & 3;              // tensor-memory lanes 32 * quarter .. + 31
    const int row = quarter * 32 + lane;       // query row inside the tile
    const int64_t qrow = q0 + row;             // global query row
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    constexpr int kHC = kBN / 2;               // columns per thread
    float m_used = -INFINITY, l = 0.f;
    bool ok = n > 0, waits_ok = true;
    for (int j = 0; ok && j < n; ++j) {
      waits_ok = waits_ok && wait_or_flag(&ss->s_full[j & 1], (uint32_t)((j / 2) & 1), ss);
      tc_fence_after_sync();
      // this thread's 64 columns of S into registers; S may then be overwritten by the
      // Q K^T after next
      uint32_t s[kHC];
      {
        const uint32_t base = tmem + lane_base + ((j & 1) ? kColS1 : kColS0) + half * kHC;
        tmem_ld32(base, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_ld32(base + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
        tmem_wait_ld();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&ss->s_empty[j & 1]);

      const int64_t kv0 = (int64_t)j * kBN + half * kHC; // first key column of this thread
      const bool need_mask = (right_bounded && (int64_t)j * kBN + kBN - 1 > q0 + shift + p.window_right) ||
                             ((int64_t)j * kBN + kBN > p.Sk) || left_bounded;
      if (need_mask) { // visible columns for this row among this thread's 64: [lo, hi]
        const int64_t hi64 = (right_bounded ? min(p.Sk - 1, qrow + shift + p.window_right) : p.Sk - 1) - kv0;
        const int64_t lo64 = (left_bounded ? qrow + shift - p.window_left : 0) - kv0;
        const int hi = (int)max((int64_t)-1, min((int64_t)kHC - 1, hi64));
        const int lo = (int)max((int64_t)0, min((int64_t)kHC, lo64));
#pragma unroll
        for (int c = 0; c < kHC; ++c)
          if (c > hi || c < lo)
            s[c] = 0xff800000u; // -inf
      }
      float mx8[8];
#pragma unroll
      for (int e = 0; e < 8; ++e)
        mx8[e] = fmaxf(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1]));
#pragma unroll
      for (int c = 16; c < kHC; c += 16) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          mx8[e] = fmaxf(mx8[e], fmaxf(__uint_as_float(s[c + 2 * e]), __uint_as_float(s[c + 2 * e + 1])));
      }
      float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                       fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
      // the other half's maximum of the same row (buffers alternate with the tile's parity)
      ss->xch[j & 1][half][row] = mx;
      if (named_bar_or_n<256>(!waits_ok)) { // a wait ran out somewhere: all 256 leave together
        ok = false;
        break;
      }
      mx = fmaxf(mx, ss->xch[j & 1][half ^ 1][row]);
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      float alpha = 1.f;
      const bool grew = m_new - m_used > kRescaleThreshold; // also true for -inf -> finite
      const bool rescale = j > 0 && __any_sync(0xffffffffu, grew); // same verdict in both halves
      if (j == 0) {
        m_used = m_new;
      } else if (rescale) {
        alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(m_used - m_new);
        m_used = m_new;
        l *= alpha;
      }
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
      // probabilities (one in kPolyEvery on the FMA pipes, the rest on the MUFU unit), four
      // independent partial sums; the packed 16-bit P reuses the front of the registers
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < kHC; c += 2) {
        const float x0 = fmaf(__uint_as_float(s[c]), p.scale_log2, -m_safe);
        const float x1 = fmaf(__uint_as_float(s[c + 1]), p.scale_log2, -m_safe);
        const float p0 = fast_exp2(x0);
        const float p1 = (kPolyEvery > 0 && (c + 1) % kPolyEvery == kPolyEvery - 1) ? exp2_poly(x1) : fast_exp2(x1);
        sum4[(c >> 1) & 3] += p0 + p1;
        s[c >> 1] = pack2(p0, p1, kBF16);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);

      // P's buffer and O are busy until P V of the previous tile has finished (a wait that runs
      // out is reported at the next barrier)
      if (j > 0)
        waits_ok = waits_ok && wait_or_flag(&ss->o_done, (uint32_t)((j - 1) & 1), ss);
      tc_fence_after_sync();
      // P row -> shared memory, K-major 128-byte swizzled: [2 key blocks][128 rows][128 B];
      // this thread's 64 columns are exactly key block `half`
#pragma unroll
      for (int chunk = 0; chunk < 8; ++chunk)
        *reinterpret_cast<uint4 *>(sP + half * kHalfTile + row * 128 + ((chunk ^ (row & 7)) << 4)) =
            make_uint4(s[chunk * 4], s[chunk * 4 + 1], s[chunk * 4 + 2], s[chunk * 4 + 3]);
      fence_proxy_async_smem();
      if (rescale) { // this thread's 64 of the row's 128 head dims
        const uint32_t base = tmem + lane_base + kColO + half * kHC;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(base + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(base + c * 32, r);
        }
        tmem_wait_st();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&ss->p_full);
    }

    // ---- epilogue: O / l -> 16 bit -> shared -> TMA store; LSE
    if (ok && n > 0)
      waits_ok = waits_ok && wait_or_flag(&ss->o_done, (uint32_t)((n - 1) & 1), ss);
    tc_fence_after_sync();
    ss->xch[n & 1][half][row] = l; // the row sum is the sum of the two halves' sums
    if (named_bar_or_n<256>(!waits_ok))
      ok = false;
    l += ss->xch[n & 1][half ^ 1][row];
    const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
    const bool have_o = ok && n > 0;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t r[32];
      if (have_o) {
        tmem_ld32(tmem + lane_base + kColO + half * kHC + c * 32, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          r[i] = 0u;
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) { // 8 columns = one 16-byte chunk of head-dim block `half`
        uint4 v;
        v.x = pack2(__uint_as_float(r[g * 8 + 0]) * inv_l, __uint_as_float(r[g * 8 + 1]) * inv_l, kBF16);
        v.y = pack2(__uint_as_float(r[g * 8 + 2]) * inv_l, __uint_as_float(r[g * 8 + 3]) * inv_l, kBF16);
        v.z = pack2(__uint_as_float(r[g * 8 + 4]) * inv_l, __uint_as_float(r[g * 8 + 5]) * inv_l, kBF16);
        v.w = pack2(__uint_as_float(r[g * 8 + 6]) * inv_l, __uint_as_float(r[g * 8 + 7]) * inv_l, kBF16);
        const int chunk = c * 4 + g;
        *reinterpret_cast<uint4 *>(sP + half * kHalfTile + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
      }
    }
    fence_proxy_async_smem();
    if (half == 0 && qrow < p.Sq)
      p.lse[((int64_t)b * p.H + h) * p.Sq + qrow] =
          (l > 0.f) ? (m_used + log2f(l)) * 0.6931471805599453f : INFINITY;
    asm volatile("bar.sync 1, 256;" ::: "memory"); // the eight softmax warps
    if (warp == 2 && lane == 0 && ss->failed == 0) {
      tma_store_4d(&o_map, sP, 0, h, (int)q0, b);
      tma_store_4d(&o_map, sP + kHalfTile, 64, h, (int)q0, b);
      bulk_commit();
      bulk_wait_all<0>();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && ss->failed && p.status)
    *p.status = 2;
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

int make_qkv_map(CUtensorMap *map, bool bf16, const void *base, int64_t d, int64_t heads, int64_t seq,
                 int64_t batch, int64_t head_stride, int64_t row_stride, int64_t batch_stride) {
  const uint64_t dims[4] = {(uint64_t)d, (uint64_t)heads, (uint64_t)seq, (uint64_t)batch};
  const uint64_t strides[3] = {(uint64_t)head_stride * 2, (uint64_t)row_stride * 2, (uint64_t)batch_stride * 2};
  const uint32_t box[4] = {64, 1, 128, 1};
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

constexpr uint32_t kColDP = 128, kColAcc0 = 256, kColAcc1 = 384;

struct BwdParams {
  const float *lse;   // [B, H, Sq]
  const float *dsum;  // [B, H, Sq_rounded]
  int64_t H, Hk, Sq, Sk, Sq_rounded;
  float scale, scale_log2;
  int64_t window_left, window_right;
};

struct BwdShared {
  uint64_t bar_resident;          // the block's own tiles (K,V or Q,dO)
  uint64_t full[2], empty[2];     // streamed tile pairs
  uint64_t st_full, st_empty;     // S / dP in tensor memory
  uint64_t pds_full, pds_empty;   // P / dS in shared memory
  uint32_t tmem_base;
  int failed;
};
struct BwdStats { // row statistics of the streamed query tile (dK/dV kernel only)
  float lse2[2][128];
  float dsum[2][128];
};

__device__ __forceinline__ bool named_bar_or(bool pred) { return named_bar_or_n<128>(pred); }

__device__ __forceinline__ bool bwd_wait(uint64_t *bar, uint32_t parity, BwdShared *ss) {
  if (mbar_wait(bar, parity))
    return true;
  ss->failed = 1;
  return false;
}

// 16-byte chunk `chunk16` (0..15: 8 columns each) of row `row` of a 128 x 128 16-bit
// tile stored as [2 column blocks][128 rows][128 B] with the 128-byte swizzle
__device__ __forceinline__ void store_tile_chunk(unsigned char *tile, int row, int chunk16, uint4 v) {
  const int blk = chunk16 >> 3, chunk = chunk16 & 7;
  *reinterpret_cast<uint4 *>(tile + blk * kHalfTile + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
}

__global__ void __launch_bounds__(256)
    bwd_dot_do_o_kernel(const void *__restrict__ dout, const void *__restrict__ out, float *__restrict__ dsum,
                        int64_t B, int64_t H, int64_t Sq, int64_t Sq_rounded, int64_t o_batch_stride,
                        int64_t o_row_stride, int64_t o_head_stride, bool bf16) {
  // 16 threads per (b, h, row): 8 elements each of the 128-wide row
  const int64_t gid = (int64_t)blockIdx.x * 16 + (threadIdx.x >> 4);
  const int sub = threadIdx.x & 15;
  const int64_t total = B * H * Sq;
  float acc = 0.f;
  if (gid < total) {
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

// kDKDV = true : block owns keys [kv0, kv0+128) (rows of the transposed tiles), streams (Q, dO) tiles
// kDKDV = false: block owns queries [q0, q0+128), streams (K, V) tiles
template <bool kBF16, bool kDKDV>
__global__ void __launch_bounds__(kBwdThreads, 1)
    flash_bwd_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                     const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap do_map,
                     const __grid_constant__ CUtensorMap out0_map, // dK (kDKDV) or dQ
                     const __grid_constant__ CUtensorMap out1_map, // dV (kDKDV), unused otherwise
                     const BwdParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *smem =
      reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  // resident pair, streamed pairs, then the dS tile (and the P tile for dK/dV).
  // Shared memory holds 7 tiles: the dK/dV kernel needs P and dS, so it streams
  // through a single stage; the dQ kernel needs only dS and double-buffers.
  constexpr int kBwdStages = kDKDV ? 1 : 2;
  unsigned char *sRes0 = smem;                       // K (kDKDV) / Q
  unsigned char *sRes1 = sRes0 + kTileBytes;         // V (kDKDV) / dO
  unsigned char *sStr = sRes1 + kTileBytes;          // [stage][2 tiles]: (Q, dO) or (K, V)
  unsigned char *sDS = sStr + kBwdStages * 2 * kTileBytes;
  unsigned char *sP = sDS + kTileBytes;              // kDKDV only
  BwdShared *ss = reinterpret_cast<BwdShared *>(sDS + (kDKDV ? 2 : 1) * kTileBytes);
  BwdStats *stats = reinterpret_cast<BwdStats *>(ss + 1); // present only if kDKDV

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int64_t shift = p.Sk - p.Sq;
  const bool right_bounded = p.window_right >= 0;
  const bool left_bounded = p.window_left >= 0;
  const int group = (int)(p.H / p.Hk);
  const int n_q_tiles = (int)((p.Sq + kBM - 1) / kBM);
  const int n_k_tiles = (int)((p.Sk + kBN - 1) / kBN);

  // the tile this block owns, and the range of streamed tiles [t_begin, t_end)
  int own_tile, head, t_begin, t_end, heads_in_loop;
  if (kDKDV) {
    own_tile = blockIdx.x;
    head = blockIdx.y; // key/value head
    heads_in_loop = group;
    t_begin = 0;
    t_end = n_q_tiles;
    if (right_bounded) { // queries that can see key kv0: q >= kv0 - shift - window_right
      const int64_t first_q = (int64_t)own_tile * kBN - shift - p.window_right;
      t_begin = first_q <= 0 ? 0 : (int)min((int64_t)n_q_tiles, first_q / kBM);
    }
  } else {
    own_tile = n_q_tiles - 1 - (int)blockIdx.x;
    head = blockIdx.y; // query head
    heads_in_loop = 1;
    t_begin = 0;
    t_end = n_k_tiles;
    if (right_bounded) {
      const int64_t last_visible = (int64_t)own_tile * kBM + kBM - 1 + shift + p.window_right;
      t_end = last_visible < 0 ? 0 : (int)min((int64_t)n_k_tiles, last_visible / kBN + 1);
    }
  }
  const int tiles_per_head = max(0, t_end - t_begin);
  const int T = tiles_per_head * heads_in_loop;
  const int64_t own0 = (int64_t)own_tile * 128;

  if (threadIdx.x == 0) {
    mbar_init(&ss->bar_resident, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ss->full[s], 1);
      mbar_init(&ss->empty[s], 1);
    }
    mbar_init(&ss->st_full, 1);
    mbar_init(&ss->st_empty, 4);
    mbar_init(&ss->pds_full, 4);
    mbar_init(&ss->pds_empty, 1);
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
      mbar_arrive_expect_tx(&ss->bar_resident, 2 * kTileBytes);
      if (kDKDV) {
        tma_load_4d(sRes0, &k_map, 0, kv_head, (int)own0, b, &ss->bar_resident);
        tma_load_4d(sRes0 + kHalfTile, &k_map, 64, kv_head, (int)own0, b, &ss->bar_resident);
        tma_load_4d(sRes1, &v_map, 0, kv_head, (int)own0, b, &ss->bar_resident);
        tma_load_4d(sRes1 + kHalfTile, &v_map, 64, kv_head, (int)own0, b, &ss->bar_resident);
      } else {
        tma_load_4d(sRes0, &q_map, 0, head, (int)own0, b, &ss->bar_resident);
        tma_load_4d(sRes0 + kHalfTile, &q_map, 64, head, (int)own0, b, &ss->bar_resident);
        tma_load_4d(sRes1, &do_map, 0, head, (int)own0, b, &ss->bar_resident);
        tma_load_4d(sRes1 + kHalfTile, &do_map, 64, head, (int)own0, b, &ss->bar_resident);
      }
      for (int it = 0; it < T; ++it) {
        const int st = it % kBwdStages;
        if (!bwd_wait(&ss->empty[st], (uint32_t)(((it / kBwdStages) & 1) ^ 1), ss))
          break;
        mbar_arrive_expect_tx(&ss->full[st], 2 * kTileBytes);
        unsigned char *t0 = sStr + st * 2 * kTileBytes, *t1 = t0 + kTileBytes;
        const int row0 = iter_tile(it) * 128;
        const CUtensorMap *m0 = kDKDV ? &q_map : &k_map, *m1 = kDKDV ? &do_map : &v_map;
        const int hh = kDKDV ? iter_head(it) : kv_head;
        tma_load_4d(t0, m0, 0, hh, row0, b, &ss->full[st]);
        tma_load_4d(t0 + kHalfTile, m0, 64, hh, row0, b, &ss->full[st]);
        tma_load_4d(t1, m1, 0, hh, row0, b, &ss->full[st]);
        tma_load_4d(t1 + kHalfTile, m1, 64, hh, row0, b, &ss->full[st]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0 && T > 0) {
      constexpr uint32_t idesc_nt = umma_idesc_f16(kBF16, 128, 128, false, false); // A, B both K-major
      constexpr uint32_t idesc_nn = umma_idesc_f16(kBF16, 128, 128, false, true);  // B rows = K index
      const uint32_t res0 = smem_addr(sRes0), res1 = smem_addr(sRes1), str = smem_addr(sStr);
      const uint32_t p_addr = smem_addr(sP), ds_addr = smem_addr(sDS);
      bool ok = bwd_wait(&ss->bar_resident, 0, ss);
      for (int it = 0; ok && it < T; ++it) {
        const int st = it % kBwdStages;
        const uint32_t t0 = str + st * 2 * kTileBytes, t1 = t0 + kTileBytes;
        ok = bwd_wait(&ss->full[st], (uint32_t)((it / kBwdStages) & 1), ss) &&
             bwd_wait(&ss->st_empty, (uint32_t)((it & 1) ^ 1), ss);
        if (!ok)
          break;
        tc_fence_after_sync();
        // kDKDV: S^T = K Q^T, dP^T = V dO^T ; else: S = Q K^T, dP = dO V^T  (contraction over head dim)
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t off = kb * kHalfTile + ks * 32;
            umma_ss(tmem + kColS0, umma_smem_desc(res0 + off, 16, 1024), umma_smem_desc(t0 + off, 16, 1024),
                    idesc_nt, (kb | ks) != 0);
          }
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t off = kb * kHalfTile + ks * 32;
            umma_ss(tmem + kColDP, umma_smem_desc(res1 + off, 16, 1024), umma_smem_desc(t1 + off, 16, 1024),
                    idesc_nt, (kb | ks) != 0);
          }
        umma_commit(&ss->st_full);
        ok = bwd_wait(&ss->pds_full, (uint32_t)(it & 1), ss);
        if (!ok)
          break;
        tc_fence_after_sync();
        // contraction over the 128 streamed (kDKDV: query) or owned-side columns of P / dS
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t a_off = kb * kHalfTile + ks * 32;
            const uint32_t b_off = (kb * 64 + ks * 16) * 128;
            if (kDKDV) {
              // dV += P^T dO ; dK += dS^T Q   (B = streamed tiles, rows = queries)
              umma_ss(tmem + kColAcc0, umma_smem_desc(p_addr + a_off, 16, 1024),
                      umma_smem_desc(t1 + b_off, kHalfTile, 1024), idesc_nn, (it | kb | ks) != 0);
              umma_ss(tmem + kColAcc1, umma_smem_desc(ds_addr + a_off, 16, 1024),
                      umma_smem_desc(t0 + b_off, kHalfTile, 1024), idesc_nn, (it | kb | ks) != 0);
            } else {
              // dQ += dS K   (B = streamed K tile, rows = keys)
              umma_ss(tmem + kColAcc0, umma_smem_desc(ds_addr + a_off, 16, 1024),
                      umma_smem_desc(t0 + b_off, kHalfTile, 1024), idesc_nn, (it | kb | ks) != 0);
            }
          }
        umma_commit(&ss->pds_empty);
        umma_commit(&ss->empty[st]);
      }
    }
  } else {
    // ------------------------------------------------------------- elementwise warps
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;       // owned-side row: a key (kDKDV) or a query
    const int64_t own_idx = own0 + row;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int tid128 = (warp - 2) * 32 + lane; // 0..127 among the four warps
    const float kLog2e = 1.4426950408889634f;
    float my_lse2 = 0.f, my_dsum = 0.f;
    if (!kDKDV && own_idx < p.Sq) {
      my_lse2 = p.lse[((int64_t)b * p.H + head) * p.Sq + own_idx] * kLog2e;
      my_dsum = p.dsum[((int64_t)b * p.H + head) * p.Sq_rounded + own_idx];
    }
    bool ok = T > 0;
    for (int it = 0; ok && it < T; ++it) {
      const int64_t str0 = (int64_t)iter_tile(it) * 128;
      if (kDKDV) { // statistics of the streamed query tile, one element per thread
        const int64_t qi = str0 + tid128;
        const int qh = iter_head(it);
        float l2 = INFINITY, dd = 0.f; // rows past the end: P = exp2(-inf) = 0
        if (qi < p.Sq) {
          l2 = p.lse[((int64_t)b * p.H + qh) * p.Sq + qi] * kLog2e;
          dd = p.dsum[((int64_t)b * p.H + qh) * p.Sq_rounded + qi];
        }
        stats->lse2[it & 1][tid128] = l2;
        stats->dsum[it & 1][tid128] = dd;
      }
      const bool waited = bwd_wait(&ss->st_full, (uint32_t)(it & 1), ss) &&
                          (it == 0 || bwd_wait(&ss->pds_empty, (uint32_t)((it - 1) & 1), ss));
      // one barrier per tile: publishes the statistics above and makes giving up unanimous
      if (named_bar_or(!waited)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // visibility of (query, key): key <= query + shift + wr, key >= query + shift - wl, both in range
      const int64_t q_base = kDKDV ? str0 : own_idx; // + column if kDKDV
      const int64_t k_base = kDKDV ? own_idx : str0; // + column if !kDKDV
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t sr[32], dr[32];
        tmem_ld32(tmem + lane_base + kColS0 + c * 32, sr);
        tmem_ld32(tmem + lane_base + kColDP + c * 32, dr);
        tmem_wait_ld();
        if (c == 3) { // all of S / dP has been read: the tensor core may overwrite them
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0)
            mbar_arrive(&ss->st_empty);
        }
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = c * 32 + i + e;
            const int64_t qi = kDKDV ? q_base + col : q_base;
            const int64_t ki = kDKDV ? k_base : k_base + col;
            const float l2 = kDKDV ? stats->lse2[it & 1][col] : my_lse2;
            const float ds_ = kDKDV ? stats->dsum[it & 1][col] : my_dsum;
            bool vis = qi < p.Sq && ki < p.Sk;
            if (right_bounded)
              vis = vis && ki <= qi + shift + p.window_right;
            if (left_bounded)
              vis = vis && ki >= qi + shift - p.window_left;
            const float pr = vis ? fast_exp2(fmaf(__uint_as_float(sr[i + e]), p.scale_log2, -l2)) : 0.f;
            pv[e] = pr;
            dv[e] = pr * (__uint_as_float(dr[i + e]) - ds_);
          }
          pp[i / 2] = pack2(pv[0], pv[1], kBF16);
          dd[i / 2] = pack2(dv[0], dv[1], kBF16);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (kDKDV)
            store_tile_chunk(sP, row, c * 4 + g, make_uint4(pp[g * 4], pp[g * 4 + 1], pp[g * 4 + 2], pp[g * 4 + 3]));
          store_tile_chunk(sDS, row, c * 4 + g, make_uint4(dd[g * 4], dd[g * 4 + 1], dd[g * 4 + 2], dd[g * 4 + 3]));
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&ss->pds_full);
    }

    // ---- epilogue: accumulators -> 16 bit -> shared -> TMA store
    if (ok && T > 0)
      ok = bwd_wait(&ss->pds_empty, (uint32_t)((T - 1) & 1), ss);
    tc_fence_after_sync();
    const bool have = ok && T > 0;
    const int n_acc = kDKDV ? 2 : 1;
    for (int a = 0; a < n_acc; ++a) {
      // kDKDV: acc0 = dV (unscaled) -> sP, acc1 = dK (* scale) -> sDS ; else acc0 = dQ (* scale) -> sDS
      const uint32_t col0 = a == 0 ? kColAcc0 : kColAcc1;
      unsigned char *stage = (kDKDV && a == 0) ? sP : sDS;
      const float mul = (kDKDV && a == 0) ? 1.f : p.scale;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        if (have) {
          tmem_ld32(tmem + lane_base + col0 + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            r[i] = 0u;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 v;
          v.x = pack2(__uint_as_float(r[g * 8 + 0]) * mul, __uint_as_float(r[g * 8 + 1]) * mul, kBF16);
          v.y = pack2(__uint_as_float(r[g * 8 + 2]) * mul, __uint_as_float(r[g * 8 + 3]) * mul, kBF16);
          v.z = pack2(__uint_as_float(r[g * 8 + 4]) * mul, __uint_as_float(r[g * 8 + 5]) * mul, kBF16);
          v.w = pack2(__uint_as_float(r[g * 8 + 6]) * mul, __uint_as_float(r[g * 8 + 7]) * mul, kBF16);
          store_tile_chunk(stage, row, c * 4 + g, v);
        }
      }
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (warp == 2 && lane == 0 && ss->failed == 0) {
      if (kDKDV) {
        tma_store_4d(&out1_map, sP, 0, head, (int)own0, b);
        tma_store_4d(&out1_map, sP + kHalfTile, 64, head, (int)own0, b);
      }
      tma_store_4d(&out0_map, sDS, 0, head, (int)own0, b);
      tma_store_4d(&out0_map, sDS + kHalfTile, 64, head, (int)own0, b);
      bulk_commit();
      bulk_wait_all<0>();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <bool kBF16, bool kDKDV>
int launch_bwd(const CUtensorMap &q_map, const CUtensorMap &k_map, const CUtensorMap &v_map,
               const CUtensorMap &do_map, const CUtensorMap &out0, const CUtensorMap &out1,
               const BwdParams &p, dim3 grid, cudaStream_t stream) {
  const size_t smem = kDKDV ? (size_t)6 * kTileBytes + sizeof(BwdShared) + sizeof(BwdStats) + 1024
                            : (size_t)7 * kTileBytes + sizeof(BwdShared) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (int rc = check_cuda(cudaFuncSetAttribute(flash_bwd_kernel<kBF16, kDKDV>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)))
      return rc;
    attr_set = true;
  }
  flash_bwd_kernel<kBF16, kDKDV><<<grid, kBwdThreads, smem, stream>>>(q_map, k_map, v_map, do_map, out0, out1, p);
  return check_launch();
}

} // namespace
} // namespace b200

using namespace b200;

extern "C" int b200_flash_attn_fwd(int dtype, const void *q, const void *k, const void *v, void *out,
                                   float *softmax_lse, const b200_flash_attn_params *pp, cudaStream_t stream) {
  if (!pp || !q || !k || !v || !out || !softmax_lse)
    return B200_ERR_INVALID_ARG;
  const b200_flash_attn_params &a = *pp;
  if (dtype != B200_F16 && dtype != B200_BF16)
    return B200_ERR_UNSUPPORTED;
  if (a.d != kD || a.p_dropout != 0.f || a.h_k <= 0 || a.h % a.h_k != 0 || a.b <= 0 || a.seqlen_q <= 0 ||
      a.seqlen_k <= 0)
    return B200_ERR_UNSUPPORTED; // head dim 128, no dropout
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
  p.H = a.h;
  p.Hk = a.h_k;
  p.Sq = a.seqlen_q;
  p.Sk = a.seqlen_k;
  p.scale_log2 = a.softmax_scale * 1.4426950408889634f;
  p.window_left = a.window_size_left;
  p.window_right = a.window_size_right;
  const size_t smem = (size_t)(1 + 2 * kStages + 1) * kTileBytes + sizeof(SharedStorage) + 1024;
  static bool attr_set[2] = {false, false};
  if (!attr_set[bf16]) {
    cudaError_t e = bf16 ? cudaFuncSetAttribute(flash_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                         : cudaFuncSetAttribute(flash_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (int rc = check_cuda(e))
      return rc;
    attr_set[bf16] = true;
  }
  const dim3 grid((unsigned)((a.seqlen_q + kBM - 1) / kBM), (unsigned)a.h, (unsigned)a.b);
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
  if (a.d != kD || a.p_dropout != 0.f || a.h_k <= 0 || a.h % a.h_k != 0 || a.b <= 0 || a.seqlen_q <= 0 ||
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
  CUtensorMap q_map, k_map, v_map, do_map, dq_map, dk_map, dv_map;
  struct {
    CUtensorMap *m;
    const void *base;
    int64_t heads, seq, hs, rs, bs;
  } maps[] = {{&q_map, q, a.h, a.seqlen_q, a.q_head_stride, a.q_row_stride, a.q_batch_stride},
              {&k_map, k, a.h_k, a.seqlen_k, a.k_head_stride, a.k_row_stride, a.k_batch_stride},
              {&v_map, v, a.h_k, a.seqlen_k, a.v_head_stride, a.v_row_stride, a.v_batch_stride},
              {&do_map, dout, a.h, a.seqlen_q, a.o_head_stride, a.o_row_stride, a.o_batch_stride},
              {&dq_map, dq, a.h, a.seqlen_q, a.q_head_stride, a.q_row_stride, a.q_batch_stride},
              {&dk_map, dk, a.h_k, a.seqlen_k, a.k_head_stride, a.k_row_stride, a.k_batch_stride},
              {&dv_map, dv, a.h_k, a.seqlen_k, a.v_head_stride, a.v_row_stride, a.v_batch_stride}};
  for (auto &m : maps)
    if (int rc = make_qkv_map(m.m, bf16, m.base, a.d, m.heads, m.seq, a.b, m.hs, m.rs, m.bs))
      return rc;

  const int64_t rows = a.b * a.h * a.seqlen_q;
  bwd_dot_do_o_kernel<<<(unsigned)ceil_div<int64_t>(rows, 16), 256, 0, stream>>>(
      dout, out, d_softmax_sum, a.b, a.h, a.seqlen_q, a.seqlen_q_rounded, a.o_batch_stride, a.o_row_stride,
      a.o_head_stride, bf16);
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
  const dim3 grid_kv((unsigned)((a.seqlen_k + kBN - 1) / kBN), (unsigned)a.h_k, (unsigned)a.b);
  const dim3 grid_q((unsigned)((a.seqlen_q + kBM - 1) / kBM), (unsigned)a.h, (unsigned)a.b);
  int rc = bf16 ? launch_bwd<true, true>(q_map, k_map, v_map, do_map, dk_map, dv_map, p, grid_kv, stream)
                : launch_bwd<false, true>(q_map, k_map, v_map, do_map, dk_map, dv_map, p, grid_kv, stream);
  if (rc)
    return rc;
  return bf16 ? launch_bwd<true, false>(q_map, k_map, v_map, do_map, dq_map, dq_map, p, grid_q, stream)
              : launch_bwd<false, false>(q_map, k_map, v_map, do_map, dq_map, dq_map, p, grid_q, stream);
}
