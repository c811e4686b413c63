// Attention over a key/value cache (decode): the kernel behind run_flash_attn_kvcache
// (reference: external_libs/runtime/flash_attn/lib/flash_api.cu:434-566,727-811; the
// kernel it dispatches is lib/flash_fwd_kernel.h:474-1060, lengths per batch entry from
// lib/block_info.h:11-41).
//
// Per batch entry b:  cache_len = seqlens_k[b];  the new rows knew/vnew are appended to
// the cache at [cache_len, cache_len + seqlen_knew);  then every query row attends to the
// first len = cache_len + seqlen_knew rows, the mask aligned to the END of the keys: query
// i sees key j iff  j <= i + (len - seqlen_q) + window_right  and
// j >= i + (len - seqlen_q) - window_left, a negative window being unbounded.  Blocks read
// the new rows from knew/vnew, so none waits for another's append.
//
// The work is a stream over the cache: 4*d bytes per key against 4*d flops per key and
// query row, so with the few query rows of a decode step it is bound by HBM.  The
// reference runs one block per (batch, head) (num_splits = 1), which leaves most of a
// B200 idle when batch * heads < 148; here the keys of every (batch entry, kv head) are cut
// into ranges, enough to fill the GPU, and a second small kernel merges the partial (max,
// sum, output) of the ranges.  All query heads that share a kv head are rows of the same
// block, so a grouped cache is read once per row chunk.
//
// Two kernels.  Head dims 64 and 128 (decode_mma_kernel): scores and outputs on tensor-core
// tiles, 16 query rows a block.  Other head dims (decode_split_kernel): a key row of d 16-bit
// values is read by LPK = pow2(d / 8) lanes, 16 bytes each, so a warp takes 32 / LPK keys per
// step; every lane group keeps a running (max, sum, output slice) per query row in registers,
// rescaled only when the maximum grows; groups are merged by shuffles, warps through shared
// memory.
#include "common.cuh"

#include <algorithm>
#include <cmath>

namespace b200 {
namespace {

constexpr int kDecodeWarps = 8;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kMaxSplits = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct DecodeParams {
  const void *q;
  void *kcache, *vcache;
  const void *knew, *vnew;
  const int *seqlens_k;
  void *o;
  float *lse;
  float *part_o;  // [rows][splits][d]   (rows = b * h * seqlen_q), only when splits > 1
  float *part_ml; // [rows][splits][2]   running maximum (log2 units) and sum
  int64_t q_bs, k_bs, v_bs, kn_bs, vn_bs, o_bs;
  int64_t q_rs, k_rs, v_rs, kn_rs, vn_rs, o_rs;
  int64_t q_hs, k_hs, v_hs, kn_hs, vn_hs, o_hs;
  int b, h, h_k, d, group;
  int seqlen_q, seqlen_k, seqlen_knew;
  int window_left, window_right;
  int splits, chunks, rows_per_kv; // rows_per_kv = seqlen_q * group
  float scale_log2;
};

template <bool kBF16> __device__ __forceinline__ void unpack8(const uint4 &raw, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (kBF16) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}

// 2^(a - b) for running maxima, where "nothing seen yet" is -inf on either side
__device__ __forceinline__ float scale_of(float m, float m_new) {
  return m == -INFINITY ? 0.f : exp2f(m - m_new);
}

template <int LPK, int RC, bool kBF16>
__global__ void __launch_bounds__(kDecodeThreads) decode_split_kernel(const DecodeParams p) {
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  constexpr int KPW = 32 / LPK;             // keys per warp step
  constexpr int KPB = KPW * kDecodeWarps;   // keys per block step
  constexpr int kDPad = LPK * 8;
  __shared__ float sm_acc[kDecodeWarps][RC][kDPad];
  __shared__ float sm_m[kDecodeWarps][RC], sm_l[kDecodeWarps][RC];

  pdl_launch_dependents(); // the merge kernel may take free slots once every block of this grid runs
  const int split = blockIdx.x;
  const int chunk = blockIdx.y % p.chunks, hk = blockIdx.y / p.chunks;
  const int b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPK, kslot = warp * KPW + lane / LPK;
  const int e0 = sub * 8;
  const bool active = e0 < p.d;

  // lengths of this batch entry; a cache that would overflow keeps what fits
  const int n_new = p.knew ? p.seqlen_knew : 0;
  int cache_len = p.seqlens_k ? p.seqlens_k[b] : p.seqlen_k;
  cache_len = max(0, min(cache_len, p.seqlen_k));
  const int len = min(cache_len + n_new, p.seqlen_k);
  const int shift = len - p.seqlen_q;

  // the query rows of this block: row r = i * group + g  (query position i, head hk*group + g)
  const int r0 = chunk * RC;
  int qi[RC];
  bool valid[RC];
  float qf[RC][8];
  const T *qb = static_cast<const T *>(p.q) + (int64_t)b * p.q_bs;
#pragma unroll
  for (int t = 0; t < RC; ++t) {
    const int r = r0 + t;
    valid[t] = r < p.rows_per_kv;
    qi[t] = valid[t] ? r / p.group : 0;
    const int head = hk * p.group + (valid[t] ? r % p.group : 0);
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (valid[t] && active)
      raw = ld_nc_v4(qb + (int64_t)qi[t] * p.q_rs + (int64_t)head * p.q_hs + e0);
    unpack8<kBF16>(raw, qf[t]);
  }

  // keys any row of this block can see, cut into `splits` ranges of whole block steps
  const int i_min = r0 / p.group;
  const int i_max = min(r0 + RC - 1, p.rows_per_kv - 1) / p.group;
  const int lo = p.window_left >= 0 ? max(0, i_min + shift - p.window_left) : 0;
  const int hi = p.window_right >= 0 ? min(len, i_max + shift + p.window_right + 1) : len;
  const int span = max(hi - lo, 0);
  int per = (span + p.splits - 1) / p.splits;
  per = (per + KPB - 1) / KPB * KPB;
  const int j_begin = lo + split * per;
  const int j_end = min(hi, j_begin + per);

  float m[RC], l[RC], acc[RC][8];
#pragma unroll
  for (int t = 0; t < RC; ++t) {
    m[t] = -INFINITY;
    l[t] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e)
      acc[t][e] = 0.f;
  }

  T *kc = static_cast<T *>(p.kcache) + (int64_t)b * p.k_bs + (int64_t)hk * p.k_hs + e0;
  T *vc = static_cast<T *>(p.vcache) + (int64_t)b * p.v_bs + (int64_t)hk * p.v_hs + e0;
  const T *kn = static_cast<const T *>(p.knew) + (int64_t)b * p.kn_bs + (int64_t)hk * p.kn_hs + e0;
  const T *vn = static_cast<const T *>(p.vnew) + (int64_t)b * p.vn_bs + (int64_t)hk * p.vn_hs + e0;

  // append: the blocks of the first row chunk copy the new rows into the cache, all of them,
  // also those no query row of this block can see
  if (chunk == 0 && active) {
    for (int jn = split * KPB + kslot; jn < len - cache_len; jn += p.splits * KPB) {
      *reinterpret_cast<uint4 *>(kc + (int64_t)(cache_len + jn) * p.k_rs) = ld_nc_v4(kn + (int64_t)jn * p.kn_rs);
      *reinterpret_cast<uint4 *>(vc + (int64_t)(cache_len + jn) * p.v_rs) = ld_nc_v4(vn + (int64_t)jn * p.vn_rs);
    }
  }

  // the loads of the next step are issued before the arithmetic of the current one
  auto load_kv = [&](int j0, uint4 &kraw, uint4 &vraw) {
    const int j = j0 + kslot;
    kraw = vraw = make_uint4(0, 0, 0, 0);
    if (j < j_end && active) {
      if (j < cache_len) {
        kraw = ld_nc_v4(kc + (int64_t)j * p.k_rs);
        vraw = ld_nc_v4(vc + (int64_t)j * p.v_rs);
      } else { // a new row: read where it comes from, whether or not it is in the cache yet
        kraw = ld_nc_v4(kn + (int64_t)(j - cache_len) * p.kn_rs);
        vraw = ld_nc_v4(vn + (int64_t)(j - cache_len) * p.vn_rs);
      }
    }
  };
  uint4 kraw, vraw, knext, vnext;
  load_kv(j_begin, kraw, vraw);
  for (int j0 = j_begin; j0 < j_end; j0 += KPB, kraw = knext, vraw = vnext) {
    const int j = j0 + kslot;
    const bool have = j < j_end;
    load_kv(j0 + KPB, knext, vnext);
    float kf[8], vf[8];
    unpack8<kBF16>(kraw, kf);
    unpack8<kBF16>(vraw, vf);
#pragma unroll
    for (int t = 0; t < RC; ++t) {
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e)
        s = fmaf(qf[t][e], kf[e], s);
#pragma unroll
      for (int o = LPK / 2; o > 0; o >>= 1)
        s += __shfl_xor_sync(0xffffffffu, s, o);
      s *= p.scale_log2;
      bool visible = have && valid[t];
      if (p.window_right >= 0 && j > qi[t] + shift + p.window_right)
        visible = false;
      if (p.window_left >= 0 && j < qi[t] + shift - p.window_left)
        visible = false;
      if (visible) {
        if (s > m[t]) { // the running maximum grows: rescale what was accumulated
          const float alpha = scale_of(m[t], s);
          l[t] *= alpha;
#pragma unroll
          for (int e = 0; e < 8; ++e)
            acc[t][e] *= alpha;
          m[t] = s;
        }
        const float pr = exp2f(s - m[t]);
        l[t] += pr;
#pragma unroll
        for (int e = 0; e < 8; ++e)
          acc[t][e] = fmaf(pr, vf[e], acc[t][e]);
      }
    }
  }

  // merge the lane groups of the warp
#pragma unroll
  for (int t = 0; t < RC; ++t) {
#pragma unroll
    for (int off = LPK; off < 32; off <<= 1) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m[t], off);
      const float l_o = __shfl_xor_sync(0xffffffffu, l[t], off);
      const float m_n = fmaxf(m[t], m_o);
      const float a = scale_of(m[t], m_n), a_o = scale_of(m_o, m_n);
      l[t] = l[t] * a + l_o * a_o;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, acc[t][e], off);
        acc[t][e] = acc[t][e] * a + other * a_o;
      }
      m[t] = m_n;
    }
    if (lane < LPK) {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        sm_acc[warp][t][e0 + e] = acc[t][e];
      if (lane == 0) {
        sm_m[warp][t] = m[t];
        sm_l[warp][t] = l[t];
      }
    }
  }
  __syncthreads();

  // merge the warps; one thread per (row, element)
  for (int idx = threadIdx.x; idx < RC * p.d; idx += kDecodeThreads) {
    const int t = idx / p.d, e = idx % p.d;
    const int r = r0 + t;
    if (r >= p.rows_per_kv)
      continue;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w)
      mx = fmaxf(mx, sm_m[w][t]);
    float sum = 0.f, val = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float a = scale_of(sm_m[w][t], mx);
      sum += sm_l[w][t] * a;
      val += sm_acc[w][t][e] * a;
    }
    const int i = r / p.group, head = hk * p.group + r % p.group;
    const int64_t row = ((int64_t)b * p.h + head) * p.seqlen_q + i;
    if (p.splits == 1) {
      T *op = static_cast<T *>(p.o) + (int64_t)b * p.o_bs + (int64_t)i * p.o_rs + (int64_t)head * p.o_hs;
      op[e] = Elt<T>::from_f32(sum > 0.f ? val / sum : 0.f);
      if (e == 0) // a row that sees no key: output 0, LSE +inf, as the reference's kernel leaves it
        p.lse[row] = sum > 0.f ? mx * kLn2 + logf(sum) : INFINITY;
    } else {
      const int64_t slot = row * p.splits + split;
      p.part_o[slot * p.d + e] = val;
      if (e == 0) {
        p.part_ml[slot * 2] = mx;
        p.part_ml[slot * 2 + 1] = sum;
      }
    }
  }
}

// ---- head dims 64 and 128: the same split, scores and outputs on mma.sync tiles ----------------
// With grouped heads a block has up to 16 query rows per key, more multiply-adds than the scalar
// cores sustain at HBM speed; as one m16n8k16 tile they cost nothing.  Every warp walks its own
// 16-key tiles: K and V go from global memory straight into the B-operand registers, with no
// shared-memory stage, by permuting the contraction index: in S = Q K^T lane (g, c) of a quad
// contributes the 8 consecutive head-dim values [32 s + 8 c, +8) of key g to two k-steps, and Q's
// A fragments are loaded with the same permutation; in O = P V the lane takes the 8 consecutive
// output columns [64 hb + 8 g, +8) of its four keys, so that every load is one 16-byte vector
// and a warp reads whole 128-byte lines.  The output column of accumulator (n-tile t, logical
// column n) is 64 (t / 8) + 8 n + t % 8.  The vectors travel through a ring of cp.async stages
// in shared memory in which every thread owns the slots it later reads itself, so the ring
// needs no barrier: it only takes the loads of the next one or two tiles off the registers' hands.
template <bool kBF16>
__device__ __forceinline__ void mma16816(float (&acc)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kBF16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool kBF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBF16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
  } else {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
  }
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int w) {
  return w == 0 ? v.x : (w == 1 ? v.y : (w == 2 ? v.z : v.w));
}

__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void *src, bool real) {
  // bytes = 0: the 16 bytes are filled with zeros and src is not read.  The L2 hint pulls the rest of
  // the 256-byte row (or the neighbouring head's 128-byte row) into L2 with the first request.
  const int bytes = real ? 16 : 0;
  asm volatile("cp.async.cg.shared.global.L2::256B [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) { // 2^x; -inf gives 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t smem_addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_addr));
  return v;
}

constexpr int kMmaRows = 16;                   // query rows of one block
// tiles of the cp.async ring: the one in use and one (head dim 128) or two (64) in flight; measured:
// a third stage slows head dim 128 down (104 -> 117 us on a 512 MiB cache) and speeds 64 up (65 -> 59 us)
constexpr int mma_stages(int d) { return d == 128 ? 2 : 3; }
constexpr int kMmaWarps = 4;                   // up to three (head dim 128) or two (64) such blocks share an SM
constexpr int kMmaThreads = kMmaWarps * 32;
constexpr int kMmaKeysPerStep = 16 * kMmaWarps;

template <int D, bool kBF16>
__global__ void __launch_bounds__(kMmaThreads, D == 128 ? 3 : 2) decode_mma_kernel(const DecodeParams p) {
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  constexpr int NT = D / 8;  // output n-tiles
  constexpr int KS2 = D / 32; // pairs of k-steps of Q K^T
  constexpr int HB = D / 64;
  constexpr int NV = 2 * KS2 + 4 * HB; // 16-byte vectors of K and V a thread takes per tile
  constexpr int kMmaStages = mma_stages(D);
  extern __shared__ __align__(16) float decode_smem[];
  // ring: [stage][vector][thread] 16-byte slots; after the loop the same memory holds the merge buffers
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(decode_smem) + threadIdx.x * 16u;
  float *sm_acc = decode_smem;                                 // [warp][row][D]
  float *sm_m = decode_smem + kMmaWarps * kMmaRows * D;     // [warp][row]
  float *sm_l = sm_m + kMmaWarps * kMmaRows;

  pdl_launch_dependents(); // the merge kernel may take free slots once every block of this grid runs
  const int split = blockIdx.x;
  const int chunk = blockIdx.y % p.chunks, hk = blockIdx.y / p.chunks;
  const int b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;

  const int n_new = p.knew ? p.seqlen_knew : 0;
  int cache_len = p.seqlens_k ? p.seqlens_k[b] : p.seqlen_k;
  cache_len = max(0, min(cache_len, p.seqlen_k));
  const int len = min(cache_len + n_new, p.seqlen_k);
  const int shift = len - p.seqlen_q;

  // this lane's two query rows: r0 + g and r0 + g + 8
  const int r0 = chunk * kMmaRows;
  const int r_a = r0 + g, r_b = r0 + g + 8;
  const bool valid_a = r_a < p.rows_per_kv, valid_b = r_b < p.rows_per_kv;
  const int qi_a = valid_a ? r_a / p.group : 0, qi_b = valid_b ? r_b / p.group : 0;
  uint32_t qa[KS2][2][4];
  {
    const T *qb = static_cast<const T *>(p.q) + (int64_t)b * p.q_bs;
    const T *row_a = qb + (int64_t)qi_a * p.q_rs + (int64_t)(hk * p.group + (valid_a ? r_a % p.group : 0)) * p.q_hs;
    const T *row_b = qb + (int64_t)qi_b * p.q_rs + (int64_t)(hk * p.group + (valid_b ? r_b % p.group : 0)) * p.q_hs;
#pragma unroll
    for (int s2 = 0; s2 < KS2; ++s2) {
      const uint4 zero = make_uint4(0, 0, 0, 0);
      const uint4 va = valid_a ? ld_nc_v4(row_a + 32 * s2 + 8 * c) : zero;
      const uint4 vb = valid_b ? ld_nc_v4(row_b + 32 * s2 + 8 * c) : zero;
      qa[s2][0][0] = va.x, qa[s2][0][1] = vb.x, qa[s2][0][2] = va.y, qa[s2][0][3] = vb.y;
      qa[s2][1][0] = va.z, qa[s2][1][1] = vb.z, qa[s2][1][2] = va.w, qa[s2][1][3] = vb.w;
    }
  }

  const int i_min = r0 / p.group;
  const int i_max = min(r0 + kMmaRows - 1, p.rows_per_kv - 1) / p.group;
  const int lo = p.window_left >= 0 ? max(0, i_min + shift - p.window_left) : 0;
  const int hi = p.window_right >= 0 ? min(len, i_max + shift + p.window_right + 1) : len;
  const int span = max(hi - lo, 0);
  int per = (span + p.splits - 1) / p.splits;
  per = (per + kMmaKeysPerStep - 1) / kMmaKeysPerStep * kMmaKeysPerStep;
  const int j_begin = lo + split * per;
  const int j_end = min(hi, j_begin + per);

  T *kc = static_cast<T *>(p.kcache) + (int64_t)b * p.k_bs + (int64_t)hk * p.k_hs;
  T *vc = static_cast<T *>(p.vcache) + (int64_t)b * p.v_bs + (int64_t)hk * p.v_hs;
  const T *kn = static_cast<const T *>(p.knew) + (int64_t)b * p.kn_bs + (int64_t)hk * p.kn_hs;
  const T *vn = static_cast<const T *>(p.vnew) + (int64_t)b * p.vn_bs + (int64_t)hk * p.vn_hs;

  // append: the blocks of the first row chunk copy all new rows into the cache, 16 bytes a thread
  if (chunk == 0) {
    const int pieces = (len - cache_len) * (D / 8);
    for (int idx = split * kMmaThreads + (int)threadIdx.x; idx < pieces; idx += p.splits * kMmaThreads) {
      const int jn = idx / (D / 8), e = (idx % (D / 8)) * 8;
      *reinterpret_cast<uint4 *>(kc + (int64_t)(cache_len + jn) * p.k_rs + e) = ld_nc_v4(kn + (int64_t)jn * p.kn_rs + e);
      *reinterpret_cast<uint4 *>(vc + (int64_t)(cache_len + jn) * p.v_rs + e) = ld_nc_v4(vn + (int64_t)jn * p.vn_rs + e);
    }
  }

  // vectors of a tile: K of keys j0 + 8 nt + g, head-dim values [32 s2 + 8 c, +8)  (index nt * KS2 + s2);
  // V of keys j0 + 8 (ki / 2) + 2 c + ki % 2, columns [64 hb + 8 g, +8)  (index 2 KS2 + ki * HB + hb).
  // Tiles that lie wholly in the old part of the cache (all but the last few) take their row
  // addresses from running pointers; the others work them out row by row.
  const int j_first = j_begin + warp * 16;
  const T *kp[2], *vp[4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
    kp[nt] = kc + (int64_t)(j_first + 8 * nt + g) * p.k_rs + 8 * c;
#pragma unroll
  for (int ki = 0; ki < 4; ++ki)
    vp[ki] = vc + (int64_t)(j_first + 8 * (ki >> 1) + 2 * c + (ki & 1)) * p.v_rs + 8 * g;
  const int64_t k_step = (int64_t)kMmaKeysPerStep * p.k_rs, v_step = (int64_t)kMmaKeysPerStep * p.v_rs;
  const int plain_end = min(cache_len, j_end);
  auto issue_tile = [&](int j0, int stage) { // tiles are issued in order, one block step apart
    const uint32_t base = ring + (uint32_t)stage * (NV * kMmaThreads * 16);
    if (j0 + 16 <= plain_end) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int s2 = 0; s2 < KS2; ++s2)
          cp_async16(base + (nt * KS2 + s2) * (kMmaThreads * 16), kp[nt] + 32 * s2, true);
#pragma unroll
      for (int ki = 0; ki < 4; ++ki)
#pragma unroll
        for (int hb = 0; hb < HB; ++hb)
          cp_async16(base + (2 * KS2 + ki * HB + hb) * (kMmaThreads * 16), vp[ki] + 64 * hb, true);
    } else {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int j = j0 + 8 * nt + g;
        const bool real = j < j_end;
        const T *row = !real ? kc : (j < cache_len ? kc + (int64_t)j * p.k_rs : kn + (int64_t)(j - cache_len) * p.kn_rs);
#pragma unroll
        for (int s2 = 0; s2 < KS2; ++s2)
          cp_async16(base + (nt * KS2 + s2) * (kMmaThreads * 16), row + 32 * s2 + 8 * c, real);
      }
#pragma unroll
      for (int ki = 0; ki < 4; ++ki) {
        const int j = j0 + 8 * (ki >> 1) + 2 * c + (ki & 1);
        const bool real = j < j_end;
        const T *row = !real ? vc : (j < cache_len ? vc + (int64_t)j * p.v_rs : vn + (int64_t)(j - cache_len) * p.vn_rs);
#pragma unroll
        for (int hb = 0; hb < HB; ++hb)
          cp_async16(base + (2 * KS2 + ki * HB + hb) * (kMmaThreads * 16), row + 64 * hb + 8 * g, real);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
      kp[nt] += k_step;
#pragma unroll
    for (int ki = 0; ki < 4; ++ki)
      vp[ki] += v_step;
  };
  // tiles [j0, j0 + 16) inside [seen_lo, seen_hi) are visible to every row of the block: no masking
  const int seen_lo = p.window_left >= 0 ? i_max + shift - p.window_left : 0;
  const int seen_hi = min(j_end, p.window_right >= 0 ? i_min + shift + p.window_right + 1 : j_end);

  float o[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
    o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

  int j0 = j_first;
#pragma unroll
  for (int st = 0; st < kMmaStages - 1; ++st) { // one group per tile, empty past the end
    if (j0 + st * kMmaKeysPerStep < j_end)
      issue_tile(j0 + st * kMmaKeysPerStep, st);
    cp_async_commit();
  }
  for (int it = 0; j0 < j_end; j0 += kMmaKeysPerStep, ++it) {
    cp_async_wait<kMmaStages - 2>(); // this tile has landed
    {
      // the stage refilled here was read, by this thread, in the previous iteration
      const int j_ahead = j0 + (kMmaStages - 1) * kMmaKeysPerStep;
      if (j_ahead < j_end)
        issue_tile(j_ahead, (it + kMmaStages - 1) % kMmaStages);
      cp_async_commit();
    }
    const uint32_t base = ring + (uint32_t)(it % kMmaStages) * (NV * kMmaThreads * 16);
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int s2 = 0; s2 < KS2; ++s2) {
        const uint4 kv = lds_v4(base + (nt * KS2 + s2) * (kMmaThreads * 16));
        mma16816<kBF16>(s[nt], qa[s2][0], kv.x, kv.y);
        mma16816<kBF16>(s[nt], qa[s2][1], kv.z, kv.w);
      }
    }

    // s[nt][e]: key j0 + 8 nt + 2 c + (e & 1), row a for e < 2, row b otherwise
    if (j0 >= seen_lo && j0 + 16 <= seen_hi) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          s[nt][e] *= p.scale_log2;
    } else {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + 8 * nt + 2 * c + (e & 1);
          const int qi = e < 2 ? qi_a : qi_b;
          bool visible = j < j_end && (e < 2 ? valid_a : valid_b);
          if (p.window_right >= 0 && j > qi + shift + p.window_right)
            visible = false;
          if (p.window_left >= 0 && j < qi + shift - p.window_left)
            visible = false;
          s[nt][e] = visible ? s[nt][e] * p.scale_log2 : -INFINITY;
        }
    }
    float mx_a = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    float mx_b = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float new_a = fmaxf(m_a, mx_a), new_b = fmaxf(m_b, mx_b);
    if (__any_sync(0xffffffffu, new_a > m_a || new_b > m_b)) { // some row's maximum grew: rescale
      const float alpha_a = scale_of(m_a, new_a), alpha_b = scale_of(m_b, new_b);
      l_a *= alpha_a;
      l_b *= alpha_b;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        o[t][0] *= alpha_a, o[t][1] *= alpha_a;
        o[t][2] *= alpha_b, o[t][3] *= alpha_b;
      }
      m_a = new_a, m_b = new_b;
    }
    // a row that has seen nothing yet has only -inf scores: subtract 0 from them, not -inf
    const float sub_a = m_a == -INFINITY ? 0.f : m_a, sub_b = m_b == -INFINITY ? 0.f : m_b;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pr = ex2_approx(s[nt][e] - (e < 2 ? sub_a : sub_b));
        s[nt][e] = pr;
        if (e < 2)
          l_a += pr;
        else
          l_b += pr;
      }
    const uint32_t pa[4] = {pack2<kBF16>(s[0][0], s[0][1]), pack2<kBF16>(s[0][2], s[0][3]),
                            pack2<kBF16>(s[1][0], s[1][1]), pack2<kBF16>(s[1][2], s[1][3])};
#pragma unroll
    for (int hb = 0; hb < HB; ++hb) {
      uint4 vreg[4];
#pragma unroll
      for (int ki = 0; ki < 4; ++ki)
        vreg[ki] = lds_v4(base + (2 * KS2 + ki * HB + hb) * (kMmaThreads * 16));
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
        const uint32_t b0 = __byte_perm(word_of(vreg[0], e >> 1), word_of(vreg[1], e >> 1), sel);
        const uint32_t b1 = __byte_perm(word_of(vreg[2], e >> 1), word_of(vreg[3], e >> 1), sel);
        mma16816<kBF16>(o[hb * 8 + e], pa, b0, b1);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads(); // every warp is done with the ring: its memory becomes the merge buffers

  // the row sums are spread over the four lanes of a quad
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  float *acc_w = sm_acc + (size_t)warp * kMmaRows * D;
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const int col = 64 * (t / 8) + 16 * c + t % 8; // logical columns 2c and 2c+1 are 8 apart
    acc_w[g * D + col] = o[t][0];
    acc_w[g * D + col + 8] = o[t][1];
    acc_w[(g + 8) * D + col] = o[t][2];
    acc_w[(g + 8) * D + col + 8] = o[t][3];
  }
  if (c == 0) {
    sm_m[warp * kMmaRows + g] = m_a, sm_m[warp * kMmaRows + g + 8] = m_b;
    sm_l[warp * kMmaRows + g] = l_a, sm_l[warp * kMmaRows + g + 8] = l_b;
  }
  __syncthreads();

  // merge the warps; one thread per (row, element)
  for (int idx = threadIdx.x; idx < kMmaRows * D; idx += kMmaThreads) {
    const int t = idx / D, e = idx % D;
    const int r = r0 + t;
    if (r >= p.rows_per_kv)
      continue;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w)
      mx = fmaxf(mx, sm_m[w * kMmaRows + t]);
    float sum = 0.f, val = 0.f;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) {
      const float a = scale_of(sm_m[w * kMmaRows + t], mx);
      sum += sm_l[w * kMmaRows + t] * a;
      val += sm_acc[((size_t)w * kMmaRows + t) * D + e] * a;
    }
    const int i = r / p.group, head = hk * p.group + r % p.group;
    const int64_t row = ((int64_t)b * p.h + head) * p.seqlen_q + i;
    if (p.splits == 1) {
      T *op = static_cast<T *>(p.o) + (int64_t)b * p.o_bs + (int64_t)i * p.o_rs + (int64_t)head * p.o_hs;
      op[e] = Elt<T>::from_f32(sum > 0.f ? val / sum : 0.f);
      if (e == 0)
        p.lse[row] = sum > 0.f ? mx * kLn2 + logf(sum) : INFINITY;
    } else {
      const int64_t slot = row * p.splits + split;
      p.part_o[slot * p.d + e] = val;
      if (e == 0) {
        p.part_ml[slot * 2] = mx;
        p.part_ml[slot * 2 + 1] = sum;
      }
    }
  }
}

// one block per query row: merges the partial results of the splits.  Thread s takes split s's
// (max, sum), so those loads are one round trip; the output columns then read the splits eight
// at a time.
template <bool kBF16>
__global__ void __launch_bounds__(128) decode_merge_kernel(const DecodeParams p) {
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  static_assert(kMaxSplits <= 128, "one thread per split");
  __shared__ float weight[kMaxSplits];
  __shared__ float red[2][4];
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait(); // the partial results of the split kernel
  const int i = (int)(row % p.seqlen_q);
  const int head = (int)((row / p.seqlen_q) % p.h);
  const int b = (int)(row / ((int64_t)p.seqlen_q * p.h));
  const float2 ml = tid < p.splits ? reinterpret_cast<const float2 *>(p.part_ml)[row * p.splits + tid]
                                   : make_float2(-INFINITY, 0.f);
  float mx = ml.x;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0)
    red[0][warp] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red[0][0], red[0][1]), fmaxf(red[0][2], red[0][3]));
  const float w = scale_of(ml.x, mx);
  if (tid < p.splits)
    weight[tid] = w;
  float sum = ml.y * w;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0)
    red[1][warp] = sum;
  __syncthreads();
  const float total = red[1][0] + red[1][1] + red[1][2] + red[1][3];
  if (tid == 0)
    p.lse[row] = total > 0.f ? mx * kLn2 + logf(total) : INFINITY;
  const float inv = total > 0.f ? 1.f / total : 0.f;
  const float *po = p.part_o + row * p.splits * p.d;
  T *op = static_cast<T *>(p.o) + (int64_t)b * p.o_bs + (int64_t)i * p.o_rs + (int64_t)head * p.o_hs;
  for (int e = tid; e < p.d; e += blockDim.x) {
    float val = 0.f;
    for (int s0 = 0; s0 < p.splits; s0 += 8) {
      float part[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        part[u] = s0 + u < p.splits ? po[(int64_t)(s0 + u) * p.d + e] : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        val = fmaf(part[u], s0 + u < p.splits ? weight[s0 + u] : 0.f, val);
    }
    op[e] = Elt<T>::from_f32(val * inv);
  }
}

int g_splits_override = 0; // tuning door: a fixed number of key ranges per (batch, kv head, row chunk)

struct DecodePlan {
  bool mma; // head dim 64 or 128: the tensor-core kernel, 16 query rows a block
  int lpk, rc, chunks, splits;
  int64_t rows;
  size_t workspace_bytes;
};

bool strides_ok(const b200_flash_kvcache_params &p) {
  const int64_t s[] = {p.q_batch_stride,  p.k_batch_stride,    p.v_batch_stride,    p.knew_batch_stride,
                       p.vnew_batch_stride, p.o_batch_stride,  p.q_row_stride,      p.k_row_stride,
                       p.v_row_stride,    p.knew_row_stride,   p.vnew_row_stride,   p.o_row_stride,
                       p.q_head_stride,   p.k_head_stride,     p.v_head_stride,     p.knew_head_stride,
                       p.vnew_head_stride, p.o_head_stride};
  for (int64_t v : s)
    if (v < 0)
      return false;
  return true;
}

// a pure function of the shapes, so the workspace size is known without a device
int make_plan(const b200_flash_kvcache_params &p, DecodePlan *plan) {
  if (p.b <= 0 || p.h <= 0 || p.h_k <= 0 || p.h % p.h_k != 0 || p.seqlen_q <= 0 || p.seqlen_k <= 0 || p.seqlen_knew < 0)
    return B200_ERR_INVALID_ARG;
  if (p.d <= 0 || p.d > 256 || p.d % 8 != 0)
    return B200_ERR_UNSUPPORTED;
  if (!strides_ok(p))
    return B200_ERR_INVALID_ARG;
  const int64_t group = p.h / p.h_k;
  const int64_t rows_per_kv = p.seqlen_q * group;
  plan->mma = p.d == 64 || p.d == 128;
  plan->lpk = std::max(4, pow2_ceil(p.d / 8));
  plan->rc = plan->mma ? kMmaRows : (rows_per_kv >= 4 ? 4 : (rows_per_kv >= 2 ? 2 : 1));
  plan->chunks = (int)ceil_div<int64_t>(rows_per_kv, plan->rc);
  if ((int64_t)plan->chunks * p.h_k > 65535 || p.b > 65535)
    return B200_ERR_UNSUPPORTED;
  const int64_t keys_per_step = plan->mma ? kMmaKeysPerStep : (int64_t)kDecodeWarps * 32 / plan->lpk;
  const int64_t base = p.b * p.h_k * plan->chunks;
  // Measured: the tensor-core kernel streams fastest as ONE wave of at most two blocks per SM
  // (a block keeps a fixed number of bytes in flight, and a ragged second wave costs more than
  // the idle slots of a first one); when (batch, kv head, row chunk) alone exceed that, and for
  // the scalar kernel, about four blocks per SM, taking among the counts up to twice that the
  // one whose last wave is fullest.  Every range keeps at least four block steps of keys.
  const int64_t slots = (int64_t)kNumSMs * (plan->mma ? 3 : 4); // blocks the GPU holds at a time
  const int64_t room = std::max<int64_t>(1, p.seqlen_k / (4 * keys_per_step));
  const int64_t cap = std::min<int64_t>(room, kMaxSplits);
  int64_t best;
  if (plan->mma && base <= 2 * kNumSMs) {
    best = std::min<int64_t>(cap, 2 * kNumSMs / base);
  } else {
    const int64_t want = std::min<int64_t>(cap, ceil_div<int64_t>((int64_t)kNumSMs * 4, base));
    best = want;
    double best_fill = 0.0;
    for (int64_t n = want; n <= std::min<int64_t>(cap, 2 * want); ++n) {
      const double fill = (double)(base * n) / (double)(ceil_div<int64_t>(base * n, slots) * slots);
      if (fill > best_fill + 1e-9)
        best = n, best_fill = fill;
    }
  }
  plan->splits = (int)std::max<int64_t>(1, best);
  if (g_splits_override > 0)
    plan->splits = (int)std::min<int64_t>(g_splits_override, cap);
  plan->rows = p.b * p.h * p.seqlen_q;
  plan->workspace_bytes =
      plan->splits > 1 ? (size_t)plan->rows * plan->splits * ((size_t)p.d + 2) * sizeof(float) : 0;
  return B200_OK;
}

template <int LPK, bool kBF16> int launch_split(const DecodeParams &dp, int rc, dim3 grid, cudaStream_t stream) {
  switch (rc) {
  case 1:
    decode_split_kernel<LPK, 1, kBF16><<<grid, kDecodeThreads, 0, stream>>>(dp);
    break;
  case 2:
    decode_split_kernel<LPK, 2, kBF16><<<grid, kDecodeThreads, 0, stream>>>(dp);
    break;
  default:
    decode_split_kernel<LPK, 4, kBF16><<<grid, kDecodeThreads, 0, stream>>>(dp);
  }
  return check_launch();
}

template <bool kBF16> int launch_decode(const DecodeParams &dp, const DecodePlan &plan, cudaStream_t stream) {
  const dim3 grid((unsigned)plan.splits, (unsigned)(plan.chunks * dp.h_k), (unsigned)dp.b);
  int rc;
  if (plan.mma) {
    // the cp.async ring (16 bytes x d/8 vectors x 128 threads a stage); the merge buffers reuse it
    const size_t ring = (size_t)mma_stages(dp.d) * (dp.d / 8) * kMmaThreads * 16;
    const size_t smem = std::max(ring, ((size_t)kMmaWarps * kMmaRows * (dp.d + 2)) * sizeof(float));
    auto kernel = dp.d == 128 ? decode_mma_kernel<128, kBF16> : decode_mma_kernel<64, kBF16>;
    // the attribute belongs to the current device's context: set it on every call
    if (int e = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)))
      return e;
    kernel<<<grid, kMmaThreads, smem, stream>>>(dp);
    rc = check_launch();
  } else
  switch (plan.lpk) {
  case 4:
    rc = launch_split<4, kBF16>(dp, plan.rc, grid, stream);
    break;
  case 8:
    rc = launch_split<8, kBF16>(dp, plan.rc, grid, stream);
    break;
  case 16:
    rc = launch_split<16, kBF16>(dp, plan.rc, grid, stream);
    break;
  default:
    rc = launch_split<32, kBF16>(dp, plan.rc, grid, stream);
  }
  if (rc != B200_OK || plan.splits == 1)
    return rc;
  // launched while the split kernel's last wave still runs; it waits for that grid before it reads
  return launch_pdl(decode_merge_kernel<kBF16>, dim3((unsigned)plan.rows), dim3(128), 0, stream, dp);
}

} // namespace
} // namespace b200

using namespace b200;

// not in the header: fixes the number of key ranges (0 = automatic), for tuning runs
extern "C" void b200_flash_attn_kvcache_tune(int splits) { g_splits_override = splits; }

extern "C" int64_t b200_flash_attn_kvcache_workspace_bytes(const b200_flash_kvcache_params *params) {
  DecodePlan plan;
  if (!params || make_plan(*params, &plan) != B200_OK)
    return -1;
  return (int64_t)plan.workspace_bytes;
}

extern "C" int b200_flash_attn_kvcache(int dtype, const void *q, void *kcache, void *vcache, const void *knew,
                                       const void *vnew, const int32_t *seqlens_k, void *out, float *softmax_lse,
                                       const b200_flash_kvcache_params *params, void *workspace,
                                       size_t workspace_bytes, cudaStream_t stream) {
  if (!params || !q || !kcache || !vcache || !out || !softmax_lse)
    return B200_ERR_INVALID_ARG;
  if (dtype != B200_F16 && dtype != B200_BF16)
    return B200_ERR_UNSUPPORTED;
  const b200_flash_kvcache_params &p = *params;
  DecodePlan plan;
  if (int rc = make_plan(p, &plan))
    return rc;
  const bool has_new = knew != nullptr && vnew != nullptr && p.seqlen_knew > 0;
  if ((knew != nullptr) != (vnew != nullptr))
    return B200_ERR_INVALID_ARG;
  // rows are read and written as 16-byte vectors
  const int64_t vec_strides[] = {p.q_batch_stride, p.q_row_stride, p.q_head_stride, p.k_batch_stride, p.k_row_stride,
                                 p.k_head_stride,  p.v_batch_stride, p.v_row_stride, p.v_head_stride};
  for (int64_t s : vec_strides)
    if (s % 8 != 0)
      return B200_ERR_ALIGNMENT;
  if (!aligned16(q) || !aligned16(kcache) || !aligned16(vcache))
    return B200_ERR_ALIGNMENT;
  if (has_new) {
    const int64_t new_strides[] = {p.knew_batch_stride, p.knew_row_stride, p.knew_head_stride,
                                   p.vnew_batch_stride, p.vnew_row_stride, p.vnew_head_stride};
    for (int64_t s : new_strides)
      if (s % 8 != 0)
        return B200_ERR_ALIGNMENT;
    if (!aligned16(knew) || !aligned16(vnew))
      return B200_ERR_ALIGNMENT;
  }
  if (reinterpret_cast<uintptr_t>(out) % 2 != 0 || reinterpret_cast<uintptr_t>(softmax_lse) % 4 != 0)
    return B200_ERR_ALIGNMENT;

  DecodeParams dp{};
  dp.q = q;
  dp.kcache = kcache;
  dp.vcache = vcache;
  dp.knew = has_new ? knew : nullptr;
  dp.vnew = has_new ? vnew : nullptr;
  dp.seqlens_k = seqlens_k;
  dp.o = out;
  dp.lse = softmax_lse;
  dp.q_bs = p.q_batch_stride, dp.k_bs = p.k_batch_stride, dp.v_bs = p.v_batch_stride;
  dp.kn_bs = p.knew_batch_stride, dp.vn_bs = p.vnew_batch_stride, dp.o_bs = p.o_batch_stride;
  dp.q_rs = p.q_row_stride, dp.k_rs = p.k_row_stride, dp.v_rs = p.v_row_stride;
  dp.kn_rs = p.knew_row_stride, dp.vn_rs = p.vnew_row_stride, dp.o_rs = p.o_row_stride;
  dp.q_hs = p.q_head_stride, dp.k_hs = p.k_head_stride, dp.v_hs = p.v_head_stride;
  dp.kn_hs = p.knew_head_stride, dp.vn_hs = p.vnew_head_stride, dp.o_hs = p.o_head_stride;
  dp.b = (int)p.b, dp.h = (int)p.h, dp.h_k = (int)p.h_k, dp.d = (int)p.d, dp.group = (int)(p.h / p.h_k);
  dp.seqlen_q = (int)p.seqlen_q, dp.seqlen_k = (int)p.seqlen_k, dp.seqlen_knew = has_new ? (int)p.seqlen_knew : 0;
  dp.window_left = (int)p.window_size_left, dp.window_right = (int)p.window_size_right;
  dp.splits = plan.splits, dp.chunks = plan.chunks, dp.rows_per_kv = (int)(p.seqlen_q * (p.h / p.h_k));
  dp.scale_log2 = p.softmax_scale * kLog2e;

  void *owned = nullptr;
  if (plan.workspace_bytes > 0) {
    if (workspace) {
      if (workspace_bytes < plan.workspace_bytes || !aligned16(workspace))
        return B200_ERR_WORKSPACE;
    } else { // the custom-call ABI has no workspace operand: take it from the stream's pool
      if (int rc = check_cuda(cudaMallocAsync(&owned, plan.workspace_bytes, stream)))
        return rc;
      workspace = owned;
    }
    dp.part_o = static_cast<float *>(workspace);
    dp.part_ml = dp.part_o + (size_t)plan.rows * plan.splits * (size_t)p.d;
  }
  const int rc = dtype == B200_BF16 ? launch_decode<true>(dp, plan, stream) : launch_decode<false>(dp, plan, stream);
  if (owned) {
    const int rc_free = check_cuda(cudaFreeAsync(owned, stream));
    return rc != B200_OK ? rc : rc_free;
  }
  return rc;
}
