// ReduceSumOp / ReduceMaxOp for sm_100a.
//
// The tensor is viewed as A x B x C (row-major) and B is reduced, as the
// reference does (reduction/reduce_impl.h:28-59).  Both shapes of the problem
// are bound by HBM bandwidth, so every path is built around 128-bit coalesced
// streaming loads with several loads in flight per thread:
//
//   C == 1  ("rows"):    a group of 1..256 threads owns one row (or one segment
//                        of a long row); warp shuffles, then shared memory,
//                        combine the group.  Long rows with few rows in total are
//                        cut into segments: up to 8 segments are combined inside
//                        one thread-block cluster through distributed shared
//                        memory (single launch, no workspace); more segments go
//                        through f32 partials in the workspace and a second pass.
//   C  > 1  ("columns"): a warp reads one (or several short) contiguous rows of a
//                        column slab per step, 8 warps stride over the B rows,
//                        and B is split over enough blocks to fill 148 SMs
//                        (split-K); the f32 partials of the splits are combined in
//                        split order by a second pass, so the result does not
//                        depend on scheduling.  (Folding in the first launch - the
//                        last block of a slab to finish, found by a ticket, folds
//                        it - was measured slower: 14.4 against 13.6 us on f16
//                        [32768, 1024], because the fence, the ticket and the fold
//                        are one more latency chain after the last load, while
//                        the second pass is already resident and waiting.)
//
// Max semantics (reduction_helper.h:159-180 folded in ascending index order):
// NaN wins; otherwise the largest value; between +0 and -0, which compare equal,
// the one at the higher index.  The streaming pass uses the hardware max (which
// ranks -0 below +0); only a result that is exactly zero triggers a short
// backward scan for the last zero of the range to fix the sign.
#include <cooperative_groups.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kSum = B200_REDUCE_SUM;
constexpr int kMax = B200_REDUCE_MAX;
constexpr int kBlock = 256;
constexpr int kFinalizeBlock = 1024; // second pass: 32 outputs x 32 slices

__device__ __forceinline__ float max_nan_f32(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

template <int OP> __device__ __forceinline__ float op_init() {
  return OP == kSum ? 0.f : -INFINITY;
}
// order-insensitive combine of two partial results (zero signs fixed up later)
template <int OP> __device__ __forceinline__ float op_combine(float a, float b) {
  return OP == kSum ? a + b : max_nan_f32(a, b);
}
// the reference's apply(lhs, rhs) with lhs covering the lower indices
template <int OP> __device__ __forceinline__ float op_apply_ordered(float lhs, float rhs) {
  if (OP == kSum)
    return lhs + rhs;
  return (isnan(lhs) || lhs > rhs) ? lhs : rhs;
}

// ---- per-thread accumulators over 16-byte vectors --------------------------
template <typename T, int OP> struct Acc;

template <> struct Acc<float, kSum> {
  float a = 0.f, b = 0.f;
  __device__ __forceinline__ void vec(uint4 v) {
    a += __uint_as_float(v.x);
    b += __uint_as_float(v.y);
    a += __uint_as_float(v.z);
    b += __uint_as_float(v.w);
  }
  __device__ __forceinline__ void one(float v) { a += v; }
  __device__ __forceinline__ float get() const { return a + b; }
};
template <> struct Acc<float, kMax> {
  float m = -INFINITY;
  __device__ __forceinline__ void vec(uint4 v) {
    m = max_nan_f32(m, max_nan_f32(max_nan_f32(__uint_as_float(v.x), __uint_as_float(v.y)),
                                   max_nan_f32(__uint_as_float(v.z), __uint_as_float(v.w))));
  }
  __device__ __forceinline__ void one(float v) { m = max_nan_f32(m, v); }
  __device__ __forceinline__ float get() const { return m; }
};
template <> struct Acc<__half, kSum> {
  float a = 0.f, b = 0.f;
  __device__ __forceinline__ void word(uint32_t w) {
    float2 f = __half22float2(*reinterpret_cast<__half2 *>(&w));
    a += f.x;
    b += f.y;
  }
  __device__ __forceinline__ void vec(uint4 v) {
    word(v.x), word(v.y), word(v.z), word(v.w);
  }
  __device__ __forceinline__ void one(__half v) { a += __half2float(v); }
  __device__ __forceinline__ float get() const { return a + b; }
};
template <> struct Acc<__nv_bfloat16, kSum> {
  float a = 0.f, b = 0.f;
  __device__ __forceinline__ void word(uint32_t w) {
    a += __uint_as_float(w << 16);
    b += __uint_as_float(w & 0xffff0000u);
  }
  __device__ __forceinline__ void vec(uint4 v) {
    word(v.x), word(v.y), word(v.z), word(v.w);
  }
  __device__ __forceinline__ void one(__nv_bfloat16 v) { a += __bfloat162float(v); }
  __device__ __forceinline__ float get() const { return a + b; }
};
template <> struct Acc<__half, kMax> {
  __half2 m = __half2half2(__ushort_as_half((unsigned short)0xfc00)); // -inf
  __device__ __forceinline__ void word(uint32_t w) {
    m = __hmax2_nan(m, *reinterpret_cast<__half2 *>(&w));
  }
  __device__ __forceinline__ void vec(uint4 v) {
    word(v.x), word(v.y), word(v.z), word(v.w);
  }
  __device__ __forceinline__ void one(__half v) { m = __hmax2_nan(m, __half2half2(v)); }
  __device__ __forceinline__ float get() const {
    return max_nan_f32(__low2float(m), __high2float(m));
  }
};
template <> struct Acc<__nv_bfloat16, kMax> {
  __nv_bfloat162 m = __bfloat162bfloat162(__ushort_as_bfloat16((unsigned short)0xff80)); // -inf
  __device__ __forceinline__ void word(uint32_t w) {
    m = __hmax2_nan(m, *reinterpret_cast<__nv_bfloat162 *>(&w));
  }
  __device__ __forceinline__ void vec(uint4 v) {
    word(v.x), word(v.y), word(v.z), word(v.w);
  }
  __device__ __forceinline__ void one(__nv_bfloat16 v) {
    m = __hmax2_nan(m, __bfloat162bfloat162(v));
  }
  __device__ __forceinline__ float get() const {
    return max_nan_f32(__low2float(m), __high2float(m));
  }
};

template <typename OutT> __device__ __forceinline__ void store_out(OutT *p, float v) {
  *p = Elt<OutT>::from_f32(v);
}

// =============================================================================
// rows: C == 1
// =============================================================================
// Grid: one group of `tpr` threads per (row, segment); kBlock / tpr groups per
// block.  kCluster: the `segs` blocks of a row form one cluster (tpr == kBlock).
template <typename T, int OP, bool VEC, bool kCluster, typename OutT>
__global__ void __launch_bounds__(kBlock)
    reduce_rows_kernel(const T *__restrict__ in, OutT *__restrict__ out,
                       float *__restrict__ partial, int64_t A, int64_t B, int tpr,
                       int segs, int64_t seg_len) {
  constexpr int N = 16 / sizeof(T);
  __shared__ float warp_part[kBlock / 32];
  __shared__ float cluster_part;
  pdl_launch_dependents();

  const int groups_per_block = kBlock / tpr;
  const int64_t g = (int64_t)blockIdx.x * groups_per_block + threadIdx.x / tpr;
  const int t = threadIdx.x % tpr;
  const int64_t a = g / segs;
  const int s = (int)(g % segs);
  const bool active = a < A;
  const int64_t e0 = (int64_t)s * seg_len;
  const int64_t e1 = active ? min(B, e0 + seg_len) : e0;
  const T *row = in + (active ? a : 0) * B;

  if (VEC) { // the first loads, on their way into L2 while the kernel in front of this one ends
    const uint4 *vp = reinterpret_cast<const uint4 *>(row + e0);
    const int64_t nvec = (e1 - e0) / N;
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (t + (int64_t)k * tpr < nvec)
        prefetch_l2(vp + t + (int64_t)k * tpr);
  }
  pdl_wait();
  Acc<T, OP> acc;
  if (VEC) {
    const uint4 *vp = reinterpret_cast<const uint4 *>(row + e0);
    const int64_t nvec = (e1 - e0) / N;
    int64_t v = t;
    for (; v + 3 * (int64_t)tpr < nvec; v += 4 * (int64_t)tpr) {
      uint4 x0 = ld_nc_v4(vp + v);
      uint4 x1 = ld_nc_v4(vp + v + tpr);
      uint4 x2 = ld_nc_v4(vp + v + 2 * tpr);
      uint4 x3 = ld_nc_v4(vp + v + 3 * tpr);
      acc.vec(x0), acc.vec(x1), acc.vec(x2), acc.vec(x3);
    }
    for (; v < nvec; v += tpr)
      acc.vec(ld_nc_v4(vp + v));
    for (int64_t e = e0 + nvec * N + t; e < e1; e += tpr)
      acc.one(row[e]);
  } else {
    for (int64_t e = e0 + t; e < e1; e += tpr)
      acc.one(row[e]);
  }
  float r = acc.get();

  // combine the group; every thread of the group ends up with the result
  const int width = tpr < 32 ? tpr : 32;
  for (int off = width >> 1; off > 0; off >>= 1)
    r = op_combine<OP>(r, __shfl_xor_sync(0xffffffffu, r, off));
  if (tpr > 32) {
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0)
      warp_part[warp] = r;
    __syncthreads();
    const int w0 = (threadIdx.x / tpr) * (tpr >> 5);
    r = warp_part[w0];
    for (int w = 1; w < (tpr >> 5); ++w)
      r = op_combine<OP>(r, warp_part[w0 + w]);
  }

  // max == 0: the sign is that of the last zero of the range
  if (OP == kMax && active && r == 0.f) {
    const int lanes = width; // the first `width` threads of the group scan backwards
    const unsigned gmask =
        tpr >= 32 ? 0xffffffffu : (((1u << tpr) - 1u) << ((threadIdx.x & 31) / tpr * tpr));
    if (t < lanes) {
      float found = 0.f;
      for (int64_t hi = e1; hi > e0; hi -= lanes) {
        const int64_t e = hi - 1 - t;
        const float v = e >= e0 ? Elt<T>::to_f32(row[e]) : 1.f;
        const unsigned hit = __ballot_sync(gmask, v == 0.f);
        if (hit) {
          // lowest t = highest index
          const int src = __ffs(hit) - 1;
          found = __shfl_sync(gmask, v, src);
          break;
        }
      }
      r = found; // thread t == 0, which writes the result, is one of the scanners
    }
  }

  if (kCluster) {
    cg::cluster_group cluster = cg::this_cluster();
    if (threadIdx.x == 0)
      cluster_part = r;
    cluster.sync();
    if (cluster.block_rank() == 0 && threadIdx.x == 0) {
      float total = r;
      for (int k = 1; k < segs; ++k)
        total = op_apply_ordered<OP>(total, *cluster.map_shared_rank(&cluster_part, k));
      store_out(out + a, total);
    }
    cluster.sync(); // keep every block's shared memory alive until rank 0 has read it
    return;
  }
  if (active && t == 0) {
    if (segs == 1)
      store_out(out + a, r);
    else
      partial[a * segs + s] = r;
  }
}

// Short rows (a row is at most VPT 16-byte vectors per thread of its group):
// persistent blocks walk over the rows, and the loads of the next row are issued
// before the current one is reduced, so that every thread keeps VPT..2*VPT loads
// in flight across row boundaries.
template <typename T, int OP, int VPT, typename OutT>
__global__ void __launch_bounds__(kBlock)
    reduce_short_rows_kernel(const T *__restrict__ in, OutT *__restrict__ out, int64_t A, int64_t B,
                             int tpr, int prefetch) {
  constexpr int N = 16 / sizeof(T);
  __shared__ float warp_part[2][kBlock / 32];
  pdl_launch_dependents();
  const int groups_per_block = kBlock / tpr;
  const int t = threadIdx.x % tpr;
  const int gib = threadIdx.x / tpr;
  const int nvec = (int)(B / N);
  const int64_t block_rows = groups_per_block;
  const int64_t iters = ceil_div<int64_t>(ceil_div<int64_t>(A, block_rows) - blockIdx.x, (int64_t)gridDim.x);
  const int width = tpr < 32 ? tpr : 32;

  uint4 cur[VPT], nxt[VPT];
  auto load_row = [&](int64_t a, uint4(&v)[VPT]) {
    const uint4 *vp = reinterpret_cast<const uint4 *>(in + a * B);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int idx = t + k * tpr;
      if (a < A && idx < nvec)
        v[k] = ld_nc_v4(vp + idx);
    }
  };
  int64_t a = (int64_t)blockIdx.x * block_rows + gib;
  // the loads of the first `prefetch` rows of this group, on their way into L2 during the wait
  for (int64_t ap = a, k = 0; k < prefetch && ap < A; ++k, ap += (int64_t)gridDim.x * block_rows) {
    const uint4 *vp = reinterpret_cast<const uint4 *>(in + ap * B);
#pragma unroll
    for (int k2 = 0; k2 < VPT; ++k2)
      if (t + k2 * tpr < nvec)
        prefetch_l2(vp + t + k2 * tpr);
  }
  pdl_wait();
  load_row(a, cur);
  for (int64_t it = 0; it < iters; ++it) {
    const int64_t a_next = a + (int64_t)gridDim.x * block_rows;
    if (it + 1 < iters)
      load_row(a_next, nxt);
    const bool active = a < A;
    Acc<T, OP> acc;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
      if (active && t + k * tpr < nvec)
        acc.vec(cur[k]);
    float r = acc.get();
    for (int off = width >> 1; off > 0; off >>= 1)
      r = op_combine<OP>(r, __shfl_xor_sync(0xffffffffu, r, off));
    if (tpr > 32) {
      float *wp = warp_part[it & 1];
      if ((threadIdx.x & 31) == 0)
        wp[threadIdx.x >> 5] = r;
      __syncthreads();
      const int w0 = gib * (tpr >> 5);
      r = wp[w0];
      for (int w = 1; w < (tpr >> 5); ++w)
        r = op_combine<OP>(r, wp[w0 + w]);
    }
    if (OP == kMax && active && r == 0.f) { // sign of the last zero of the row
      const unsigned gmask =
          tpr >= 32 ? 0xffffffffu : (((1u << tpr) - 1u) << ((threadIdx.x & 31) / tpr * tpr));
      if (t < width) {
        const T *row = in + a * B;
        float found = 0.f;
        for (int64_t hi = B; hi > 0; hi -= width) {
          const int64_t e = hi - 1 - t;
          const float v = e >= 0 ? Elt<T>::to_f32(row[e]) : 1.f;
          const unsigned hit = __ballot_sync(gmask, v == 0.f);
          if (hit) {
            found = __shfl_sync(gmask, v, __ffs(hit) - 1);
            break;
          }
        }
        r = found;
      }
    }
    if (active && t == 0)
      store_out(out + a, r);
#pragma unroll
    for (int k = 0; k < VPT; ++k)
      cur[k] = nxt[k];
    a = a_next;
  }
}

// =============================================================================
// columns: C > 1
// =============================================================================
// NV = elements per lane per load (16 / sizeof(T) when 16-byte loads are
// possible, else 1).  A warp covers `rpw = 32 / lpr` rows of a slab of
// lpr * NV columns per step; 8 warps stride over the rows of this block's split.
template <typename T, int OP, int NV, typename OutT>
__global__ void __launch_bounds__(kBlock, 4)
    reduce_cols_kernel(const T *__restrict__ in, OutT *__restrict__ out, float *partial,
                       int64_t A, int64_t B, int64_t C, int lpr, int slabs, int splits,
                       int64_t rows_per_split, int prefetch) {
  __shared__ float smem[kBlock * NV]; // [row lane][column of the slab]
  pdl_launch_dependents(); // lets the next kernel (the second pass) be scheduled while this one runs

  const int64_t bid = blockIdx.x;
  const int slab = (int)(bid % slabs);
  const int64_t rest = bid / slabs;
  const int split = (int)(rest % splits);
  const int64_t a = rest / splits;
  // `lpr` threads cover one row of the slab (16 bytes each); kBlock / lpr rows per step
  const int row_lanes = kBlock / lpr;
  const int lane_col = threadIdx.x % lpr, lane_row = threadIdx.x / lpr;
  const int64_t slab_col0 = (int64_t)slab * lpr * NV;
  const int64_t col0 = slab_col0 + (int64_t)lane_col * NV;
  const bool col_ok = col0 < C; // C % NV == 0, so a thread is all-in or all-out
  const int64_t r0 = (int64_t)split * rows_per_split;
  const int64_t r1 = min(B, r0 + rows_per_split);
  const T *base = in + a * B * C + col0;
  const int64_t step = row_lanes;
  if (col_ok) { // the first `prefetch` batches of this thread's loads, on their way into L2 during the wait
    for (int64_t r = r0 + lane_row, k = 0; k < prefetch && r < r1; ++k, r += 8 * step) {
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (r + u * step < r1)
          prefetch_l2(base + (r + u * step) * C);
    }
  }
  pdl_wait(); // inputs may come from the kernel launched just before this one

  float acc[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j)
    acc[j] = op_init<OP>();

  auto consume = [&](const uint4 &v) {
    if constexpr (NV == 1) {
      // unused
    } else if constexpr (sizeof(T) == 4) {
      acc[0] = op_combine<OP>(acc[0], __uint_as_float(v.x));
      acc[1] = op_combine<OP>(acc[1], __uint_as_float(v.y));
      acc[2] = op_combine<OP>(acc[2], __uint_as_float(v.z));
      acc[3] = op_combine<OP>(acc[3], __uint_as_float(v.w));
    } else {
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float lo, hi;
        if constexpr (std::is_same<T, __half>::value) {
          float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
          lo = f.x, hi = f.y;
        } else {
          lo = __uint_as_float(w[k] << 16);
          hi = __uint_as_float(w[k] & 0xffff0000u);
        }
        acc[2 * k] = op_combine<OP>(acc[2 * k], lo);
        acc[2 * k + 1] = op_combine<OP>(acc[2 * k + 1], hi);
      }
    }
  };

  if (col_ok) {
    int64_t r = r0 + lane_row;
    if constexpr (NV > 1) {
      // 8 loads in flight per thread; the last, partial batch is predicated rather than
      // handled load by load, so the tail does not pay one memory latency per row
      for (; r < r1; r += 8 * step) {
        uint4 x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (r + u * step < r1)
            x[u] = ld_nc_v4(base + (r + u * step) * C);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (r + u * step < r1)
            consume(x[u]);
      }
    } else {
      for (; r + 3 * step < r1; r += 4 * step) {
        float x0 = Elt<T>::to_f32(base[r * C]);
        float x1 = Elt<T>::to_f32(base[(r + step) * C]);
        float x2 = Elt<T>::to_f32(base[(r + 2 * step) * C]);
        float x3 = Elt<T>::to_f32(base[(r + 3 * step) * C]);
        acc[0] = op_combine<OP>(op_combine<OP>(acc[0], x0), op_combine<OP>(x1, op_combine<OP>(x2, x3)));
      }
      for (; r < r1; r += step)
        acc[0] = op_combine<OP>(acc[0], Elt<T>::to_f32(base[r * C]));
    }
  }
#pragma unroll
  for (int j = 0; j < NV; ++j)
    smem[(lane_row * lpr + lane_col) * NV + j] = acc[j];
  __syncthreads();
  const int ncols = lpr * NV;
  for (int j = threadIdx.x; j < ncols; j += kBlock) {
    const int64_t col = slab_col0 + j;
    if (col >= C)
      continue;
    float r = smem[j];
    for (int w = 1; w < row_lanes; ++w)
      r = op_combine<OP>(r, smem[w * ncols + j]);
    if (OP == kMax && r == 0.f) { // sign of the last zero in [r0, r1)
      const T *colp = in + a * B * C + col;
      for (int64_t rr = r1 - 1; rr >= r0; --rr) {
        const float v = Elt<T>::to_f32(colp[rr * C]);
        if (v == 0.f) {
          r = v;
          break;
        }
      }
    }
    if (splits == 1)
      store_out(out + a * C + col, r);
    else
      partial[((int64_t)split * A + a) * C + col] = r;
  }
}

// second pass: out[i] = fold over s of partial[i * stride_i + s * stride_s].
// 32 outputs per block; 32 warps each fold a contiguous slice of the `count`
// partials with 8 loads in flight, then warp 0 folds the slice results in order.
// (The second pass is a latency chain, not a bandwidth problem: with 8 warps and 4
// loads in flight it took a third as long as the first pass over 64 MB.)
template <int OP, typename OutT>
__global__ void __launch_bounds__(kFinalizeBlock)
    reduce_finalize_kernel(const float *__restrict__ partial, OutT *__restrict__ out,
                           int64_t n, int count, int64_t stride_i, int64_t stride_s) {
  __shared__ float sm[kFinalizeBlock / 32][32];
  pdl_wait(); // the partials come from the kernel launched just before this one
  pdl_launch_dependents();
  constexpr int kSlices = kFinalizeBlock / 32;
  const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int64_t i = (int64_t)blockIdx.x * 32 + lane;
  const int per = (count + kSlices - 1) / kSlices;
  const int s0 = slice * per, s1 = min(count, s0 + per);
  float r = 0.f;
  if (i < n && s0 < s1) {
    const float *p = partial + i * stride_i;
    r = p[s0 * stride_s];
    // batches of eight loads in flight, the last one predicated: one memory latency per batch
    for (int s = s0 + 1; s < s1; s += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s + u < s1)
          v[u] = p[(s + u) * stride_s];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s + u < s1)
          r = op_apply_ordered<OP>(r, v[u]);
    }
  }
  sm[slice][lane] = r;
  __syncthreads();
  if (slice == 0 && i < n) {
    r = sm[0][lane];
    for (int w = 1; w < kSlices && w * per < count; ++w)
      r = op_apply_ordered<OP>(r, sm[w][lane]);
    store_out(out + i, r);
  }
}

template <typename OutT>
__global__ void __launch_bounds__(kBlock)
    cast_from_f32_kernel(const float *__restrict__ in, OutT *__restrict__ out, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x;
  if (i < n)
    out[i] = Elt<OutT>::from_f32(in[i]);
}

// plan constants of the column path (threads that cover one row of a slab; blocks per SM aimed at)
constexpr int kColsThreadsPerRow = 32;
// Measurement override of the column plan (b200_reduce_cols_plan_override): threads per slab
// row (0 = the rule above).
int g_cols_lpr_override = 0;
// How many batches of eight loads (column kernel) and rows (short-row kernel) a thread hints into L2
// before it waits for the kernel in front of it, and how many blocks per SM the two kernels aim at
// (both use 64 registers per thread, so four blocks of 256 threads fill an SM: more would be a
// second wave).  Measured on f16 [64, 512, 1024] (us per op, graph replay): column sum 13.6 with one
// batch hinted, 14.1 with two, 15.3 with four, 14.4 with none; row max 12.5 with nothing hinted,
// 10.5 with one row, 10.2 with four; two or three column blocks per SM 16.4 / 15.5 against 13.6.
// b200_reduce_tune changes them for such measurements.
int g_prefetch_cols = 1;
int g_prefetch_rows = 4;
int g_cols_blocks_per_sm = 4;
int g_rows_blocks_per_sm = 4;
// Block slots of a one-wave grid that are left free (b200_reduce_reserve_blocks).  The column and the
// short-row kernels fill every SM exactly (4 blocks of 256 threads x 64 registers), so a small kernel
// that runs beside them, like the exchange of a sharded sum, would push blocks into a second wave.
int g_reserved_blocks = 0;

// ---- launch plan: a pure function of the shape -----------------------------
struct Plan {
  bool rows;
  // rows
  int tpr, segs;
  int64_t seg_len;
  bool cluster;
  // columns
  int lpr, slabs, splits;
  int64_t rows_per_split;
  size_t ws_bytes;
};

Plan make_plan(int esize, int64_t A, int64_t B, int64_t C, bool vec_cols) {
  Plan p{};
  const int N = 16 / esize;
  if (C == 1) {
    p.rows = true;
    const int64_t row_bytes = B * esize;
    const int64_t target_groups = 4LL * kNumSMs;
    p.segs = 1;
    p.seg_len = B;
    if (A < 2LL * kNumSMs && row_bytes > 32768) {
      int64_t segs = std::min<int64_t>(ceil_div<int64_t>(row_bytes, 16384),
                                       ceil_div<int64_t>(target_groups, A));
      int64_t seg_len = ceil_div<int64_t>(ceil_div<int64_t>(B, segs), N * 4) * (N * 4);
      segs = ceil_div<int64_t>(B, seg_len);
      p.segs = (int)segs;
      p.seg_len = seg_len;
    }
    const int64_t vec_per_seg = ceil_div<int64_t>(p.seg_len, N);
    p.tpr = (int)std::min<int64_t>(kBlock, pow2_ceil(ceil_div<int64_t>(vec_per_seg, 4)));
    if (p.segs > 1)
      p.tpr = kBlock;
    p.cluster = p.segs > 1 && p.segs <= 8;
    p.ws_bytes = (p.segs > 1 && !p.cluster) ? (size_t)A * p.segs * sizeof(float) : 0;
  } else {
    p.rows = false;
    const int NV = vec_cols ? N : 1;
    auto split_for = [&](int lpr) {
      p.lpr = lpr;
      p.slabs = (int)ceil_div<int64_t>(C, (int64_t)p.lpr * NV);
      const int64_t rows_per_step = kBlock / p.lpr;
      const int64_t blocks = A * p.slabs;
      const int64_t wave = (int64_t)g_cols_blocks_per_sm * kNumSMs - g_reserved_blocks;
      int64_t splits = std::max<int64_t>(1, g_reserved_blocks > 0 ? wave / blocks : ceil_div<int64_t>(wave, blocks));
      splits = std::min<int64_t>(splits, std::max<int64_t>(1, B / (rows_per_step * 4)));
      p.rows_per_split = ceil_div<int64_t>(B, splits);
      p.splits = (int)ceil_div<int64_t>(B, p.rows_per_split);
    };
    int lpr = (int)std::min<int64_t>(kColsThreadsPerRow, pow2_ceil(ceil_div<int64_t>(C, NV)));
    if (g_cols_lpr_override > 0)
      lpr = std::min(lpr, g_cols_lpr_override);
    split_for(lpr);
    p.ws_bytes = p.splits > 1 ? (size_t)p.splits * A * C * sizeof(float) : 0;
  }
  return p;
}

// Whether 16-byte loads are possible for the column kernel is a property of the
// shape (C a multiple of the vector width); a misaligned base pointer falls back
// to scalar loads inside the same split plan.
bool cols_vec_by_shape(int esize, int64_t C) { return C % (16 / esize) == 0; }

template <typename T, int OP, typename OutT>
int launch(const T *in, OutT *out, int64_t A, int64_t B, int64_t C, void *ws,
           size_t ws_bytes, cudaStream_t stream) {
  constexpr int N = 16 / sizeof(T);
  const Plan p = make_plan(sizeof(T), A, B, C, cols_vec_by_shape(sizeof(T), C));
  if (p.ws_bytes > 0 && (ws == nullptr || ws_bytes < p.ws_bytes))
    return B200_ERR_WORKSPACE;
  float *partial = static_cast<float *>(ws);
  if (p.rows) {
    const bool vec = aligned16(in) && (B % N == 0);
    const int groups_per_block = kBlock / p.tpr;
    const int64_t groups = A * p.segs;
    const int64_t grid = ceil_div<int64_t>(groups, groups_per_block);
    if (grid > 0x7fffffffLL)
      return B200_ERR_UNSUPPORTED;
    if (p.cluster) {
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3((unsigned)grid);
      cfg.blockDim = dim3(kBlock);
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = p.segs;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      cudaError_t e;
      if (vec)
        e = cudaLaunchKernelEx(&cfg, reduce_rows_kernel<T, OP, true, true, OutT>, in, out,
                               partial, A, B, p.tpr, p.segs, p.seg_len);
      else
        e = cudaLaunchKernelEx(&cfg, reduce_rows_kernel<T, OP, false, true, OutT>, in, out,
                               partial, A, B, p.tpr, p.segs, p.seg_len);
      return check_cuda(e);
    }
    const int64_t nvec = B / N;
    if (vec && p.segs == 1 && nvec <= 4LL * p.tpr) {
      const int vpt = (int)ceil_div<int64_t>(nvec, p.tpr);
      const int64_t row_blocks = ceil_div<int64_t>(A, groups_per_block);
      const unsigned pgrid = (unsigned)std::min<int64_t>(
          row_blocks, std::max<int64_t>(1, (int64_t)kNumSMs * g_rows_blocks_per_sm - g_reserved_blocks));
      if (vpt <= 1)
        return launch_pdl(reduce_short_rows_kernel<T, OP, 1, OutT>, dim3(pgrid), dim3(kBlock), 0, stream, in, out, A, B, p.tpr, g_prefetch_rows);
      else if (vpt == 2)
        return launch_pdl(reduce_short_rows_kernel<T, OP, 2, OutT>, dim3(pgrid), dim3(kBlock), 0, stream, in, out, A, B, p.tpr, g_prefetch_rows);
      else
        return launch_pdl(reduce_short_rows_kernel<T, OP, 4, OutT>, dim3(pgrid), dim3(kBlock), 0, stream, in, out, A, B, p.tpr, g_prefetch_rows);
    }
    int rc;
    if (vec)
      rc = launch_pdl(reduce_rows_kernel<T, OP, true, false, OutT>, dim3((unsigned)grid), dim3(kBlock), 0, stream, in,
                      out, partial, A, B, p.tpr, p.segs, p.seg_len);
    else
      rc = launch_pdl(reduce_rows_kernel<T, OP, false, false, OutT>, dim3((unsigned)grid), dim3(kBlock), 0, stream, in,
                      out, partial, A, B, p.tpr, p.segs, p.seg_len);
    if (rc)
      return rc;
    if (p.segs > 1) {
      return launch_pdl(reduce_finalize_kernel<OP, OutT>, dim3((unsigned)ceil_div<int64_t>(A, 32)),
                        dim3(kFinalizeBlock), 0, stream, (const float *)partial, out, A, p.segs,
                        (int64_t)p.segs, (int64_t)1);
    }
    return B200_OK;
  }
  const bool vec = cols_vec_by_shape(sizeof(T), C) && aligned16(in);
  // the split plan is fixed by the shape; only the lane layout follows `vec`
  Plan q = p;
  if (!vec && cols_vec_by_shape(sizeof(T), C)) {
    q.lpr = (int)std::min<int64_t>(kColsThreadsPerRow, pow2_ceil(C));
    q.slabs = (int)ceil_div<int64_t>(C, q.lpr);
  }
  const int64_t grid = A * q.slabs * q.splits;
  if (grid > 0x7fffffffLL)
    return B200_ERR_UNSUPPORTED;
  int rc;
  if (vec)
    rc = launch_pdl(reduce_cols_kernel<T, OP, N, OutT>, dim3((unsigned)grid), dim3(kBlock), 0, stream, in, out,
                    partial, A, B, C, q.lpr, q.slabs, q.splits, q.rows_per_split, g_prefetch_cols);
  else
    rc = launch_pdl(reduce_cols_kernel<T, OP, 1, OutT>, dim3((unsigned)grid), dim3(kBlock), 0, stream, in, out,
                    partial, A, B, C, q.lpr, q.slabs, q.splits, q.rows_per_split, g_prefetch_cols);
  if (rc)
    return rc;
  if (q.splits > 1) {
    const int64_t n = A * C;
    return launch_pdl(reduce_finalize_kernel<OP, OutT>, dim3((unsigned)ceil_div<int64_t>(n, 32)),
                      dim3(kFinalizeBlock), 0, stream, (const float *)partial, out, n, q.splits, (int64_t)1, n);
  }
  return B200_OK;
}

template <typename T>
int dispatch_op(int op, const void *in, void *out, int64_t A, int64_t B, int64_t C, void *ws,
                size_t ws_bytes, cudaStream_t stream) {
  if (op == kSum)
    return launch<T, kSum, T>((const T *)in, (T *)out, A, B, C, ws, ws_bytes, stream);
  if (op == kMax)
    return launch<T, kMax, T>((const T *)in, (T *)out, A, B, C, ws, ws_bytes, stream);
  return B200_ERR_INVALID_ARG;
}

int esize_of(int dtype) {
  return dtype == B200_F32 ? 4 : (dtype == B200_F16 || dtype == B200_BF16) ? 2 : 0;
}

} // namespace
} // namespace b200

using namespace b200;

// Measurement hook (not part of the drop-in ABI): pins the column plan's threads per slab row
// (0 = the shape rule).  Workspace sizes follow the pinned plan, so ask for them after calling this.
extern "C" void b200_reduce_cols_plan_override(int threads_per_row) { g_cols_lpr_override = threads_per_row; }

extern "C" void b200_reduce_reserve_blocks(int blocks) { g_reserved_blocks = blocks > 0 ? blocks : 0; }

extern "C" void b200_reduce_tune(int prefetch_cols, int prefetch_rows, int cols_blocks_per_sm, int rows_blocks_per_sm) {
  g_prefetch_cols = prefetch_cols;
  g_prefetch_rows = prefetch_rows;
  g_cols_blocks_per_sm = cols_blocks_per_sm > 0 ? cols_blocks_per_sm : 4;
  g_rows_blocks_per_sm = rows_blocks_per_sm > 0 ? rows_blocks_per_sm : 4;
}

extern "C" size_t b200_reduce_workspace_bytes(int op, int dtype, int64_t A, int64_t B, int64_t C) {
  (void)op;
  const int es = esize_of(dtype);
  if (!es || A <= 0 || B <= 0 || C <= 0)
    return 0;
  return make_plan(es, A, B, C, cols_vec_by_shape(es, C)).ws_bytes;
}

extern "C" int b200_reduce(int op, int dtype, const void *in, void *out, int64_t A, int64_t B,
                           int64_t C, void *workspace, size_t workspace_bytes,
                           cudaStream_t stream) {
  const int es = esize_of(dtype);
  if (!es || A < 0 || B < 0 || C < 0 || (op != kSum && op != kMax))
    return B200_ERR_INVALID_ARG;
  if (A == 0 && B == 0) { // nothing to reduce: a copy, as reduce_impl.h:70-73
    if (C == 0)
      return B200_OK;
    if (!in || !out)
      return B200_ERR_INVALID_ARG;
    return check_cuda(cudaMemcpyAsync(out, in, (size_t)C * es, cudaMemcpyDeviceToDevice, stream));
  }
  if (A == 0 || C == 0)
    return B200_OK; // empty output
  if (B == 0 || !in || !out)
    return B200_ERR_INVALID_ARG;
  switch (dtype) {
  case B200_F32:
    return dispatch_op<float>(op, in, out, A, B, C, workspace, workspace_bytes, stream);
  case B200_F16:
    return dispatch_op<__half>(op, in, out, A, B, C, workspace, workspace_bytes, stream);
  default:
    return dispatch_op<__nv_bfloat16>(op, in, out, A, B, C, workspace, workspace_bytes, stream);
  }
}

extern "C" int b200_reduce_sum_to_f32(int dtype, const void *in, float *out, int64_t A, int64_t B,
                                      int64_t C, void *workspace, size_t workspace_bytes,
                                      cudaStream_t stream) {
  const int es = esize_of(dtype);
  if (!es || A <= 0 || B <= 0 || C <= 0 || !in || !out)
    return B200_ERR_INVALID_ARG;
  switch (dtype) {
  case B200_F32:
    return launch<float, kSum, float>((const float *)in, out, A, B, C, workspace, workspace_bytes, stream);
  case B200_F16:
    return launch<__half, kSum, float>((const __half *)in, out, A, B, C, workspace, workspace_bytes, stream);
  default:
    return launch<__nv_bfloat16, kSum, float>((const __nv_bfloat16 *)in, out, A, B, C, workspace,
                                              workspace_bytes, stream);
  }
}

extern "C" int b200_cast_from_f32(int dtype, const float *in, void *out, int64_t n,
                                  cudaStream_t stream) {
  if (n < 0 || !esize_of(dtype))
    return B200_ERR_INVALID_ARG;
  if (n == 0)
    return B200_OK;
  if (!in || !out)
    return B200_ERR_INVALID_ARG;
  const unsigned grid = (unsigned)ceil_div<int64_t>(n, kBlock);
  switch (dtype) {
  case B200_F32:
    cast_from_f32_kernel<float><<<grid, kBlock, 0, stream>>>(in, (float *)out, n);
    break;
  case B200_F16:
    cast_from_f32_kernel<__half><<<grid, kBlock, 0, stream>>>(in, (__half *)out, n);
    break;
  default:
    cast_from_f32_kernel<__nv_bfloat16><<<grid, kBlock, 0, stream>>>(in, (__nv_bfloat16 *)out, n);
  }
  return check_launch();
}

// ---- reduction without a caller-provided workspace ----------------------------
// Scratch for b200_reduce_no_alloc: one fixed block of device memory per GPU that
// loads this library, held until the process exits.
namespace {
constexpr size_t kStaticScratchBytes = 1u << 20;
static __device__ __align__(256) unsigned char g_reduce_static_scratch[kStaticScratchBytes];

// `g_reduce_static_scratch` names a host-side handle here, not device memory: the
// device address has to be asked for, once per device, with that device current.
int static_scratch_for_current_device(void **ptr) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void *addr[kMaxDevices] = {};
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev)))
    return rc;
  if (dev < 0 || dev >= kMaxDevices)
    return B200_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void *p = nullptr;
    if (int rc = check_cuda(cudaGetSymbolAddress(&p, g_reduce_static_scratch)))
      return rc;
    addr[dev] = p;
  }
  *ptr = addr[dev];
  return B200_OK;
}
} // namespace

extern "C" size_t b200_reduce_no_alloc_max_bytes(void) { return kStaticScratchBytes; }

extern "C" int b200_reduce_no_alloc(int op, int dtype, const void *in, void *out, int64_t A, int64_t B,
                                    int64_t C, cudaStream_t stream) {
  const size_t need = b200_reduce_workspace_bytes(op, dtype, A, B, C);
  if (need > kStaticScratchBytes)
    return B200_ERR_WORKSPACE; // this shape needs more scratch than the fixed block holds
  void *scratch = nullptr;
  if (need > 0)
    if (int rc = static_scratch_for_current_device(&scratch))
      return rc;
  return b200_reduce(op, dtype, in, out, A, B, C, scratch, need ? kStaticScratchBytes : 0, stream);
}
