// Flash-attention forward for sm_100a (head dim 128, f16 / bf16, f32 accumulate).
//
// One block owns 128 query rows of one (batch, head) and walks over the key/value
// tiles of 128 rows that the mask lets it see.  Warp roles:
//   warp 0      TMA producer: Q once, then K and V tiles into 2-stage rings
//   warp 1      MMA issuer (one lane): S = Q K^T and O += P V with tcgen05.mma,
//               accumulators in tensor memory (S double-buffered, O resident)
//   warps 2..5  softmax: thread t owns query row t; it reads its row of S from
//               tensor memory, keeps the running max / sum, writes P (16-bit) to
//               shared memory as the A operand of P V, rescales O in tensor
//               memory when the running max moved, and writes O / LSE at the end
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
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS0 = 0, kColS1 = 128, kColO = 256;
constexpr float kRescaleThreshold = 8.0f; // log2 units

struct FwdParams {
  float *lse;
  int *status;
  int64_t H, Hk, Sq, Sk;
  float scale_log2;
  int64_t window_left, window_right; // < 0: unbounded
};

struct SharedStorage {
  uint64_t bar_q;
  uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, o_done;
  uint32_t tmem_base;
  int failed;
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
      mbar_init(&ss->s_empty[s], 4);
    }
    mbar_init(&ss->p_full, 4);
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
    const int quarter = warp & 3;            // tensor-memory lanes 32 * quarter .. + 31
    const int row = quarter * 32 + lane;     // query row inside the tile
    const int64_t qrow = q0 + row;           // global query row
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = n > 0;
    for (int j = 0; ok && j < n; ++j) {
      if (!wait_or_flag(&ss->s_full[j & 1], (uint32_t)((j / 2) & 1), ss)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      float s[kBN];
      {
        const uint32_t base = tmem + lane_base + ((j & 1) ? kColS1 : kColS0);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(base + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            s[c * 32 + i] = __uint_as_float(r[i]);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&ss->s_empty[j & 1]);

      const int64_t kv0 = (int64_t)j * kBN;
      const bool need_mask = (right_bounded && kv0 + kBN - 1 > q0 + shift + p.window_right) ||
                             (kv0 + kBN > p.Sk) || left_bounded;
      if (need_mask) {
        const int64_t hi = right_bounded ? min(p.Sk - 1, qrow + shift + p.window_right) : p.Sk - 1;
        const int64_t lo = left_bounded ? qrow + shift - p.window_left : 0;
#pragma unroll
        for (int c = 0; c < kBN; ++c) {
          const int64_t kv = kv0 + c;
          if (kv > hi || kv < lo)
            s[c] = -INFINITY;
        }
      }
      float mx = s[0];
#pragma unroll
      for (int c = 1; c < kBN; ++c)
        mx = fmaxf(mx, s[c]);
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      float alpha = 1.f;
      const bool grew = m_new - m_used > kRescaleThreshold; // also true for -inf -> finite
      const bool rescale = j > 0 && __any_sync(0xffffffffu, grew);
      if (j == 0) {
        m_used = m_new;
      } else if (rescale) {
        alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(m_used - m_new);
        m_used = m_new;
        l *= alpha;
      }
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
      float sum = 0.f;
      uint32_t packed[kBN / 2];
#pragma unroll
      for (int c = 0; c < kBN; c += 2) {
        const float p0 = fast_exp2(fmaf(s[c], p.scale_log2, -m_safe));
        const float p1 = fast_exp2(fmaf(s[c + 1], p.scale_log2, -m_safe));
        sum += p0 + p1;
        packed[c / 2] = pack2(p0, p1, kBF16);
      }
      l += sum;

      // P's buffer and O are busy until P V of the previous tile has finished
      if (j > 0 && !wait_or_flag(&ss->o_done, (uint32_t)((j - 1) & 1), ss)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // P row -> shared memory, K-major 128-byte swizzled: [2 key blocks][128 rows][128 B]
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        const int kb = ch >> 3, chunk = ch & 7;
        uint4 v = make_uint4(packed[ch * 4], packed[ch * 4 + 1], packed[ch * 4 + 2], packed[ch * 4 + 3]);
        *reinterpret_cast<uint4 *>(sP + kb * kHalfTile + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      if (rescale) {
        const uint32_t base = tmem + lane_base + kColO;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
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
      ok = wait_or_flag(&ss->o_done, (uint32_t)((n - 1) & 1), ss);
    tc_fence_after_sync();
    const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
    const bool have_o = ok && n > 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      if (have_o) {
        tmem_ld32(tmem + lane_base + kColO + c * 32, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          r[i] = 0u;
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) { // 8 columns = one 16-byte chunk
        uint4 v;
        v.x = pack2(__uint_as_float(r[g * 8 + 0]) * inv_l, __uint_as_float(r[g * 8 + 1]) * inv_l, kBF16);
        v.y = pack2(__uint_as_float(r[g * 8 + 2]) * inv_l, __uint_as_float(r[g * 8 + 3]) * inv_l, kBF16);
        v.z = pack2(__uint_as_float(r[g * 8 + 4]) * inv_l, __uint_as_float(r[g * 8 + 5]) * inv_l, kBF16);
        v.w = pack2(__uint_as_float(r[g * 8 + 6]) * inv_l, __uint_as_float(r[g * 8 + 7]) * inv_l, kBF16);
        const int col = c * 32 + g * 8; // head-dim column of this chunk
        const int db = col >> 6, chunk = (col & 63) >> 3;
        *reinterpret_cast<uint4 *>(sP + db * kHalfTile + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
      }
    }
    fence_proxy_async_smem();
    if (qrow < p.Sq)
      p.lse[((int64_t)b * p.H + h) * p.Sq + qrow] =
          (l > 0.f) ? (m_used + log2f(l)) * 0.6931471805599453f : INFINITY;
    asm volatile("bar.sync 1, 128;" ::: "memory"); // the four softmax warps
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

extern "C" int b200_flash_attn_bwd(int, const void *, const void *, const void *, const void *, const void *,
                                   const float *, void *, void *, void *, float *, float *,
                                   const b200_flash_attn_params *, cudaStream_t) {
  return B200_ERR_UNSUPPORTED;
}
