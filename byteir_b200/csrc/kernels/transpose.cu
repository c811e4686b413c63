// TransposeOp for sm_100a: batched 2-D transpose  [batch, rows, cols] ->
// [batch, cols, rows], which covers the reference's 2-D kernel and its two 4-D
// NCHW <-> NHWC permutations, plus a general permutation fallback.
//
// Fast path (2- and 4-byte elements, row pitches multiples of 16 bytes): a
// persistent block walks over 128-byte x 128-byte tiles.  TMA loads a tile into
// shared memory in the 128-byte swizzled layout, the block transposes it out of
// shared memory through registers into a second swizzled tile, and TMA stores
// that tile; loads of the next tile and stores of the previous one overlap the
// shuffle.  With the swizzle both the column-wise reads and the 16-byte writes
// are free of bank conflicts.  Out-of-range parts of edge tiles are zero-filled
// on load and clipped on store by the TMA unit.
//
// Everything else goes through a padded 32 x 32 shared-memory tile with plain
// loads and stores.
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "tma.cuh"

namespace b200 {
namespace {

// =============================================================================
// TMA path
// =============================================================================
constexpr int kMaxInStages = 6;
constexpr int kOutStages = 2;
// Input tiles a block keeps in its ring (loads run in_stages - 1 tiles ahead), blocks per SM of the
// persistent grid, and the width of a panel of the tile order; 0 = the rule in launch_tma.
// b200_transpose_tune sets them for measurements.  Measured (TB/s of bytes read + written; ring depth /
// blocks per SM): bf16 8192 x 8192: 2/6 4.3, 3/5 5.2, 4/4 5.4; f16 [32] x 128 x 4096: 2/6 4.2, 3/5 6.4,
// 4/4 6.2; f16 1000 x 30000 (panels of 16): 3/5 5.6, 4/4 5.9, row-major order 4.5 / 4.8; f32 4096 x 4096 with
// tiles of 64 rows (two output tiles per input tile): 2/6 4.3, 3/5 6.0, 4/4 6.0 (with tiles of 32 rows: 4.9 at best).
int g_in_stages = 0, g_blocks_per_sm = 0, g_panel = 0;

// byte offset of 16-byte chunk `chunk` (0..7) of tile row `row` in the 128-byte
// swizzled layout the TMA unit reads and writes
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

template <int ES> // element size: 2 or 4
__global__ void __launch_bounds__(256)
    transpose_tma_kernel(const __grid_constant__ CUtensorMap in_map,
                         const __grid_constant__ CUtensorMap out_map, int tiles_c, int tiles_r,
                         int64_t num_tiles, int in_stages, int panel, int64_t rows, int *error) {
  constexpr int TC = 128 / ES; // tile columns = elements per 128-byte row
  constexpr int TR = 64;       // tile rows
  constexpr int TRo = 128 / ES; // elements of an output row that one 128-byte swizzled row holds
  constexpr int H = TR / TRo;  // output tiles per input tile: TC rows of TRo elements each (1, or 2 for 4-byte elements)
  constexpr uint32_t kInBytes = TR * 128;  // TR rows of 128 bytes
  constexpr uint32_t kOutHalf = TC * 128;  // TC rows of 128 bytes
  constexpr uint32_t kOutBytes = H * kOutHalf;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // 1024-byte alignment is what the 128-byte swizzle pattern repeats on
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char *in_tile = smem;
  unsigned char *out_tile = smem + in_stages * kInBytes;
  __shared__ uint64_t full[kMaxInStages];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    prefetch_tensormap(&in_map);
    prefetch_tensormap(&out_map);
    for (int s = 0; s < in_stages; ++s)
      mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  const int64_t my_tiles = (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
  // Tile order inside one matrix: panels of `panel` tile columns, row-major inside a panel.  The tiles
  // in flight at one time (a contiguous range of the order) then cover a roughly square region, so that
  // the loads AND the stores fall on a few kilobytes of every memory row they touch; in plain row-major
  // order the stores of the tiles in flight are 128-byte pieces of thousands of output rows.
  const int per_matrix = tiles_c * tiles_r;
  const int full_panels = tiles_c / panel;
  auto coords = [&](int64_t k, int &b, int &tr, int &tc) {
    const int64_t tile = blockIdx.x + k * gridDim.x;
    b = (int)(tile / per_matrix);
    const int t = (int)(tile - (int64_t)b * per_matrix);
    const int p = min(t / (panel * tiles_r), full_panels);
    const int width = p < full_panels ? panel : tiles_c - full_panels * panel;
    const int u = t - p * panel * tiles_r;
    tr = u / width;
    tc = p * panel + u - tr * width;
  };
  // Thread 0 issues the loads and thread 32 the stores.  Each works out the coordinates of its next
  // tile (a few integer divisions) while it would otherwise wait, so that no division sits between the
  // arrival of a tile and the issue of the next load.
  int nb = 0, ntr = 0, ntc = 0; // thread 0: coordinates of the next tile to load
  int64_t next_load = 0;
  int load_stage = 0; // stage of the next load (counted, not divided: the ring depth is a run-time value)
  auto issue_next = [&]() {
    mbar_arrive_expect_tx(&full[load_stage], kInBytes);
    tma_load_3d(in_tile + load_stage * kInBytes, &in_map, ntc * TC, ntr * TR, nb, &full[load_stage]);
    load_stage = load_stage + 1 == in_stages ? 0 : load_stage + 1;
    ++next_load;
    if (next_load < my_tiles)
      coords(next_load, nb, ntr, ntc);
  };

  // The first tiles of this block are hinted into L2 before the wait for the kernel in front of this
  // one (a hint returns nothing, and L2 is the point of coherence, so it is harmless even if that kernel
  // is still writing the input): the DRAM fetch then overlaps the other kernel's tail.
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int64_t k = 0; k < my_tiles && k < 2; ++k) {
      int b, tr, tc;
      coords(k, b, tr, tc);
      tma_prefetch_3d(&in_map, tc * TC, tr * TR, b);
    }
    if (my_tiles > 0)
      coords(0, nb, ntr, ntc);
  }
  pdl_wait();
  const int ahead = in_stages - 1;
  if (threadIdx.x == 0)
    for (int64_t k = 0; k < my_tiles && k < ahead; ++k)
      issue_next();

  int s = 0;          // stage of tile k
  uint32_t phase = 0; // parity of its barrier
  for (int64_t k = 0; k < my_tiles; ++k) {
    const int so = (int)(k % kOutStages);
    int sb = 0, str = 0, stc = 0; // thread 32: where tile k goes
    if (threadIdx.x == 32) {
      bulk_wait_read<kOutStages - 1>(); // the store that last read out_tile[so] is done
      coords(k, sb, str, stc);
    }
    const bool arrived = mbar_wait(&full[s], phase);
    // block-wide agreement (and the barrier after which tile k-1's input stage
    // may be refilled, which is where tile k + ahead goes): if the tile never arrived,
    // all threads leave together
    if (!__syncthreads_and(arrived)) {
      if (error)
        *error = 2;
      break;
    }
    if (threadIdx.x == 0 && next_load < my_tiles)
      issue_next();

    const unsigned char *src = in_tile + s * kInBytes;
    unsigned char *dst = out_tile + so * kOutBytes;
    if (ES == 2) {
      // thread: columns c, c+1 (c = 2 * lane) x rows 8 * warp .. 8 * warp + 7
      const int c = 2 * lane, r0 = 8 * warp;
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        w[i] = *reinterpret_cast<const uint32_t *>(src + swz(r0 + i, c >> 3) + ((c & 7) << 1));
      uint4 even, odd; // output rows c and c + 1, elements r0 .. r0 + 7
      even.x = __byte_perm(w[0], w[1], 0x5410);
      even.y = __byte_perm(w[2], w[3], 0x5410);
      even.z = __byte_perm(w[4], w[5], 0x5410);
      even.w = __byte_perm(w[6], w[7], 0x5410);
      odd.x = __byte_perm(w[0], w[1], 0x7632);
      odd.y = __byte_perm(w[2], w[3], 0x7632);
      odd.z = __byte_perm(w[4], w[5], 0x7632);
      odd.w = __byte_perm(w[6], w[7], 0x7632);
      // half of each quarter-warp writes its odd row first, so that the eight
      // 16-byte stores of a quarter-warp fall into eight different bank groups
      if (lane & 4) {
        *reinterpret_cast<uint4 *>(dst + swz(c + 1, warp)) = odd;
        *reinterpret_cast<uint4 *>(dst + swz(c, warp)) = even;
      } else {
        *reinterpret_cast<uint4 *>(dst + swz(c, warp)) = even;
        *reinterpret_cast<uint4 *>(dst + swz(c + 1, warp)) = odd;
      }
    } else {
      // thread: column c = lane x rows 4 * warp .. 4 * warp + 3 of each 32-row half of the tile
      const int c = lane;
#pragma unroll
      for (int h = 0; h < H; ++h) {
        const int r0 = h * TRo + 4 * warp;
        uint4 v;
        v.x = *reinterpret_cast<const uint32_t *>(src + swz(r0 + 0, c >> 2) + ((c & 3) << 2));
        v.y = *reinterpret_cast<const uint32_t *>(src + swz(r0 + 1, c >> 2) + ((c & 3) << 2));
        v.z = *reinterpret_cast<const uint32_t *>(src + swz(r0 + 2, c >> 2) + ((c & 3) << 2));
        v.w = *reinterpret_cast<const uint32_t *>(src + swz(r0 + 3, c >> 2) + ((c & 3) << 2));
        *reinterpret_cast<uint4 *>(dst + h * kOutHalf + swz(c, warp)) = v;
      }
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (threadIdx.x == 32) {
#pragma unroll
      for (int h = 0; h < H; ++h)
        if ((int64_t)str * TR + h * TRo < rows) // a store that would start past the end of the rows is left out
          tma_store_3d(&out_map, dst + h * kOutHalf, str * TR + h * TRo, stc * TC, sb);
      bulk_commit();
    }
    if (++s == in_stages) {
      s = 0;
      phase ^= 1u;
    }
  }
  if (threadIdx.x == 32)
    bulk_wait_all<0>();
}

template <int ES>
int launch_tma(const void *in, void *out, int64_t batch, int64_t rows, int64_t cols,
               cudaStream_t stream) {
  constexpr int TC = 128 / ES;
  constexpr int TR = 64;
  constexpr int TRo = 128 / ES;
  CUtensorMap in_map, out_map;
  const CUtensorMapDataType dt = ES == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  {
    const uint64_t dims[3] = {(uint64_t)cols, (uint64_t)rows, (uint64_t)batch};
    const uint64_t strides[2] = {(uint64_t)cols * ES, (uint64_t)rows * cols * ES};
    const uint32_t box[3] = {TC, TR, 1};
    if (int rc = make_tensor_map(&in_map, dt, 3, const_cast<void *>(in), dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t dims[3] = {(uint64_t)rows, (uint64_t)cols, (uint64_t)batch};
    const uint64_t strides[2] = {(uint64_t)rows * ES, (uint64_t)rows * cols * ES};
    const uint32_t box[3] = {TRo, TC, 1};
    if (int rc = make_tensor_map(&out_map, dt, 3, out, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  const int tiles_c = (int)ceil_div<int64_t>(cols, TC);
  const int tiles_r = (int)ceil_div<int64_t>(rows, TR);
  const int64_t num_tiles = (int64_t)tiles_c * tiles_r * batch;
  // large matrices: four tiles in the ring and four blocks per SM; everything else three and five
  const bool deep = (int64_t)tiles_c * tiles_r >= 4096;
  const int in_stages = g_in_stages > 0 ? std::max(2, std::min(g_in_stages, kMaxInStages)) : (deep ? 4 : 3);
  const int blocks_per_sm = g_blocks_per_sm > 0 ? g_blocks_per_sm : (deep ? 4 : 5);
  const int panel = std::max(1, std::min(g_panel > 0 ? g_panel : 16, tiles_c));
  const size_t smem = (size_t)in_stages * TR * 128 + (size_t)kOutStages * TC * TR * ES + 1024;
  // the attribute belongs to the current device's context: set on every call (a host-side table write)
  if (int rc = check_cuda(cudaFuncSetAttribute(transpose_tma_kernel<ES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)smem)))
    return rc;
  const unsigned grid = (unsigned)std::min<int64_t>(num_tiles, (int64_t)kNumSMs * blocks_per_sm);
  return launch_pdl(transpose_tma_kernel<ES>, dim3(grid), dim3(256), smem, stream, in_map, out_map, tiles_c, tiles_r,
                    num_tiles, in_stages, panel, rows, (int *)nullptr);
}

// =============================================================================
// plain path: any element size, any shape
// =============================================================================
template <typename T>
__global__ void __launch_bounds__(256)
    transpose_plain_kernel(const T *__restrict__ in, T *__restrict__ out, int64_t batch,
                           int64_t rows, int64_t cols, int64_t tiles_c, int64_t tiles_r) {
  __shared__ T tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t num_tiles = tiles_c * tiles_r * batch;
  for (int64_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const int64_t tc = t % tiles_c;
    const int64_t rest = t / tiles_c;
    const int64_t tr = rest % tiles_r;
    const int64_t b = rest / tiles_r;
    const T *src = in + b * rows * cols;
    T *dst = out + b * rows * cols;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      const int64_t r = tr * 32 + ty + j, c = tc * 32 + tx;
      if (r < rows && c < cols)
        tile[ty + j][tx] = src[r * cols + c];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      const int64_t c = tc * 32 + ty + j, r = tr * 32 + tx;
      if (r < rows && c < cols)
        dst[c * rows + r] = tile[tx][ty + j];
    }
    __syncthreads();
  }
}

template <typename T>
int launch_plain(const void *in, void *out, int64_t batch, int64_t rows, int64_t cols,
                 cudaStream_t stream) {
  const int64_t tiles_c = ceil_div<int64_t>(cols, 32), tiles_r = ceil_div<int64_t>(rows, 32);
  const int64_t num_tiles = tiles_c * tiles_r * batch;
  const unsigned grid = (unsigned)std::min<int64_t>(num_tiles, (int64_t)kNumSMs * 64);
  transpose_plain_kernel<T><<<grid, 256, 0, stream>>>((const T *)in, (T *)out, batch, rows, cols,
                                                      tiles_c, tiles_r);
  return check_launch();
}

// general permutation: one thread per output element, reads through strides
struct PermuteDims {
  int rank;
  int64_t out_shape[8];
  int64_t src_stride[8];
};

template <typename T>
__global__ void __launch_bounds__(256)
    permute_plain_kernel(const T *__restrict__ in, T *__restrict__ out, PermuteDims d, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    int64_t rem = i, off = 0;
#pragma unroll 1
    for (int k = d.rank - 1; k >= 0; --k) {
      const int64_t q = rem / d.out_shape[k];
      off += (rem - q * d.out_shape[k]) * d.src_stride[k];
      rem = q;
    }
    out[i] = in[off];
  }
}

template <typename T>
int launch_permute_plain(const void *in, void *out, const PermuteDims &d, int64_t n,
                         cudaStream_t stream) {
  const unsigned grid = (unsigned)std::min<int64_t>(ceil_div<int64_t>(n, 256), (int64_t)kNumSMs * 32);
  permute_plain_kernel<T><<<grid, 256, 0, stream>>>((const T *)in, (T *)out, d, n);
  return check_launch();
}

} // namespace
} // namespace b200

using namespace b200;

extern "C" void b200_transpose_tune(int in_stages, int blocks_per_sm, int panel) {
  g_panel = panel;
  g_in_stages = in_stages;
  g_blocks_per_sm = blocks_per_sm;
}

extern "C" int b200_transpose_batched_path(int path, int elt_bytes, const void *in, void *out,
                                           int64_t batch, int64_t rows, int64_t cols,
                                           cudaStream_t stream) {
  if (batch < 0 || rows < 0 || cols < 0)
    return B200_ERR_INVALID_ARG;
  if (batch == 0 || rows == 0 || cols == 0)
    return B200_OK;
  if (!in || !out || in == out)
    return B200_ERR_INVALID_ARG;
  if (rows == 1 || cols == 1) // a transpose that moves nothing
    return check_cuda(cudaMemcpyAsync(out, in, (size_t)batch * rows * cols * elt_bytes,
                                      cudaMemcpyDeviceToDevice, stream));
  const bool tma_ok = (elt_bytes == 2 || elt_bytes == 4) && aligned16(in) && aligned16(out) &&
                      (cols * elt_bytes) % 16 == 0 && (rows * elt_bytes) % 16 == 0 &&
                      rows < (1LL << 31) && cols < (1LL << 31) && batch < (1LL << 31) &&
                      get_encode_tiled() != nullptr;
  if (path == 1 && !tma_ok)
    return B200_ERR_ALIGNMENT;
  if ((path == 0 && tma_ok) || path == 1)
    return elt_bytes == 2 ? launch_tma<2>(in, out, batch, rows, cols, stream)
                          : launch_tma<4>(in, out, batch, rows, cols, stream);
  switch (elt_bytes) {
  case 1:
    return launch_plain<uint8_t>(in, out, batch, rows, cols, stream);
  case 2:
    return launch_plain<uint16_t>(in, out, batch, rows, cols, stream);
  case 4:
    return launch_plain<uint32_t>(in, out, batch, rows, cols, stream);
  case 8:
    return launch_plain<uint64_t>(in, out, batch, rows, cols, stream);
  default:
    return B200_ERR_UNSUPPORTED;
  }
}

extern "C" int b200_transpose_batched(int elt_bytes, const void *in, void *out, int64_t batch,
                                      int64_t rows, int64_t cols, cudaStream_t stream) {
  return b200_transpose_batched_path(0, elt_bytes, in, out, batch, rows, cols, stream);
}

extern "C" int b200_permute(int elt_bytes, const void *in, void *out, int rank, const int64_t *shape,
                            const int64_t *perm, cudaStream_t stream) {
  if (rank < 1 || rank > 8 || !shape || !perm)
    return B200_ERR_INVALID_ARG;
  bool seen[8] = {false};
  int64_t n = 1;
  for (int k = 0; k < rank; ++k) {
    if (perm[k] < 0 || perm[k] >= rank || seen[perm[k]] || shape[k] < 0)
      return B200_ERR_INVALID_ARG;
    seen[perm[k]] = true;
    n *= shape[k];
  }
  if (n == 0)
    return B200_OK;
  if (!in || !out)
    return B200_ERR_INVALID_ARG;
  // Drop size-1 dims, then merge input dims that stay adjacent and in order in
  // the output.  Work in output order: entry k is input dim p[k].
  int compact[8], next_id = 0; // input dim -> its position among the kept dims
  for (int i = 0; i < rank; ++i)
    compact[i] = shape[i] != 1 ? next_id++ : -1;
  std::vector<int64_t> p, s; // permutation entry and its size, output order
  for (int k = 0; k < rank; ++k)
    if (shape[perm[k]] != 1) {
      p.push_back(compact[perm[k]]);
      s.push_back(shape[perm[k]]);
    }
  std::vector<int64_t> mp, ms;
  for (size_t k = 0; k < p.size(); ++k) {
    if (!mp.empty() && p[k] == p[k - 1] + 1) {
      ms.back() *= s[k];
      // the merged group keeps the id of its first input dim
    } else {
      mp.push_back(p[k]);
      ms.push_back(s[k]);
    }
  }
  const size_t g = mp.size();
  // rank of each group in input order
  std::vector<int> order(g);
  for (size_t k = 0; k < g; ++k) {
    int r = 0;
    for (size_t j = 0; j < g; ++j)
      if (mp[j] < mp[k])
        ++r;
    order[k] = r;
  }
  if (g <= 1)
    return check_cuda(cudaMemcpyAsync(out, in, (size_t)n * elt_bytes, cudaMemcpyDeviceToDevice, stream));
  if (g == 2) // (1, 0)
    return b200_transpose_batched(elt_bytes, in, out, 1, ms[1], ms[0], stream);
  if (g == 3 && order[0] == 0 && order[1] == 2 && order[2] == 1) // (0, 2, 1)
    return b200_transpose_batched(elt_bytes, in, out, ms[0], ms[2], ms[1], stream);
  // general case: strides of the merged input dims
  std::vector<int64_t> in_sizes(g), in_strides(g);
  for (size_t k = 0; k < g; ++k)
    in_sizes[order[k]] = ms[k];
  int64_t st = 1;
  for (int i = (int)g - 1; i >= 0; --i) {
    in_strides[i] = st;
    st *= in_sizes[i];
  }
  PermuteDims d{};
  d.rank = (int)g;
  for (size_t k = 0; k < g; ++k) {
    d.out_shape[k] = ms[k];
    d.src_stride[k] = in_strides[order[k]];
  }
  switch (elt_bytes) {
  case 1:
    return launch_permute_plain<uint8_t>(in, out, d, n, stream);
  case 2:
    return launch_permute_plain<uint16_t>(in, out, d, n, stream);
  case 4:
    return launch_permute_plain<uint32_t>(in, out, d, n, stream);
  case 8:
    return launch_permute_plain<uint64_t>(in, out, d, n, stream);
  default:
    return B200_ERR_UNSUPPORTED;
  }
}
