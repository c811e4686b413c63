// IndexSelectOp (row gather) and IndexPutOp with accumulate (deterministic
// scatter-add) for sm_100a.
//
// Gather.  out[a, ob, :] = in[a, idx[ob], :].  When a row is a multiple of 16
// bytes the rows never pass through registers: one warp per block drives a
// 4-stage ring of shared-memory tiles; each lane issues bulk (TMA) copies
// global -> shared for its rows of the tile, the tile's mbarrier counts the
// bytes, and one bulk copy shared -> global writes the tile, which is contiguous
// in the output.  Other row sizes use vector loads sized to the row.
//
// Scatter-add.  out = in; out[idx[i], :] += upd[i, :].  The reference uses
// atomicAdd, so its f32 result depends on scheduling.  Here the (index, i) pairs
// are sorted by index with a stable LSD radix sort, which leaves the updates of
// a row adjacent and in ascending i.  The sorted list is cut into chunks of 32
// entries; one warp sums each chunk's runs in f32.  A run that lies inside one
// chunk is finished at once (table value + sum, one rounding).  A run that
// crosses chunk borders leaves f32 partials, and the warp of the chunk where the
// run starts adds the partials of the following chunks in order.  The summation
// tree is therefore a function of the index list alone.
#include <algorithm>
#include <map>
#include <mutex>
#include <type_traits>
#include <utility>

#include "common.cuh"
#include "tma.cuh"

namespace b200 {
namespace {

// =============================================================================
// gather
// =============================================================================
constexpr int kGatherStages = 4;
constexpr int kGatherMaxRowsPerTile = 128;

template <typename IdxT>
__global__ void __launch_bounds__(32)
    gather_rows_bulk_kernel(const char *__restrict__ in, const IdxT *__restrict__ idx,
                            char *__restrict__ out, int64_t IB, int64_t OB, uint32_t row_bytes,
                            int rows_per_tile, int64_t tiles_per_a, int64_t num_tiles,
                            int *status) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[kGatherStages];
  const int lane = threadIdx.x;
  const uint32_t stage_bytes = (uint32_t)rows_per_tile * row_bytes;

  if (lane == 0) {
    for (int s = 0; s < kGatherStages; ++s)
      mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncwarp();

  const int64_t my_tiles = (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;

  auto issue = [&](int64_t k) {
    const int64_t tile = blockIdx.x + k * gridDim.x;
    const int stage = (int)(k % kGatherStages);
    const int64_t a = tile / tiles_per_a;
    const int64_t ob0 = (tile - a * tiles_per_a) * rows_per_tile;
    const int nrows = (int)min((int64_t)rows_per_tile, OB - ob0);
    unsigned char *dst = smem + (size_t)stage * stage_bytes;
    const char *src = in + (size_t)a * IB * row_bytes;
    int64_t my_idx[kGatherMaxRowsPerTile / 32];
    int valid = 0;
#pragma unroll
    for (int u = 0; u < kGatherMaxRowsPerTile / 32; ++u) {
      const int r = lane + 32 * u;
      int64_t i = -1;
      if (r < nrows) {
        i = (int64_t)idx[ob0 + r];
        if (i < 0 || i >= IB)
          i = -1;
        else
          ++valid;
      }
      my_idx[u] = i;
    }
    valid = __reduce_add_sync(0xffffffffu, valid);
    if (lane == 0)
      mbar_arrive_expect_tx(&full[stage], (uint32_t)valid * row_bytes);
    __syncwarp();
    bool zero_filled = false;
#pragma unroll
    for (int u = 0; u < kGatherMaxRowsPerTile / 32; ++u) {
      const int r = lane + 32 * u;
      if (r >= nrows)
        continue;
      if (my_idx[u] >= 0) {
        bulk_g2s(dst + (size_t)r * row_bytes, src + (size_t)my_idx[u] * row_bytes, row_bytes,
                 &full[stage]);
      } else {
        uint4 *z = reinterpret_cast<uint4 *>(dst + (size_t)r * row_bytes);
        for (uint32_t b = 0; b < row_bytes / 16; ++b)
          z[b] = make_uint4(0, 0, 0, 0);
        zero_filled = true;
        if (status)
          *status = 1;
      }
    }
    if (zero_filled)
      fence_proxy_async_smem();
  };

  const int prologue = (int)min((int64_t)(kGatherStages - 1), my_tiles);
  for (int k = 0; k < prologue; ++k)
    issue(k);

  for (int64_t k = 0; k < my_tiles; ++k) {
    const int stage = (int)(k % kGatherStages);
    const uint32_t parity = (uint32_t)((k / kGatherStages) & 1);
    if (!__all_sync(0xffffffffu, mbar_wait(&full[stage], parity))) {
      if (status)
        *status = 2; // a copy never arrived: give up instead of spinning
      break;
    }
    if (lane == 0) {
      const int64_t tile = blockIdx.x + k * gridDim.x;
      const int64_t a = tile / tiles_per_a;
      const int64_t ob0 = (tile - a * tiles_per_a) * rows_per_tile;
      const int nrows = (int)min((int64_t)rows_per_tile, OB - ob0);
      bulk_s2g(out + ((size_t)a * OB + ob0) * row_bytes, smem + (size_t)stage * stage_bytes,
               (uint32_t)nrows * row_bytes);
      bulk_commit();
    }
    if (k + kGatherStages - 1 < my_tiles) {
      // the stage to refill was last read by the store of tile k - 1
      if (lane == 0)
        bulk_wait_read<1>();
      __syncwarp();
      issue(k + kGatherStages - 1);
    }
  }
  if (lane == 0)
    bulk_wait_all<0>();
}

// Vector gather for any row size: V is the widest type that divides a row.
template <typename V, typename IdxT>
__global__ void __launch_bounds__(256)
    gather_generic_kernel(const V *__restrict__ in, const IdxT *__restrict__ idx,
                          V *__restrict__ out, int64_t A, int64_t IB, int64_t OB, int64_t vpr,
                          int tx_log2, int *status) {
  const int TX = 1 << tx_log2, TY = 256 >> tx_log2;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> tx_log2;
  constexpr int U = 4;
  for (int64_t a = blockIdx.y; a < A; a += gridDim.y) {
    const V *src = in + a * IB * vpr;
    V *dst = out + a * OB * vpr;
    for (int64_t ob0 = (int64_t)blockIdx.x * TY * U; ob0 < OB; ob0 += (int64_t)gridDim.x * TY * U) {
      int64_t row[U];
      bool live[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t ob = ob0 + u * TY + ty;
        live[u] = ob < OB;
        row[u] = live[u] ? (int64_t)idx[ob] : 0;
        if (live[u] && (row[u] < 0 || row[u] >= IB)) {
          row[u] = -1;
          if (status && tx == 0)
            *status = 1;
        }
      }
      for (int64_t v = tx; v < vpr; v += TX) {
        V val[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          val[u] = V{};
          if (live[u] && row[u] >= 0)
            val[u] = src[row[u] * vpr + v];
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (live[u])
            dst[(ob0 + u * TY + ty) * vpr + v] = val[u];
      }
    }
  }
}

// The same gather as a persistent kernel: a block walks over groups of TY * U output rows,
// keeps U row loads per thread in flight, and reads the indices of its next group before it
// waits for the rows of the current one, so that the index load never stands between two
// batches of row loads.
template <typename V, typename IdxT, int U>
__global__ void __launch_bounds__(256, U <= 8 ? 3 : 1)
    gather_rows_vec_kernel(const V *__restrict__ in, const IdxT *__restrict__ idx, V *__restrict__ out,
                           int64_t A, int64_t IB, int64_t OB, int64_t vpr, int tx_log2, int *status) {
  const int TX = 1 << tx_log2, TY = 256 >> tx_log2;
  const int tx = threadIdx.x & (TX - 1), ty = threadIdx.x >> tx_log2;
  const int64_t group = (int64_t)TY * U;
  auto load_rows = [&](int64_t ob0, int(&row)[U]) { // IB < 2^31: checked by the launcher
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t ob = ob0 + u * TY + ty;
      const int64_t i = ob < OB ? (int64_t)idx[ob] : 0;
      row[u] = ob < OB ? (int)i : -2; // -2: past the end; -1: out of range
      if (ob < OB && (i < 0 || i >= IB)) {
        row[u] = -1;
        if (status && tx == 0)
          *status = 1;
      }
    }
  };
  for (int64_t a = blockIdx.y; a < A; a += gridDim.y) {
    const V *src = in + a * IB * vpr;
    V *dst = out + a * OB * vpr;
    int64_t ob0 = (int64_t)blockIdx.x * group;
    int row[U], next[U];
    if (ob0 < OB)
      load_rows(ob0, row);
    for (; ob0 < OB; ob0 += (int64_t)gridDim.x * group) {
      const int64_t ob_next = ob0 + (int64_t)gridDim.x * group;
      if (ob_next < OB)
        load_rows(ob_next, next);
      for (int64_t v = tx; v < vpr; v += TX) {
        V val[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          val[u] = V{};
          if (row[u] >= 0)
            val[u] = src[(int64_t)row[u] * vpr + v];
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (row[u] != -2)
            dst[(ob0 + u * TY + ty) * vpr + v] = val[u];
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        row[u] = next[u];
    }
  }
}

template <typename V, typename IdxT, int U>
int launch_gather_vec(const void *in, const void *idx, void *out, int64_t A, int64_t IB, int64_t OB,
                      int64_t row_bytes, int blocks_per_sm, int *status, cudaStream_t stream) {
  const int64_t vpr = row_bytes / (int64_t)sizeof(V);
  int tx_log2 = 0;
  while ((1 << tx_log2) < vpr && tx_log2 < 8)
    ++tx_log2;
  const int TY = 256 >> tx_log2;
  const int64_t groups = ceil_div<int64_t>(OB, (int64_t)TY * U);
  dim3 grid((unsigned)std::min<int64_t>(groups, (int64_t)kNumSMs * blocks_per_sm), (unsigned)std::min<int64_t>(A, 65535));
  gather_rows_vec_kernel<V, IdxT, U><<<grid, 256, 0, stream>>>((const V *)in, (const IdxT *)idx, (V *)out, A, IB, OB,
                                                               vpr, tx_log2, status);
  return check_launch();
}

// Rows of 64 .. 1024 bytes through the tensor-map gather: one cp.async.bulk.tensor instruction
// in the tile::gather4 form fetches four table rows, named by four row coordinates, into four
// consecutive rows of a shared-memory tile; the tile's mbarrier counts the bytes, and one bulk
// copy shared -> global writes the tile, which is contiguous in the output.  One warp per block
// drives a ring of kGatherStages tiles, lane q of it the q-th quad of rows of each tile.  The
// tensor map is two-dimensional over this GPU's table only, [A * IB rows][row_bytes / 4 32-bit
// columns], box = one row; a row coordinate past the end reads zeros (an index out of range).
template <typename IdxT>
__global__ void __launch_bounds__(32)
    gather_rows_g4_kernel(const __grid_constant__ CUtensorMap table_map, const IdxT *__restrict__ idx,
                          char *__restrict__ out, int64_t IB, int64_t OB, int64_t total_rows, uint32_t row_bytes,
                          int rows_per_tile, int64_t tiles_per_a, int64_t num_tiles, int *status) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[kGatherStages];
  const int lane = threadIdx.x;
  const uint32_t stage_bytes = (uint32_t)rows_per_tile * row_bytes;
  if (lane == 0) {
    prefetch_tensormap(&table_map);
    for (int s = 0; s < kGatherStages; ++s)
      mbar_init(&full[s], 1);
    mbar_fence_init();
  }
  __syncwarp();
  const int64_t my_tiles = (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
  // the index words of the first tiles, on their way into L2 while the kernel in front of this one ends
  pdl_launch_dependents();
  for (int64_t k = 0; k < my_tiles && k < kGatherStages - 1; ++k) {
    const int64_t tile = blockIdx.x + k * gridDim.x;
    const int64_t ob0 = (tile % tiles_per_a) * rows_per_tile;
    if (lane * 16 < rows_per_tile * (int)sizeof(IdxT) && ob0 + lane * (16 / (int)sizeof(IdxT)) < OB)
      prefetch_l2(reinterpret_cast<const char *>(idx + ob0) + lane * 16);
  }
  pdl_wait();

  auto issue = [&](int64_t k) {
    const int64_t tile = blockIdx.x + k * gridDim.x;
    const int stage = (int)(k % kGatherStages);
    const int64_t a = tile / tiles_per_a;
    const int64_t ob0 = (tile - a * tiles_per_a) * rows_per_tile;
    const int nrows = (int)min((int64_t)rows_per_tile, OB - ob0);
    const int quads = (nrows + 3) >> 2;
    unsigned char *dst = smem + (size_t)stage * stage_bytes;
    if (lane == 0)
      mbar_arrive_expect_tx(&full[stage], (uint32_t)quads * 4u * row_bytes);
    __syncwarp();
    if (lane < quads) {
      int r[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = lane * 4 + u;
        int64_t i = (int64_t)total_rows; // past the end of the map: zeros
        if (rr < nrows) {
          const int64_t v = (int64_t)idx[ob0 + rr];
          if (v < 0 || v >= IB) {
            if (status)
              *status = 1;
          } else {
            i = a * IB + v;
          }
        }
        r[u] = (int)i;
      }
      tma_gather4_2d(dst + (size_t)lane * 4 * row_bytes, &table_map, 0, r[0], r[1], r[2], r[3], &full[stage]);
    }
  };

  const int prologue = (int)min((int64_t)(kGatherStages - 1), my_tiles);
  for (int k = 0; k < prologue; ++k)
    issue(k);
  for (int64_t k = 0; k < my_tiles; ++k) {
    const int stage = (int)(k % kGatherStages);
    const uint32_t parity = (uint32_t)((k / kGatherStages) & 1);
    if (!__all_sync(0xffffffffu, mbar_wait(&full[stage], parity))) {
      if (status)
        *status = 2; // a copy never arrived: give up instead of spinning
      break;
    }
    if (lane == 0) {
      const int64_t tile = blockIdx.x + k * gridDim.x;
      const int64_t a = tile / tiles_per_a;
      const int64_t ob0 = (tile - a * tiles_per_a) * rows_per_tile;
      const int nrows = (int)min((int64_t)rows_per_tile, OB - ob0);
      bulk_s2g(out + ((size_t)a * OB + ob0) * row_bytes, smem + (size_t)stage * stage_bytes,
               (uint32_t)nrows * row_bytes);
      bulk_commit();
    }
    if (k + kGatherStages - 1 < my_tiles) {
      if (lane == 0)
        bulk_wait_read<1>(); // the stage to refill was last read by the store of tile k - 1
      __syncwarp();
      issue(k + kGatherStages - 1);
    }
  }
  if (lane == 0)
    bulk_wait_all<0>();
}

template <typename V, typename IdxT>
int launch_gather_generic(const void *in, const void *idx, void *out, int64_t A, int64_t IB,
                          int64_t OB, int64_t row_bytes, int *status, cudaStream_t stream) {
  const int64_t vpr = row_bytes / (int64_t)sizeof(V);
  int tx_log2 = 0;
  while ((1 << tx_log2) < vpr && tx_log2 < 8)
    ++tx_log2;
  const int TY = 256 >> tx_log2;
  const int64_t row_blocks = ceil_div<int64_t>(OB, (int64_t)TY * 4);
  dim3 grid((unsigned)std::min<int64_t>(row_blocks, 1 << 20), (unsigned)std::min<int64_t>(A, 65535));
  gather_generic_kernel<V, IdxT><<<grid, 256, 0, stream>>>((const V *)in, (const IdxT *)idx, (V *)out,
                                                           A, IB, OB, vpr, tx_log2, status);
  return check_launch();
}

template <typename IdxT>
int launch_gather(int path, const void *in, const void *idx, void *out, int64_t A, int64_t IB,
                  int64_t OB, int64_t row_bytes, int *status, cudaStream_t stream) {
  const bool bulk_ok = row_bytes % 16 == 0 && aligned16(in) && aligned16(out) && row_bytes <= 49152;
  if (path == 1 && !bulk_ok)
    return B200_ERR_ALIGNMENT;
  // Measured on 64 MB of gathered rows out of a 256 MB table.  The tensor-map gather with 8 KiB
  // tiles beats both other forms for rows of 64 bytes .. 1 KiB: 3.9 TB/s at 64 B, 5.1 at 128 B,
  // 6.1 at 256 B, 6.3 at 512 B, 6.5 at 1 KiB, against 3.2 .. 4.4 through vector loads and
  // 2.0 .. 5.7 with one bulk copy per row (a bulk copy per small row is mostly descriptor
  // overhead).  Longer rows (a box holds at most 256 columns) run at 5.7 .. 6.4 TB/s through the
  // ring of per-row bulk copies and 4.4 .. 4.9 TB/s through vector loads.
  const bool g4_ok = bulk_ok && row_bytes % 32 == 0 && row_bytes >= 64 && row_bytes <= 1024 && A * IB < 0x7fffffffLL;
  if (path == 0 && g4_ok)
    path = 10;
  if ((path == 0 && bulk_ok && row_bytes >= 512) || path == 1) {
    int rows_per_tile =
        (int)std::max<int64_t>(1, std::min<int64_t>(kGatherMaxRowsPerTile, 16384 / row_bytes));
    rows_per_tile = (int)std::min<int64_t>(rows_per_tile, OB);
    const int64_t tiles_per_a = ceil_div<int64_t>(OB, rows_per_tile);
    const int64_t num_tiles = tiles_per_a * A;
    const size_t smem = (size_t)kGatherStages * rows_per_tile * row_bytes;
    // the attribute belongs to the current device's context, so it is set on every call (a
    // host-side table write) rather than once per process
    if (int rc = check_cuda(cudaFuncSetAttribute(gather_rows_bulk_kernel<IdxT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 kGatherStages * 49152)))
      return rc;
    const int ctas_per_sm = (int)std::max<size_t>(1, std::min<size_t>(8, (200 * 1024) / (smem + 1024)));
    const unsigned grid = (unsigned)std::min<int64_t>(num_tiles, (int64_t)kNumSMs * ctas_per_sm);
    gather_rows_bulk_kernel<IdxT><<<grid, 32, smem, stream>>>(
        (const char *)in, (const IdxT *)idx, (char *)out, IB, OB, (uint32_t)row_bytes, rows_per_tile,
        tiles_per_a, num_tiles, status);
    return check_launch();
  }
  const uintptr_t both = reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) |
                         (uintptr_t)row_bytes;
  // paths 3 .. 6 (measurement): the persistent vector kernel with 8 or 16 rows in flight per thread
  if (path >= 3 && path <= 6) {
    if (both % 16 != 0 || IB >= 0x7fffffffLL)
      return B200_ERR_ALIGNMENT;
    switch (path) {
    case 3: return launch_gather_vec<uint4, IdxT, 8>(in, idx, out, A, IB, OB, row_bytes, 3, status, stream);
    case 4: return launch_gather_vec<uint4, IdxT, 8>(in, idx, out, A, IB, OB, row_bytes, 4, status, stream);
    case 5: return launch_gather_vec<uint4, IdxT, 16>(in, idx, out, A, IB, OB, row_bytes, 2, status, stream);
    default: return launch_gather_vec<uint4, IdxT, 4>(in, idx, out, A, IB, OB, row_bytes, 6, status, stream);
    }
  }
  // paths 7 .. 10: the tensor-map gather, 64-, 128- and 32-row tiles, and tiles of 8 KiB
  if (path >= 7 && path <= 10) {
    const int64_t total_rows = A * IB;
    // a tensor copy lands on a 128-byte boundary of shared memory: four rows must be a multiple of that
    if (!bulk_ok || row_bytes % 32 != 0 || row_bytes > 1024 || row_bytes < 64 || total_rows >= 0x7fffffffLL)
      return B200_ERR_ALIGNMENT;
    CUtensorMap map;
    const uint64_t dims[2] = {(uint64_t)(row_bytes / 4), (uint64_t)total_rows};
    const uint64_t strides[1] = {(uint64_t)row_bytes};
    const uint32_t box[2] = {(uint32_t)(row_bytes / 4), 1};
    if (int rc = make_tensor_map(&map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(in), dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
    int rows_per_tile = (int)std::min<int64_t>(path == 7 ? 64 : path == 8 ? 128 : path == 9 ? 32 : std::max<int64_t>(8, 8192 / row_bytes), 32768 / row_bytes);
    rows_per_tile = std::max(4, rows_per_tile & ~3);
    const int64_t tiles_per_a = ceil_div<int64_t>(OB, rows_per_tile);
    const int64_t num_tiles = tiles_per_a * A;
    const size_t smem = (size_t)kGatherStages * rows_per_tile * row_bytes;
    if (int rc = check_cuda(cudaFuncSetAttribute(gather_rows_g4_kernel<IdxT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 32768)))
      return rc;
    const int ctas_per_sm = (int)std::max<size_t>(1, std::min<size_t>(8, (200 * 1024) / (smem + 1024)));
    const unsigned grid = (unsigned)std::min<int64_t>(num_tiles, (int64_t)kNumSMs * ctas_per_sm);
    return launch_pdl(gather_rows_g4_kernel<IdxT>, dim3(grid), dim3(32), smem, stream, map, (const IdxT *)idx, (char *)out,
                      IB, OB, total_rows, (uint32_t)row_bytes, rows_per_tile, tiles_per_a, num_tiles, status);
  }
  if (both % 16 == 0)
    return launch_gather_generic<uint4, IdxT>(in, idx, out, A, IB, OB, row_bytes, status, stream);
  if (both % 8 == 0)
    return launch_gather_generic<uint2, IdxT>(in, idx, out, A, IB, OB, row_bytes, status, stream);
  if (both % 4 == 0)
    return launch_gather_generic<uint32_t, IdxT>(in, idx, out, A, IB, OB, row_bytes, status, stream);
  if (both % 2 == 0)
    return launch_gather_generic<uint16_t, IdxT>(in, idx, out, A, IB, OB, row_bytes, status, stream);
  return launch_gather_generic<uint8_t, IdxT>(in, idx, out, A, IB, OB, row_bytes, status, stream);
}

// =============================================================================
// scatter-add
// =============================================================================
// Stable LSD radix sort of (row index, position).  Digits are up to 10 bits wide (a table of
// a million rows sorts in two passes); a pass is a scan kernel and a scatter kernel, and the
// scatter kernel of one pass counts the digits of the next pass on the fly (per destination
// tile, with global atomics: the counts are exact whatever the order), so that only the first
// pass needs a histogram kernel of its own.  Every kernel of the chain is launched with
// programmatic dependent launch: its blocks are resident and waiting when its predecessor ends.
constexpr int kMaxRadixBits = 10;
constexpr int kMaxRadix = 1 << kMaxRadixBits;
constexpr int kSortTile = 2048; // keys per block: 8 warps x 8 rounds x 32 lanes
constexpr int kChunk = 32;      // sorted entries per warp in the accumulate pass

__device__ __forceinline__ uint32_t key_of_index(int64_t i, int64_t rows, int *status) {
  if (i < 0 || i >= rows) {
    if (status)
      *status = 1;
    return (uint32_t)rows; // sorts after every valid row, skipped later
  }
  return (uint32_t)i;
}

// First pass only: int64 indices -> keys, and the per-tile histogram of the first digit.
// hist: [digit][tile].
__global__ void __launch_bounds__(256)
    radix_first_hist_kernel(const int64_t *__restrict__ idx, uint32_t *__restrict__ keys,
                            uint32_t *__restrict__ hist, int64_t n, int64_t rows, int radix, int ntiles,
                            int *status, uint32_t *leader_count) {
  __shared__ uint32_t sh[kMaxRadix];
  pdl_wait();
  pdl_launch_dependents();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    leader_count[0] = 0; // work-list counters of the accumulate passes, which run
    leader_count[1] = 0; // after the whole sort
  }
  for (int d = threadIdx.x; d < radix; d += 256)
    sh[d] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * kSortTile;
  const uint32_t lt = (1u << (threadIdx.x & 31)) - 1u;
  uint32_t digit[kSortTile / 256];
#pragma unroll
  for (int k = 0; k < kSortTile / 256; ++k) { // all loads first
    const int64_t i = base + k * 256 + threadIdx.x;
    digit[k] = 0xffffffffu;
    if (i < n) {
      const uint32_t key = key_of_index(idx[i], rows, status);
      keys[i] = key;
      digit[k] = key & (uint32_t)(radix - 1);
    }
  }
#pragma unroll
  for (int k = 0; k < kSortTile / 256; ++k) {
    // one atomic per distinct digit of the warp: a hot row would otherwise queue up on one counter
    const uint32_t peers = __match_any_sync(0xffffffffu, digit[k]);
    if (digit[k] != 0xffffffffu && (peers & lt) == 0)
      atomicAdd(&sh[digit[k]], (uint32_t)__popc(peers));
  }
  __syncthreads();
  for (int d = threadIdx.x; d < radix; d += 256)
    hist[(size_t)d * ntiles + blockIdx.x] = sh[d];
}

// One warp per digit: exclusive prefix of the digit's counts over the tiles, in place, and the
// digit's total.  The same warp clears the digit's row of the other histogram, which the
// scatter kernel of this pass fills for the next pass.
__global__ void __launch_bounds__(256)
    radix_scan_kernel(uint32_t *__restrict__ hist, uint32_t *__restrict__ totals,
                      uint32_t *__restrict__ hist_next, int radix, int next_radix, int ntiles) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int d = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (d < next_radix && hist_next)
    for (int t = lane; t < ntiles; t += 32)
      hist_next[(size_t)d * ntiles + t] = 0;
  if (d >= radix)
    return;
  uint32_t *row = hist + (size_t)d * ntiles;
  uint32_t carry = 0;
  for (int t0 = 0; t0 < ntiles; t0 += 32) {
    const int t = t0 + lane;
    const uint32_t v = t < ntiles ? row[t] : 0u;
    uint32_t incl = v;
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t u = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off)
        incl += u;
    }
    if (t < ntiles)
      row[t] = carry + incl - v;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0)
    totals[d] = carry;
}

// stable scatter of one digit; FIRST: the value of entry i is i itself
template <bool FIRST>
__global__ void __launch_bounds__(256)
    radix_scatter_kernel(const uint32_t *__restrict__ keys_in, const uint32_t *__restrict__ vals_in,
                         uint32_t *__restrict__ keys_out, uint32_t *__restrict__ vals_out,
                         const uint32_t *__restrict__ hist, const uint32_t *__restrict__ totals,
                         uint32_t *__restrict__ hist_next, int64_t n, int shift, int radix, int next_shift,
                         int next_radix, int ntiles) {
  __shared__ uint32_t whist[8][kMaxRadix];
  __shared__ uint32_t digit_base[kMaxRadix];
  __shared__ uint32_t warp_tot[8];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Everything the block reads from global memory is requested here, in one go: the digit totals, the
  // block's keys (and positions) and its column of the scanned histogram do not depend on one another, and
  // beside the table copy every round trip to memory waits behind the copy's queue.
  const int64_t base = (int64_t)blockIdx.x * kSortTile + warp * 256;
  uint32_t key[8], val[8], rank[8];
  uint32_t t[kMaxRadix / 256], hcol[kMaxRadix / 256];
#pragma unroll
  for (int k = 0; k < kMaxRadix / 256; ++k) {
    const int d = threadIdx.x * (kMaxRadix / 256) + k;
    t[k] = d < radix ? totals[d] : 0u;
    const int dc = threadIdx.x + k * 256;
    hcol[k] = dc < radix ? hist[(size_t)dc * ntiles + blockIdx.x] : 0u;
  }
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int64_t i = base + r * 32 + lane;
    const bool ok = i < n;
    key[r] = ok ? keys_in[i] : 0u;
    val[r] = ok ? (FIRST ? (uint32_t)i : vals_in[i]) : 0u;
  }
  for (int i = threadIdx.x; i < 8 * kMaxRadix; i += 256)
    (&whist[0][0])[i] = 0;
  // digit_base[d] = number of keys whose digit is below d: block-wide exclusive scan of the totals
  {
    uint32_t local = 0;
#pragma unroll
    for (int k = 0; k < kMaxRadix / 256; ++k)
      local += t[k];
    uint32_t incl = local;
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t u = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off)
        incl += u;
    }
    if (lane == 31)
      warp_tot[warp] = incl;
    __syncthreads();
    uint32_t run = incl - local;
    for (int w = 0; w < warp; ++w)
      run += warp_tot[w];
#pragma unroll
    for (int k = 0; k < kMaxRadix / 256; ++k) {
      digit_base[threadIdx.x * (kMaxRadix / 256) + k] = run;
      run += t[k];
    }
  }
  __syncthreads();
  const uint32_t lt = (1u << lane) - 1u;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int64_t i = base + r * 32 + lane;
    const bool ok = i < n;
    const uint32_t d = ok ? ((key[r] >> shift) & (radix - 1)) : 0xffffffffu;
    const uint32_t peers = __match_any_sync(0xffffffffu, d);
    uint32_t prefix = 0;
    if (ok)
      prefix = whist[warp][d];
    __syncwarp();
    if (ok && (peers & lt) == 0)
      whist[warp][d] = prefix + __popc(peers);
    __syncwarp();
    rank[r] = prefix + __popc(peers & lt);
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kMaxRadix / 256; ++k) {
    const int d = threadIdx.x + k * 256;
    if (d >= radix)
      break;
    uint32_t run = hcol[k] + digit_base[d];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const uint32_t c = whist[w][d];
      whist[w][d] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int64_t i = base + r * 32 + lane;
    const bool ok = i < n;
    uint32_t tag = 0xffffffffu; // counter of the next pass this entry adds to: (digit, destination tile)
    if (ok) {
      const uint32_t d = (key[r] >> shift) & (radix - 1);
      const uint32_t dst = whist[warp][d] + rank[r];
      keys_out[dst] = key[r];
      vals_out[dst] = val[r];
      tag = ((key[r] >> next_shift) & (next_radix - 1)) * (uint32_t)ntiles + dst / kSortTile;
    }
    if (hist_next) {
      // one atomic per distinct counter of the warp: thousands of equal keys (a hot row) would
      // otherwise queue up on one address
      const uint32_t peers = __match_any_sync(0xffffffffu, tag);
      if (ok && (peers & lt) == 0)
        atomicAdd(&hist_next[tag], (uint32_t)__popc(peers));
    }
  }
}

// The table copy runs beside the index sort.  It moves 32 bytes per load and marks its lines
// first to go in L2 on both sides: the table streams through L2 once and should not push out
// the few megabytes the sort kernels beside it keep going back to.  (Measured alternatives: a
// persistent copy grid that keeps only the bandwidth-delay product in flight, 2 .. 16 blocks per
// SM, made the whole op slower, 147 .. 165 us against 139 us: a kernel without shared memory
// that never leaves its SMs also keeps kernels with another shared-memory carve-out from
// starting on them until it ends.  What slows the sort beside the copy is queueing: the copy keeps
// about 37 MB in flight, which at the copy's own bandwidth is 5 .. 6 us in front of every access of the
// sort's chain of dependent accesses.  Also measured and not kept: the accumulate passes beside the copy
// with the copy leaving out the rows that some index names, 144 .. 165 us against 141 .. 145 us; the sort
// as one kernel in a cluster of 16 blocks that keeps the list in distributed shared memory, 80 .. 90 us
// alone against 50 us for the chain of kernels: scattered 8-byte stores from 16 SMs only.)
struct alignas(32) Vec32 {
  uint64_t a, b, c, d;
};
__device__ __forceinline__ Vec32 ld_stream_v32(const Vec32 *p) {
  Vec32 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v4.b64 {%0,%1,%2,%3}, [%4];"
               : "=l"(v.a), "=l"(v.b), "=l"(v.c), "=l"(v.d)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream_v32(Vec32 *p, const Vec32 &v) {
  asm volatile("st.global.L1::no_allocate.L2::evict_first.v4.b64 [%0], {%1,%2,%3,%4};" ::"l"(p), "l"(v.a), "l"(v.b),
               "l"(v.c), "l"(v.d)
               : "memory");
}

// 1024 threads, four 32-byte vectors each (blocks of 256 threads measured 3 % slower on the whole op)
constexpr int kCopyThreads = 1024;
__global__ void __launch_bounds__(kCopyThreads)
    copy_table_kernel(const Vec32 *__restrict__ in, Vec32 *__restrict__ out, int64_t nvec) {
  const int64_t i = (int64_t)blockIdx.x * (4 * kCopyThreads) + threadIdx.x;
  if (i + 3 * kCopyThreads < nvec) {
    const Vec32 a = ld_stream_v32(in + i), b = ld_stream_v32(in + i + kCopyThreads),
                c = ld_stream_v32(in + i + 2 * kCopyThreads), d = ld_stream_v32(in + i + 3 * kCopyThreads);
    st_stream_v32(out + i, a), st_stream_v32(out + i + kCopyThreads, b), st_stream_v32(out + i + 2 * kCopyThreads, c),
        st_stream_v32(out + i + 3 * kCopyThreads, d);
  } else {
    for (int64_t k = 0, j = i; k < 4; ++k, j += kCopyThreads)
      if (j < nvec)
        out[j] = in[j];
  }
}

// ---- accumulate pass --------------------------------------------------------
// LV = elements per lane per feature tile (a lane loads LV * sizeof(T) bytes).
template <typename T, int LV> struct LaneVec {
  T v[LV];
};

template <typename T, int LV> struct LaneRaw {
  using type = typename std::conditional<
      LV * sizeof(T) == 16, uint4,
      typename std::conditional<LV * sizeof(T) == 8, uint2,
                                typename std::conditional<LV * sizeof(T) == 4, uint32_t, uint16_t>::type>::type>::type;
};
template <typename T, int LV>
__device__ __forceinline__ typename LaneRaw<T, LV>::type load_raw(const T *p) {
  return *reinterpret_cast<const typename LaneRaw<T, LV>::type *>(p);
}
template <typename T, int LV>
__device__ __forceinline__ void unpack_raw(const typename LaneRaw<T, LV>::type &raw, float (&f)[LV]) {
  const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
  for (int j = 0; j < LV; ++j)
    f[j] = Elt<T>::to_f32(e[j]);
}

template <typename T, int LV>
__device__ __forceinline__ void load_lane(const T *p, float (&f)[LV]) {
  using Raw = typename std::conditional<
      LV * sizeof(T) == 16, uint4,
      typename std::conditional<LV * sizeof(T) == 8, uint2,
                                typename std::conditional<LV * sizeof(T) == 4, uint32_t, uint16_t>::type>::type>::type;
  Raw raw = *reinterpret_cast<const Raw *>(p);
  const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
  for (int j = 0; j < LV; ++j)
    f[j] = Elt<T>::to_f32(e[j]);
}

template <typename T, int LV>
__device__ __forceinline__ void store_lane(T *p, const float (&f)[LV]) {
  using Raw = typename std::conditional<
      LV * sizeof(T) == 16, uint4,
      typename std::conditional<LV * sizeof(T) == 8, uint2,
                                typename std::conditional<LV * sizeof(T) == 4, uint32_t, uint16_t>::type>::type>::type;
  Raw raw;
  T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
  for (int j = 0; j < LV; ++j)
    e[j] = Elt<T>::from_f32(f[j]);
  *reinterpret_cast<Raw *>(p) = raw;
}

// A run that starts in a chunk and continues into the next one is finished by the span pass: the
// chunk goes on one of its two work lists.  leaders[0] / leaders[1] = lengths of the short and the
// long list, leaders[64 + i] = short entries (the run goes on into at most 31 further chunks),
// leaders[64 + nchunks + i] = long entries.  All lanes of the warp call this.
__device__ __forceinline__ void register_leader(const uint32_t *__restrict__ keys, uint32_t *__restrict__ leaders,
                                                int64_t chunk, int64_t nchunks, uint32_t first_key, uint32_t last_key,
                                                uint32_t prev_key, uint32_t next_key, uint32_t invalid, int lane) {
  if (last_key == invalid || last_key != next_key || (first_key == last_key && first_key == prev_key))
    return; // uniform over the warp
  const int64_t probe = chunk + 1 + lane;
  const unsigned hits = __ballot_sync(0xffffffffu, probe < nchunks && keys[probe * kChunk] == last_key);
  if (lane == 0) {
    if (hits == 0xffffffffu)
      leaders[64 + nchunks + atomicAdd(&leaders[1], 1u)] = (uint32_t)chunk;
    else
      leaders[64 + atomicAdd(&leaders[0], 1u)] = (uint32_t)chunk;
  }
}

// One warp per chunk of kChunk sorted entries.  part: [nchunks][2][feature] f32.
// Entries are handled 8 at a time: the 8 update rows, and the table rows of the
// runs that end (and are complete) inside those 8 entries, are all loaded before
// any of them is used, so a warp keeps up to 16 row loads in flight.
template <typename T, int LV>
__global__ void __launch_bounds__(256)
    scatter_chunk_kernel(const T *in, const T *__restrict__ upd, T *out,
                         const uint32_t *__restrict__ keys, const uint32_t *__restrict__ vals,
                         float *__restrict__ part, uint32_t *__restrict__ leaders, int64_t n,
                         int64_t rows, int64_t feature) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t chunk = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t e0 = chunk * kChunk;
  if (e0 >= n)
    return;
  const int cnt = (int)min((int64_t)kChunk, n - e0);
  const uint32_t invalid = (uint32_t)rows;
  const uint32_t my_key = lane < cnt ? keys[e0 + lane] : 0xffffffffu;
  const uint32_t my_pos = lane < cnt ? vals[e0 + lane] : 0u;
  const uint32_t prev_key = e0 > 0 ? keys[e0 - 1] : 0xffffffffu;
  const uint32_t next_key = e0 + kChunk < n ? keys[e0 + kChunk] : 0xffffffffu;
  const uint32_t first_key = __shfl_sync(0xffffffffu, my_key, 0);
  const uint32_t last_key = __shfl_sync(0xffffffffu, my_key, cnt - 1);
  // per entry: does a run end here, and is that run complete inside this chunk?
  const uint32_t key_after = __shfl_down_sync(0xffffffffu, my_key, 1);
  const bool my_end = lane < cnt && (lane == cnt - 1 || key_after != my_key);
  const bool my_open = (my_key == first_key && first_key == prev_key) ||
                       (my_key == last_key && last_key == next_key);
  const uint32_t end_mask = __ballot_sync(0xffffffffu, my_end);
  const uint32_t closed_mask = __ballot_sync(0xffffffffu, my_end && !my_open && my_key != invalid);
  float *part0 = part + (size_t)chunk * 2 * feature;
  float *part1 = part0 + feature;
  register_leader(keys, leaders, chunk, ceil_div<int64_t>(n, kChunk), first_key, last_key, prev_key, next_key, invalid,
                  lane);

  // uniform over the warp (it contains shuffles); lanes past the end of a short
  // row only skip their loads and stores
  for (int64_t fbase = 0; fbase < feature; fbase += 32 * LV) {
    const int64_t f0 = fbase + (int64_t)lane * LV;
    const bool lane_on = f0 < feature;
    float acc[LV];
#pragma unroll
    for (int j = 0; j < LV; ++j)
      acc[j] = 0.f;
    for (int i0 = 0; i0 < cnt; i0 += 8) {
      // raw 16-bit/32-bit lanes stay packed until they are used: fewer registers,
      // more warps per SM, more loads in flight
      typename LaneRaw<T, LV>::type x[8], base[8];
      uint32_t k[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u;
        k[u] = __shfl_sync(0xffffffffu, my_key, i & 31);
        const uint32_t pos = __shfl_sync(0xffffffffu, my_pos, i & 31);
        const bool live = i < cnt && k[u] != invalid && lane_on;
        x[u] = typename LaneRaw<T, LV>::type{};
        base[u] = typename LaneRaw<T, LV>::type{};
        if (live)
          x[u] = load_raw<T, LV>(upd + (size_t)pos * feature + f0);
        if (live && ((closed_mask >> i) & 1u))
          base[u] = load_raw<T, LV>(in + (size_t)k[u] * feature + f0);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u;
        if (i >= cnt)
          break;
        if (k[u] == invalid || !lane_on)
          continue;
        float xf[LV];
        unpack_raw<T, LV>(x[u], xf);
#pragma unroll
        for (int j = 0; j < LV; ++j)
          acc[j] += xf[j];
        if ((end_mask >> i) & 1u) {
          if ((closed_mask >> i) & 1u) {
            float bf[LV];
            unpack_raw<T, LV>(base[u], bf);
#pragma unroll
            for (int j = 0; j < LV; ++j)
              bf[j] += acc[j];
            store_lane<T, LV>(out + (size_t)k[u] * feature + f0, bf);
          } else {
            // first run of the chunk -> slot 0, otherwise (last run) -> slot 1
            float *dst = (k[u] == first_key ? part0 : part1) + f0;
#pragma unroll
            for (int j = 0; j < LV; ++j)
              dst[j] = acc[j];
          }
#pragma unroll
          for (int j = 0; j < LV; ++j)
            acc[j] = 0.f;
        }
      }
    }
  }
}

// The same pass for rows that are multiples of 32 bytes: the 32 update rows of a chunk, and the
// table rows of the runs that end inside it, are fetched into the warp's shared-memory buffers by
// the tensor-map gather (cp.async.bulk.tensor, tile::gather4: four rows per instruction, named by
// their row coordinates), all of them in flight at once and none of them held in registers; the
// warp then adds the rows up from shared memory, in the order of the sorted list.  A row is
// handled in tiles of 256 bytes (8 bytes per lane).  Rows that are not needed (an entry out of
// range, a run that does not end here) are named by a coordinate past the end of the map, which
// reads zeros and costs no memory traffic.
// Shared memory: [warp][update rows | table rows][32 rows][tile] = 16 KiB per warp.
constexpr int kStagedWarps = 4;
constexpr int kStagedTileBytes = 256;
constexpr size_t kStagedSmemPerWarp = 2 * kChunk * kStagedTileBytes;

template <typename T>
__global__ void __launch_bounds__(kStagedWarps * 32)
    scatter_chunk_staged_kernel(const __grid_constant__ CUtensorMap upd_map,
                                const __grid_constant__ CUtensorMap in_map, T *out,
                                const uint32_t *__restrict__ keys, const uint32_t *__restrict__ vals,
                                float *__restrict__ part, uint32_t *__restrict__ leaders, int64_t n,
                                int64_t rows, int64_t feature, int *status) {
  constexpr int LV = 8 / (int)sizeof(T); // elements per lane per tile
  extern __shared__ __align__(1024) unsigned char staged_smem[];
  __shared__ uint64_t bars[kStagedWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    mbar_init(&bars[warp], 1);
    mbar_fence_init();
  }
  __syncwarp();
  pdl_wait();
  pdl_launch_dependents();
  const int64_t chunk = (int64_t)blockIdx.x * kStagedWarps + warp;
  const int64_t e0 = chunk * kChunk;
  if (e0 >= n)
    return;
  unsigned char *upd_s = staged_smem + (size_t)warp * kStagedSmemPerWarp;
  const int cnt = (int)min((int64_t)kChunk, n - e0);
  const uint32_t invalid = (uint32_t)rows;
  const uint32_t my_key = lane < cnt ? keys[e0 + lane] : 0xffffffffu;
  const uint32_t my_pos = lane < cnt ? vals[e0 + lane] : 0u;
  const uint32_t prev_key = e0 > 0 ? keys[e0 - 1] : 0xffffffffu;
  const uint32_t next_key = e0 + kChunk < n ? keys[e0 + kChunk] : 0xffffffffu;
  const uint32_t first_key = __shfl_sync(0xffffffffu, my_key, 0);
  const uint32_t last_key = __shfl_sync(0xffffffffu, my_key, cnt - 1);
  const uint32_t key_after = __shfl_down_sync(0xffffffffu, my_key, 1);
  const bool my_end = lane < cnt && (lane == cnt - 1 || key_after != my_key);
  const bool my_open = (my_key == first_key && first_key == prev_key) ||
                       (my_key == last_key && last_key == next_key);
  const bool my_live = lane < cnt && my_key != invalid;
  const bool my_closed = my_end && !my_open && my_live;
  const uint32_t end_mask = __ballot_sync(0xffffffffu, my_end);
  const uint32_t closed_mask = __ballot_sync(0xffffffffu, my_closed);
  const uint32_t live_mask = __ballot_sync(0xffffffffu, my_live);
  float *part0 = part + (size_t)chunk * 2 * feature;
  float *part1 = part0 + feature;
  register_leader(keys, leaders, chunk, ceil_div<int64_t>(n, kChunk), first_key, last_key, prev_key, next_key, invalid,
                  lane);

  // row coordinates of the two gathers; a row that is not needed lies past the end of its map
  const int upd_row = my_live ? (int)my_pos : (int)min(n, (int64_t)0x7fffffff);
  const int in_row = my_closed ? (int)my_key : (int)rows;
  const int64_t row_bytes = feature * (int64_t)sizeof(T);
  const int live_quads = (32 - __clz(live_mask | 1u) + 3) >> 2; // quads of entries holding a live one
  // the box of both maps is one row of `pitch` bytes, which is also the row pitch in shared memory;
  // the last tile of a row may be narrower: its columns past the end of the row read zeros
  const int pitch = (int)min((int64_t)kStagedTileBytes, row_bytes);
  unsigned char *base_s = upd_s + kChunk * pitch;
  uint32_t phase = 0;
  for (int64_t tb = 0; tb < row_bytes; tb += kStagedTileBytes, phase ^= 1u) {
    const int tile_bytes = (int)min((int64_t)kStagedTileBytes, row_bytes - tb);
    if (tb > 0) { // the previous tile has been read out of the buffers by every lane
      __syncwarp();
      fence_proxy_async_smem();
    }
    // lanes 0 .. 7 fetch the update rows of their quad, lanes 8 .. 15 the table rows of theirs
    const int q = lane & 7;
    int r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) { // what is exchanged is the SOURCE lane's value: both are sent, the receiver picks
      const int ru = __shfl_sync(0xffffffffu, upd_row, 4 * q + u);
      const int ri = __shfl_sync(0xffffffffu, in_row, 4 * q + u);
      r[u] = lane < 8 ? ru : ri;
    }
    const int r0 = r[0], r1 = r[1], r2 = r[2], r3 = r[3];
    const bool quad_closed = ((closed_mask >> (4 * q)) & 0xfu) != 0;
    const bool issue_upd = lane < 8 && q < live_quads;
    const bool issue_in = lane >= 8 && lane < 16 && quad_closed;
    const int nq = __popc(__ballot_sync(0xffffffffu, issue_upd || issue_in));
    if (lane == 0)
      mbar_arrive_expect_tx(&bars[warp], (uint32_t)nq * 4u * (uint32_t)pitch);
    __syncwarp();
    if (issue_upd)
      tma_gather4_2d(upd_s + q * 4 * pitch, &upd_map, (int)(tb >> 2), r0, r1, r2, r3, &bars[warp]);
    if (issue_in)
      tma_gather4_2d(base_s + q * 4 * pitch, &in_map, (int)(tb >> 2), r0, r1, r2, r3, &bars[warp]);
    if (!__all_sync(0xffffffffu, mbar_wait(&bars[warp], phase))) {
      if (status && lane == 0)
        *status = 2; // a copy never arrived: give up instead of spinning
      return;
    }
    const bool lane_on = lane * 8 < tile_bytes;
    const int64_t f0 = tb / (int64_t)sizeof(T) + (int64_t)lane * LV;
    float acc[LV];
#pragma unroll
    for (int j = 0; j < LV; ++j)
      acc[j] = 0.f;
    // this lane's piece of all 32 update rows, read before any of them is used: the additions below
    // then wait on no shared-memory latency
    uint2 xr[kChunk];
#pragma unroll
    for (int i = 0; i < kChunk; ++i)
      xr[i] = lane_on ? *reinterpret_cast<const uint2 *>(upd_s + i * pitch + lane * 8) : make_uint2(0u, 0u);
#pragma unroll
    for (int i = 0; i < kChunk; ++i) {
      if (i >= cnt || !((live_mask >> i) & 1u))
        continue;
      {
        float xf[LV];
        unpack_raw<T, LV>(xr[i], xf);
#pragma unroll
        for (int j = 0; j < LV; ++j)
          acc[j] += xf[j];
      }
      if ((end_mask >> i) & 1u) {
        const uint32_t k = __shfl_sync(0xffffffffu, my_key, i);
        if (lane_on) {
          if ((closed_mask >> i) & 1u) {
            float bf[LV];
            unpack_raw<T, LV>(*reinterpret_cast<const uint2 *>(base_s + i * pitch + lane * 8), bf);
#pragma unroll
            for (int j = 0; j < LV; ++j)
              bf[j] += acc[j];
            store_lane<T, LV>(out + (size_t)k * feature + f0, bf);
          } else {
            float *dst = (k == first_key ? part0 : part1) + f0;
#pragma unroll
            for (int j = 0; j < LV; ++j)
              dst[j] = acc[j];
          }
        }
#pragma unroll
        for (int j = 0; j < LV; ++j)
          acc[j] = 0.f;
      }
    }
  }
}

// Finishes the runs that cross chunk borders, from the two work lists the chunk pass wrote
// (register_leader).  One launch, blocks of 32 warps: the first `short_blocks` blocks give a
// warp to every short entry (the partials of up to 31 following chunks added in chunk order, eight
// loads in flight); the other blocks take one long entry at a time: the block counts how many
// following chunks the run continues into, each warp adds the slot-0 partials of a contiguous
// slice of those chunks, and warp 0 adds the 32 slice sums in order to the run's own partial
// and the table row.  Which warp or block handles which entry does not affect the result.
template <typename T, int LV>
__global__ void __launch_bounds__(1024)
    scatter_span_kernel(const T *in, T *out, const uint32_t *__restrict__ keys, const float *__restrict__ part,
                        const uint32_t *__restrict__ leaders, int64_t n, int64_t feature, int short_blocks) {
  __shared__ float sm[32][32 * LV];
  constexpr int U = LV > 4 ? 4 : 8; // rows of partials in flight per lane: 32 floats
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t nchunks = ceil_div<int64_t>(n, kChunk);
  if ((int)blockIdx.x < short_blocks) {
    const uint32_t nlead = leaders[0];
    const int64_t warps = (int64_t)short_blocks * 32;
    for (int64_t l = (int64_t)blockIdx.x * 32 + warp; l < nlead; l += warps) {
      const int64_t chunk = leaders[64 + l];
      const int64_t e0 = chunk * kChunk;
      const uint32_t key = keys[min(n, e0 + kChunk) - 1];
      const int first_slot = keys[e0] == key ? 0 : 1;
      const int64_t probe = chunk + 1 + lane;
      const unsigned hits = __ballot_sync(0xffffffffu, probe < nchunks && keys[probe * kChunk] == key);
      const int extra = __popc(hits); // keys are sorted: the hits are the low bits; at most 31 here
      for (int64_t fbase = 0; fbase < feature; fbase += 32 * LV) {
        const int64_t f0 = fbase + (int64_t)lane * LV;
        if (f0 >= feature)
          continue;
        float base[LV], sum[LV];
        load_lane<T, LV>(in + (size_t)key * feature + f0, base);
        const float *p = part + ((size_t)chunk * 2 + first_slot) * feature + f0;
#pragma unroll
        for (int j = 0; j < LV; ++j)
          sum[j] = p[j];
        for (int c0 = 1; c0 <= extra; c0 += U) {
          float q[U][LV];
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (c0 + u <= extra) {
              const float *qp = part + (size_t)(chunk + c0 + u) * 2 * feature + f0;
#pragma unroll
              for (int j = 0; j < LV; ++j)
                q[u][j] = qp[j];
            }
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (c0 + u <= extra) {
#pragma unroll
              for (int j = 0; j < LV; ++j)
                sum[j] += q[u][j];
            }
        }
#pragma unroll
        for (int j = 0; j < LV; ++j)
          base[j] += sum[j];
        store_lane<T, LV>(out + (size_t)key * feature + f0, base);
      }
    }
    return;
  }
  const uint32_t nlead = leaders[1];
  const uint32_t long_blocks = gridDim.x - short_blocks;
  for (uint32_t l = blockIdx.x - short_blocks; l < nlead; l += long_blocks) {
    const int64_t chunk = leaders[64 + nchunks + l];
    const int64_t e0 = chunk * kChunk;
    const uint32_t key = keys[min(n, e0 + kChunk) - 1];
    const int first_slot = keys[e0] == key ? 0 : 1;
    // number of following chunks that start with this key (keys are sorted, so
    // the predicate is monotone over the chunks)
    int64_t extra = 0;
    for (int64_t c = chunk + 1; c < nchunks; c += 1024) {
      const int64_t mine = c + threadIdx.x;
      const int hit = __syncthreads_count(mine < nchunks && keys[mine * kChunk] == key);
      extra += hit;
      if (hit < 1024)
        break;
    }
    const int64_t per = ceil_div<int64_t>(extra, 32);
    const int64_t c0 = chunk + 1 + warp * per;
    const int64_t c1 = min(chunk + 1 + extra, c0 + per);
    for (int64_t fbase = 0; fbase < feature; fbase += 32 * LV) {
      const int64_t f0 = fbase + (int64_t)lane * LV;
      const bool lane_on = f0 < feature;
      float total[LV];
#pragma unroll
      for (int j = 0; j < LV; ++j)
        total[j] = 0.f;
      if (lane_on) {
        for (int64_t c = c0; c < c1; c += U) { // U rows of partials in flight, the last batch predicated
          float q[U][LV];
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (c + u < c1) {
              const float *p = part + (size_t)(c + u) * 2 * feature + f0;
#pragma unroll
              for (int j = 0; j < LV; ++j)
                q[u][j] = p[j];
            }
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (c + u < c1) {
#pragma unroll
              for (int j = 0; j < LV; ++j)
                total[j] += q[u][j];
            }
        }
      }
#pragma unroll
      for (int j = 0; j < LV; ++j)
        sm[warp][lane * LV + j] = total[j];
      __syncthreads();
      if (warp == 0 && lane_on) {
        float base[LV], sum[LV];
        load_lane<T, LV>(in + (size_t)key * feature + f0, base);
        const float *p = part + ((size_t)chunk * 2 + first_slot) * feature + f0;
#pragma unroll
        for (int j = 0; j < LV; ++j)
          sum[j] = p[j];
        for (int w = 0; w < 32; ++w)
#pragma unroll
          for (int j = 0; j < LV; ++j)
            sum[j] += sm[w][lane * LV + j];
#pragma unroll
        for (int j = 0; j < LV; ++j)
          base[j] += sum[j];
        store_lane<T, LV>(out + (size_t)key * feature + f0, base);
      }
      __syncthreads();
    }
  }
}

struct ScatterPlan {
  int64_t nblocks, nchunks;
  int passes, digit_bits;
  size_t off_keys[2], off_vals[2], off_hist[2], off_totals, off_part, off_leaders, total;
};

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

ScatterPlan make_scatter_plan(int64_t rows, int64_t n, int64_t feature) {
  ScatterPlan p{};
  p.nblocks = ceil_div<int64_t>(n, kSortTile);
  p.nchunks = ceil_div<int64_t>(n, kChunk);
  int bits = 1; // of the largest key, which is `rows` itself (the key of an index out of range)
  while (bits < 32 && ((uint64_t)rows >> bits) != 0)
    ++bits;
  p.passes = (bits + kMaxRadixBits - 1) / kMaxRadixBits;
  p.digit_bits = (bits + p.passes - 1) / p.passes;
  size_t off = 0;
  for (int i = 0; i < 2; ++i) {
    p.off_keys[i] = off;
    off += align256((size_t)n * 4);
    p.off_vals[i] = off;
    off += align256((size_t)n * 4);
  }
  for (int i = 0; i < 2; ++i) {
    p.off_hist[i] = off;
    off += align256((size_t)kMaxRadix * p.nblocks * 4);
  }
  p.off_totals = off;
  off += align256((size_t)kMaxRadix * 4);
  p.off_part = off;
  off += align256((size_t)p.nchunks * 2 * feature * 4);
  p.off_leaders = off; // two counters, then two lists of chunk ids (see the span kernels)
  off += align256((size_t)(64 + 2 * p.nchunks) * 4);
  p.total = off;
  return p;
}

// measurement override of the accumulate pass (b200_index_put_tune): 0 = rule, 1 = rows through
// registers, 2 = rows staged in shared memory
int g_chunk_path_override = 0;

template <typename T, int LV>
int launch_scatter_tail(bool staged, const T *in, const T *upd, T *out, const uint32_t *keys, const uint32_t *vals,
                        float *part, uint32_t *leaders, int64_t n, int64_t rows, int64_t feature, int *status,
                        cudaStream_t stream) {
  const int64_t nchunks = ceil_div<int64_t>(n, kChunk);
  if (staged) {
    // two-dimensional maps over the update rows and the table rows, 32-bit columns, box = one
    // tile of one row
    const int64_t row_bytes = feature * (int64_t)sizeof(T);
    const uint32_t box_cols = (uint32_t)(std::min<int64_t>(row_bytes, kStagedTileBytes) / 4);
    CUtensorMap upd_map, in_map;
    const uint64_t strides[1] = {(uint64_t)row_bytes};
    const uint32_t box[2] = {box_cols, 1};
    const uint64_t upd_dims[2] = {(uint64_t)(row_bytes / 4), (uint64_t)n};
    const uint64_t in_dims[2] = {(uint64_t)(row_bytes / 4), (uint64_t)rows};
    if (int rc = make_tensor_map(&upd_map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<T *>(upd), upd_dims, strides,
                                 box, CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
    if (int rc = make_tensor_map(&in_map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<T *>(in), in_dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
    const size_t smem = kStagedWarps * kStagedSmemPerWarp + 1024;
    // the attribute belongs to the current device's context: set on every call (a host-side table write)
    if (int rc = check_cuda(cudaFuncSetAttribute(scatter_chunk_staged_kernel<T>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)))
      return rc;
    if (int rc = launch_pdl(scatter_chunk_staged_kernel<T>, dim3((unsigned)ceil_div<int64_t>(nchunks, kStagedWarps)),
                            dim3(kStagedWarps * 32), smem, stream, upd_map, in_map, out, keys, vals, part, leaders, n,
                            rows, feature, status))
      return rc;
  } else {
    if (int rc = launch_pdl(scatter_chunk_kernel<T, LV>, dim3((unsigned)ceil_div<int64_t>(nchunks, 8)), dim3(256), 0,
                            stream, in, upd, out, keys, vals, part, leaders, n, rows, feature))
      return rc;
  }
  const int short_blocks = (int)std::min<int64_t>(ceil_div<int64_t>(nchunks, 32), kNumSMs);
  const int long_blocks = (int)std::min<int64_t>(ceil_div<int64_t>(nchunks, 32), kNumSMs);
  return launch_pdl(scatter_span_kernel<T, LV>, dim3((unsigned)(short_blocks + long_blocks)), dim3(1024), 0, stream, in,
                    out, keys, (const float *)part, (const uint32_t *)leaders, n, feature, short_blocks);
}

// The index sort does not depend on the table copy, so the two run side by side:
// the sort is forked onto a helper stream and joined before the accumulate pass.
// One helper stream (and its two events) is kept per (device, caller stream): created
// by b200_index_put_prepare, or by the first call that needs them, and destroyed by
// b200_index_put_release.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};

std::mutex g_side_mu;
std::map<std::pair<int, cudaStream_t>, SideStream> g_side_pool;

int get_side_stream(cudaStream_t user, SideStream *out) {
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev)))
    return rc;
  std::lock_guard<std::mutex> lock(g_side_mu);
  auto it = g_side_pool.find({dev, user});
  if (it == g_side_pool.end()) {
    SideStream s;
    // Highest priority: the helper stream carries the sort, a chain of small kernels, beside the
    // table copy, whose sixteen thousand blocks would otherwise sit in front of every one of
    // them in the block scheduler's queue.
    int least = 0, greatest = 0;
    if (int rc = check_cuda(cudaDeviceGetStreamPriorityRange(&least, &greatest)))
      return rc;
    if (int rc = check_cuda(cudaStreamCreateWithPriority(&s.stream, cudaStreamNonBlocking, greatest)))
      return rc;
    if (int rc = check_cuda(cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming)))
      return rc;
    if (int rc = check_cuda(cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming)))
      return rc;
    it = g_side_pool.emplace(std::make_pair(dev, user), s).first;
  }
  if (out)
    *out = it->second;
  return B200_OK;
}

int release_side_stream(cudaStream_t user) {
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev)))
    return rc;
  SideStream s;
  {
    std::lock_guard<std::mutex> lock(g_side_mu);
    auto it = g_side_pool.find({dev, user});
    if (it == g_side_pool.end())
      return B200_OK;
    s = it->second;
    g_side_pool.erase(it);
  }
  (void)cudaEventDestroy(s.fork);
  (void)cudaEventDestroy(s.join);
  return check_cuda(cudaStreamDestroy(s.stream)); // work already queued on it still completes
}

template <typename T>
int scatter_add(const T *in, const int64_t *idx, const T *upd, T *out, int64_t rows, int64_t n,
                int64_t feature, void *ws, size_t ws_bytes, int *status, cudaStream_t user_stream) {
  const size_t table_bytes = (size_t)rows * feature * sizeof(T);
  const ScatterPlan p = make_scatter_plan(rows, std::max<int64_t>(n, 1), feature);
  if (n > 0 && (!ws || ws_bytes < p.total))
    return B200_ERR_WORKSPACE;
  // fork: the sort runs on the helper stream while the caller's stream copies the table
  const bool fork = in != out && n > 0 && table_bytes >= (8u << 20);
  SideStream side;
  cudaStream_t stream = user_stream; // stream of the sort
  if (fork) {
    if (int rc = get_side_stream(user_stream, &side))
      return rc;
    if (int rc = check_cuda(cudaEventRecord(side.fork, user_stream)))
      return rc;
    if (int rc = check_cuda(cudaStreamWaitEvent(side.stream, side.fork, 0)))
      return rc;
    stream = side.stream;
  }
  if (in != out) {
    cudaStream_t stream = user_stream; // the copy always runs on the caller's stream
    if (table_bytes % 32 == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 31u) == 0) {
      const int64_t nvec = (int64_t)(table_bytes / 32);
      copy_table_kernel<<<(unsigned)ceil_div<int64_t>(nvec, 4 * kCopyThreads), kCopyThreads, 0, stream>>>(
          (const Vec32 *)in, (Vec32 *)out, nvec);
      if (int rc = check_launch())
        return rc;
    } else if (int rc = check_cuda(
                   cudaMemcpyAsync(out, in, table_bytes, cudaMemcpyDeviceToDevice, stream))) {
      return rc;
    }
  }
  if (n == 0)
    return B200_OK;
  char *w = static_cast<char *>(ws);
  uint32_t *keys[2] = {(uint32_t *)(w + p.off_keys[0]), (uint32_t *)(w + p.off_keys[1])};
  uint32_t *vals[2] = {(uint32_t *)(w + p.off_vals[0]), (uint32_t *)(w + p.off_vals[1])};
  uint32_t *hist[2] = {(uint32_t *)(w + p.off_hist[0]), (uint32_t *)(w + p.off_hist[1])};
  uint32_t *totals = (uint32_t *)(w + p.off_totals);
  float *part = (float *)(w + p.off_part);
  uint32_t *leaders = (uint32_t *)(w + p.off_leaders);
  const int nb = (int)p.nblocks;
  const int radix = 1 << p.digit_bits;
  if (int rc = launch_pdl(radix_first_hist_kernel, dim3(nb), dim3(256), 0, stream, idx, keys[0], hist[0], n, rows,
                          radix, nb, status, leaders))
    return rc;
  int cur = 0;
  for (int pass = 0; pass < p.passes; ++pass) {
    const int shift = pass * p.digit_bits;
    const bool has_next = pass + 1 < p.passes;
    uint32_t *h = hist[pass & 1], *h_next = has_next ? hist[(pass + 1) & 1] : nullptr;
    if (int rc = launch_pdl(radix_scan_kernel, dim3((unsigned)ceil_div<int64_t>(radix, 8)), dim3(256), 0, stream, h,
                            totals, h_next, radix, radix, nb))
      return rc;
    int rc;
    if (pass == 0)
      rc = launch_pdl(radix_scatter_kernel<true>, dim3(nb), dim3(256), 0, stream, (const uint32_t *)keys[cur],
                      (const uint32_t *)nullptr, keys[cur ^ 1], vals[cur ^ 1], (const uint32_t *)h,
                      (const uint32_t *)totals, h_next, n, shift, radix, shift + p.digit_bits, radix, nb);
    else
      rc = launch_pdl(radix_scatter_kernel<false>, dim3(nb), dim3(256), 0, stream, (const uint32_t *)keys[cur],
                      (const uint32_t *)vals[cur], keys[cur ^ 1], vals[cur ^ 1], (const uint32_t *)h,
                      (const uint32_t *)totals, h_next, n, shift, radix, shift + p.digit_bits, radix, nb);
    if (rc)
      return rc;
    cur ^= 1;
  }
  if (fork) { // join: the accumulate pass needs both the sorted list and the copied table
    if (int rc = check_cuda(cudaEventRecord(side.join, side.stream)))
      return rc;
    if (int rc = check_cuda(cudaStreamWaitEvent(user_stream, side.join, 0)))
      return rc;
  }
  stream = user_stream;
  // lane vector width: as wide as the row and the pointers allow, but keep 32 lanes busy
  const uintptr_t mis = reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) |
                        reinterpret_cast<uintptr_t>(upd) | (uintptr_t)(feature * sizeof(T));
  int lane_bytes = 16;
  while (lane_bytes > (int)sizeof(T) && (mis % lane_bytes != 0 || feature * (int64_t)sizeof(T) < 32LL * lane_bytes))
    lane_bytes >>= 1;
  const int lv = lane_bytes / (int)sizeof(T);
  // rows staged through shared memory whenever whole rows can be copied in 16-byte pieces
  // (four rows of a tile land on a 128-byte boundary of shared memory: rows are multiples of 32 bytes;
  // row coordinates are 32-bit)
  bool staged = mis % 16 == 0 && (feature * (int64_t)sizeof(T)) % 32 == 0 && rows < 0x7fffffffLL && n < 0x7fffffffLL;
  if (g_chunk_path_override == 1)
    staged = false;
  switch (lv) {
  case 8:
    if constexpr (sizeof(T) == 2)
      return launch_scatter_tail<T, 8>(staged, in, upd, out, keys[cur], vals[cur], part, leaders, n, rows, feature, status, stream);
    return B200_ERR_UNSUPPORTED;
  case 4:
    return launch_scatter_tail<T, 4>(staged, in, upd, out, keys[cur], vals[cur], part, leaders, n, rows, feature, status, stream);
  case 2:
    return launch_scatter_tail<T, 2>(staged, in, upd, out, keys[cur], vals[cur], part, leaders, n, rows, feature, status, stream);
  default:
    return launch_scatter_tail<T, 1>(staged, in, upd, out, keys[cur], vals[cur], part, leaders, n, rows, feature, status, stream);
  }
}

} // namespace
} // namespace b200

using namespace b200;

extern "C" int b200_index_select_path(int path, int elt_bytes, int idx_bytes, const void *in,
                                      const void *idx, void *out, int64_t A, int64_t IB, int64_t OB,
                                      int64_t C, int *status, cudaStream_t stream) {
  if (elt_bytes <= 0 || (idx_bytes != 4 && idx_bytes != 8) || A < 0 || IB < 0 || OB < 0 || C < 0)
    return B200_ERR_INVALID_ARG;
  if (A == 0 || OB == 0 || C == 0)
    return B200_OK;
  if (!in || !idx || !out)
    return B200_ERR_INVALID_ARG;
  const int64_t row_bytes = C * elt_bytes;
  if (idx_bytes == 8)
    return launch_gather<int64_t>(path, in, idx, out, A, IB, OB, row_bytes, status, stream);
  return launch_gather<uint32_t>(path, in, idx, out, A, IB, OB, row_bytes, status, stream);
}

extern "C" int b200_index_select(int elt_bytes, int idx_bytes, const void *in, const void *idx,
                                 void *out, int64_t A, int64_t IB, int64_t OB, int64_t C, int *status,
                                 cudaStream_t stream) {
  return b200_index_select_path(0, elt_bytes, idx_bytes, in, idx, out, A, IB, OB, C, status, stream);
}

extern "C" void b200_index_put_tune(int chunk_path) { g_chunk_path_override = chunk_path; }

extern "C" int b200_index_put_prepare(cudaStream_t stream) { return get_side_stream(stream, nullptr); }

extern "C" int b200_index_put_release(cudaStream_t stream) { return release_side_stream(stream); }

extern "C" size_t b200_index_put_workspace_bytes(int dtype, int64_t rows, int64_t index_count,
                                                 int64_t feature) {
  (void)dtype;
  if (rows <= 0 || index_count <= 0 || feature <= 0)
    return 0;
  return make_scatter_plan(rows, index_count, feature).total;
}

extern "C" int b200_index_put_add(int dtype, const void *in, const int64_t *idx, const void *upd,
                                  void *out, int64_t rows, int64_t index_count, int64_t feature,
                                  void *workspace, size_t workspace_bytes, int *status,
                                  cudaStream_t stream) {
  if (rows < 0 || index_count < 0 || feature < 0 || rows >= 0xffffffffLL ||
      index_count >= 0xffffffffLL)
    return B200_ERR_INVALID_ARG;
  if (rows == 0 || feature == 0)
    return B200_OK;
  if (!in || !out || (index_count > 0 && (!idx || !upd)))
    return B200_ERR_INVALID_ARG;
  switch (dtype) {
  case B200_F32:
    return scatter_add<float>((const float *)in, idx, (const float *)upd, (float *)out, rows,
                              index_count, feature, workspace, workspace_bytes, status, stream);
  case B200_F16:
    return scatter_add<__half>((const __half *)in, idx, (const __half *)upd, (__half *)out, rows,
                               index_count, feature, workspace, workspace_bytes, status, stream);
  case B200_BF16:
    return scatter_add<__nv_bfloat16>((const __nv_bfloat16 *)in, idx, (const __nv_bfloat16 *)upd,
                                      (__nv_bfloat16 *)out, rows, index_count, feature, workspace,
                                      workspace_bytes, status, stream);
  default:
    return B200_ERR_INVALID_ARG;
  }
}
