// mbarrier / bulk-copy (TMA) PTX wrappers for sm_100a.  No cluster multicast
// anywhere: every copy has exactly one destination CTA.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// One poll of the barrier.  The time hint lets the hardware park the thread until the phase
// completes (or the hint expires), so a waiting warp does not burn issue slots in a spin loop.
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n"
               ".reg .pred p;\n"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
               "selp.u32 %0, 1, 0, p;\n"
               "}\n"
               : "=r"(ok)
               : "r"(smem_addr(bar)), "r"(parity), "r"(20000u)
               : "memory");
  return ok != 0;
}

// Bounded wait: gives up after `limit` polls and returns false, so that a
// protocol error can never hang the GPU.  A poll parks the thread for up to 20 us,
// so the limit (2 s) is far beyond any real wait.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity,
                                          uint32_t limit = 100000u) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity))
      return true;
  return false;
}

// global -> shared bulk copy, 16-byte aligned addresses, size multiple of 16
__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gmem_src, uint32_t bytes,
                                         uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
                   "r"(smem_addr(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

// shared -> global bulk copy (joins the thread's current bulk group)
__device__ __forceinline__ void bulk_s2g(void *gmem_dst, const void *smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_addr(smem_src)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// wait until at most N of this thread's bulk groups still READ their source
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// make generic-proxy writes to shared memory visible to the async proxy (TMA)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tiled TMA (tensor maps) ------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y,
                                            uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_addr(smem_dst)),
               "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *map, int x, int y,
                                            int z, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_addr(smem_dst)),
               "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *map, int x, int y,
                                            int z, int w, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(smem_addr(smem_dst)),
               "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_addr(bar))
               : "memory");
}
// four rows of a two-dimensional tensor, named by their row coordinates, into four consecutive
// rows of shared memory (box = one row of the map); x is the first column, a multiple of 16 bytes
__device__ __forceinline__ void tma_gather4_2d(void *smem_dst, const CUtensorMap *map, int x, int r0, int r1,
                                               int r2, int r3, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes "
               "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(smem_addr(smem_dst)),
               "l"(map), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(smem_addr(bar))
               : "memory");
}
// the tile's lines into L2, nothing into shared memory, nothing to wait for
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap *map, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(map), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, const void *smem_src, int x,
                                             int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::
                   "l"(map),
               "r"(smem_addr(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, const void *smem_src, int x,
                                             int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
      "r"(smem_addr(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- host: tensor-map encoding through the driver entry point --------------
// (looked up at run time, so the library links against the CUDA runtime only)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

// rank <= 5; dims/strides innermost first; strides in bytes for dims 1..rank-1
int make_tensor_map(CUtensorMap *map, CUtensorMapDataType dt, int rank, void *base,
                    const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box,
                    CUtensorMapSwizzle swizzle);

} // namespace b200
