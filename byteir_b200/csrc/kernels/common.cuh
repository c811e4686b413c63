// Shared device/host helpers of the sm_100a kernel library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b200_kernels.h"

namespace b200 {

// B200: 148 SMs (2 dies x 74).  Launch plans are a pure function of the problem
// shape so that workspace sizes can be computed on a host without a GPU.
constexpr int kNumSMs = 148;

void set_last_cuda_error(int e);

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error((int)e);
    return B200_ERR_CUDA;
  }
  return B200_OK;
}

inline int check_cuda(cudaError_t e) {
  if (e != cudaSuccess) {
    set_last_cuda_error((int)e);
    (void)cudaGetLastError();
    return B200_ERR_CUDA;
  }
  return B200_OK;
}

template <typename T> constexpr int64_t ceil_div(T a, T b) {
  return (a + b - 1) / b;
}

inline int pow2_ceil(int64_t v) {
  int p = 1;
  while (p < v && p < (1 << 30))
    p <<= 1;
  return p;
}

inline bool aligned16(const void *p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// ---- element traits --------------------------------------------------------
template <typename T> struct Elt;
template <> struct Elt<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elt<__half> {
  static __device__ __forceinline__ float to_f32(__half v) {
    return __half2float(v);
  }
  static __device__ __forceinline__ __half from_f32(float v) {
    return __float2half_rn(v);
  }
};
template <> struct Elt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) {
    return __bfloat162float(v);
  }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) {
    return __float2bfloat16_rn(v);
  }
};

// 16-byte streaming load through the read-only path
__device__ __forceinline__ uint4 ld_nc_v4(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void st_cs_v4(void *p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Hint that brings the line holding *p into L2 and returns nothing.  L2 is the point of coherence
// of global memory, so the hint is harmless even for a line that a kernel still running is about
// to write: a kernel launched with programmatic dependent launch may issue it BEFORE pdl_wait(),
// which overlaps the DRAM fetch of its first loads with the tail of its predecessor.
__device__ __forceinline__ void prefetch_l2(const void *p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// Programmatic dependent launch: a kernel launched with the programmatic stream
// serialization attribute may start while its predecessor still runs; it must call
// pdl_wait() before touching the predecessor's output.  The predecessor calls
// pdl_launch_dependents() to let the dependent grid be scheduled early.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                      cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

} // namespace b200
