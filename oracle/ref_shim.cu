// extern "C" doors onto the reference's own CUDA kernel launchers, which are
// compiled from where they lie in the reference checkout (see Makefile, target
// _ref).  TEST INFRASTRUCTURE ONLY: used on a GPU box as a second opinion for
// the CPU oracle and as the "reference kernel on the same GPU" comparator.
// Nothing of the product links this.
//
// Launchers bound (declared in the reference's headers):
//   kernel::call_reduce / get_reduce_workspace_in_bytes
//       runtime/lib/backends/cuda/providers/default/reduction/kernels/reduction.h
//   kernel::index_select   .../indexing/kernels/index_select.h
//   kernel::index_put      .../indexing/kernels/index_put.h
//   kernel::transpose_naive_2d  .../tensor_manipulate/kernels/transpose.h
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "reduction/kernels/reduction.h"
#include "reduction/kernels/reduction_helper.h"
#include "indexing/kernels/index_select.h"
#include "indexing/kernels/index_put.h"
#include "tensor_manipulate/kernels/transpose.h"

#include "brt/backends/cuda/device/common/cuda_call.h"

#include <cstdio>
#include <stdexcept>

// The reference kernels check launches with BRT_CUDA_CHECK, whose implementation
// (runtime/lib/backends/cuda/device/common/cuda_call.cc) drags in cuBLAS, cuDNN,
// CUTLASS and NCCL headers.  The one instantiation the four kernel files use is
// supplied here with the same contract: throw on a CUDA error.
namespace brt {
namespace cuda {
template <>
void CudaCall<cudaError, true>(cudaError retCode, const char *exprString, const char *libName,
                               cudaError successCode, const char *msg) {
  if (retCode != successCode) {
    char buf[512];
    std::snprintf(buf, sizeof(buf), "%s failure %d: %s ; expr=%s ; %s", libName, (int)retCode,
                  cudaGetErrorString(retCode), exprString, msg);
    throw std::runtime_error(buf);
  }
}
} // namespace cuda
} // namespace brt

using namespace brt::cuda::kernel;

extern "C" {

// op: 0 sum, 1 max.  dtype: 0 f32, 1 f16.  The reference sizes the f16
// workspace with sizeof(__half) although it stores f32 partials
// (reduce_impl.h:77-79); callers of this shim should pass a workspace of
// ref_reduce_workspace_bytes() computed with dtype 0 to stay in bounds.
size_t ref_reduce_workspace_bytes(int dtype, size_t A, size_t B, size_t C) {
  return dtype == 0 ? get_reduce_workspace_in_bytes<float>(A, B, C)
                    : get_reduce_workspace_in_bytes<__half>(A, B, C);
}

int ref_reduce(int op, int dtype, const void *in, void *out, size_t A, size_t B,
               size_t C, void *workspace, cudaStream_t stream) {
  if (op == 0 && dtype == 0)
    call_reduce<float, reduction::SumOp<float, float, float>>(
        (const float *)in, (float *)out, A, B, C, workspace, stream);
  else if (op == 0 && dtype == 1)
    call_reduce<__half, reduction::SumOp<__half, __half, float>>(
        (const __half *)in, (__half *)out, A, B, C, workspace, stream);
  else if (op == 1 && dtype == 0)
    call_reduce<float, reduction::MaxOp<float, float, float>>(
        (const float *)in, (float *)out, A, B, C, workspace, stream);
  else if (op == 1 && dtype == 1)
    call_reduce<__half, reduction::MaxOp<__half, __half, float>>(
        (const __half *)in, (__half *)out, A, B, C, workspace, stream);
  else
    return -1;
  return (int)cudaGetLastError();
}

// variant: 0 = f32 table / ui32 index, 1 = f32 / i64, 2 = f16 / i64
int ref_index_select(int variant, const void *in, const void *idx, void *out,
                     int A, int IB, int OB, int C, cudaStream_t stream) {
  if (variant == 0)
    index_select<float, uint32_t>((const float *)in, (const uint32_t *)idx,
                                  (float *)out, A, IB, OB, C, stream);
  else if (variant == 1)
    index_select<float, int64_t>((const float *)in, (const int64_t *)idx,
                                 (float *)out, A, IB, OB, C, stream);
  else if (variant == 2)
    index_select<__half, int64_t>((const __half *)in, (const int64_t *)idx,
                                  (__half *)out, A, IB, OB, C, stream);
  else
    return -1;
  return (int)cudaGetLastError();
}

int ref_index_put_f32(const float *in, const int64_t *idx, const float *upd,
                      float *out, int index_count, int feature, int size,
                      cudaStream_t stream) {
  index_put<float, true>(in, idx, upd, out, index_count, feature, size, stream);
  return (int)cudaGetLastError();
}

// dtype: 0 f32, 1 f16.  Grid/block as the reference's Transpose2D::Execute
// derives them (tensor_manipulate/transpose.cc:55-61 with
// MakeCUDAGridAndBlock(n, m): 32x32 blocks).
int ref_transpose2d(int dtype, const void *in, void *out, int m, int n,
                    cudaStream_t stream) {
  dim3 block(32, 32);
  dim3 grid((n + 31) / 32, (m + 31) / 32);
  if (dtype == 0)
    transpose_naive_2d<float>((const float *)in, (float *)out, m, n, grid,
                              block, stream);
  else if (dtype == 1)
    transpose_naive_2d<__half>((const __half *)in, (__half *)out, m, n, grid,
                               block, stream);
  else
    return -1;
  return (int)cudaGetLastError();
}
}
