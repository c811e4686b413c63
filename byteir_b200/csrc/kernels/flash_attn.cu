// placeholder until the tcgen05 kernels land
#include "common.cuh"
extern "C" int b200_flash_attn_fwd(int, const void *, const void *, const void *, void *, float *,
                                   const b200_flash_attn_params *, cudaStream_t) {
  return B200_ERR_UNSUPPORTED;
}
extern "C" int b200_flash_attn_bwd(int, const void *, const void *, const void *, const void *,
                                   const void *, const float *, void *, void *, void *, float *,
                                   float *, const b200_flash_attn_params *, cudaStream_t) {
  return B200_ERR_UNSUPPORTED;
}
