// Library-wide pieces of the kernel ABI: version, error reporting, and the
// tensor-map encoder looked up through the runtime's driver entry point.
#include <mutex>

#include "common.cuh"
#include "tma.cuh"

namespace b200 {

static thread_local int g_last_cuda_error = 0;
void set_last_cuda_error(int e) { g_last_cuda_error = e; }

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

int make_tensor_map(CUtensorMap *map, CUtensorMapDataType dt, int rank, void *base,
                    const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box,
                    CUtensorMapSwizzle swizzle) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc)
    return B200_ERR_UNSUPPORTED;
  cuuint64_t d[5], s[5];
  cuuint32_t b[5], e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
    if (i + 1 < rank)
      s[i] = strides_bytes[i];
  }
  CUresult r = enc(map, dt, (cuuint32_t)rank, base, d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_cuda_error((int)r);
    return B200_ERR_CUDA;
  }
  return B200_OK;
}

} // namespace b200

extern "C" const char *b200_version(void) { return "byteir-b200 0.1 (sm_100a)"; }

extern "C" int b200_last_cuda_error(void) { return b200::g_last_cuda_error; }

extern "C" const char *b200_error_string(int code) {
  switch (code) {
  case B200_OK:
    return "ok";
  case B200_ERR_INVALID_ARG:
    return "invalid argument";
  case B200_ERR_UNSUPPORTED:
    return "unsupported shape or type";
  case B200_ERR_WORKSPACE:
    return "workspace missing or too small";
  case B200_ERR_CUDA:
    return "CUDA error (see b200_last_cuda_error)";
  case B200_ERR_ALIGNMENT:
    return "pointer or stride not aligned as required";
  default:
    return "unknown error";
  }
}
