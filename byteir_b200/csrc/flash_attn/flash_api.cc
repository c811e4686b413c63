// libflash_attn.so: the byre.custom entry points of the reference's flash-attention
// library (external_libs/runtime/flash_attn/lib/flash_api.h:75-82), backed by the
// sm_100a kernels.  The custom-call ABI is
//     void f(void **tensors, void *extra_args, cudaStream_t stream)
// where extra_args is the packed attribute blob of the byre.custom op (25 fields for
// fwd and bwd, flash_api.cu:588-624; 31 for the kv-cache entry, flash_api.cu:729-776),
// integers as int64 and floats as float32, unaligned.  The ABI has no return value and carries no element type:
// the reference library assumes fp16; `_bf16` siblings of the entry points do the
// same with bf16 operands.  A failed call leaves a code that
// b200_custom_last_error() returns (and clears).
#include "b200_kernels.h"

#include <cstdint>
#include <cstring>

#ifndef __DRIVER_TYPES_H__
#endif

namespace {

thread_local int g_last_error = 0;

struct Reader {
  const char *p;
  int64_t Int() {
    int64_t v;
    std::memcpy(&v, p, sizeof(v));
    p += sizeof(v);
    return v;
  }
  float Float() {
    float v;
    std::memcpy(&v, p, sizeof(v));
    p += sizeof(v);
    return v;
  }
};

b200_flash_attn_params Unpack(void *extra_args) {
  Reader r{static_cast<const char *>(extra_args)};
  b200_flash_attn_params p;
  p.q_batch_stride = r.Int();
  p.k_batch_stride = r.Int();
  p.v_batch_stride = r.Int();
  p.o_batch_stride = r.Int();
  p.q_row_stride = r.Int();
  p.k_row_stride = r.Int();
  p.v_row_stride = r.Int();
  p.o_row_stride = r.Int();
  p.q_head_stride = r.Int();
  p.k_head_stride = r.Int();
  p.v_head_stride = r.Int();
  p.o_head_stride = r.Int();
  p.b = r.Int();
  p.h = r.Int();
  p.h_k = r.Int();
  p.d = r.Int();
  p.d_rounded = r.Int();
  p.softmax_scale = r.Float();
  p.seqlen_q = r.Int();
  p.seqlen_k = r.Int();
  p.seqlen_q_rounded = r.Int();
  p.seqlen_k_rounded = r.Int();
  p.p_dropout = r.Float();
  // the reference narrows these through uint32 (flash_api.cu:621-624); -1 means unbounded
  p.window_size_left = (int32_t)(uint32_t)r.Int();
  p.window_size_right = (int32_t)(uint32_t)r.Int();
  return p;
}

void Fwd(int dtype, void **tensors, void *extra_args, cudaStream_t stream) {
  // tensors: q, k, v, rng_state, out, softmax_lse, softmax_ptr  (flash_api.cu:626)
  const b200_flash_attn_params p = Unpack(extra_args);
  const int rc = b200_flash_attn_fwd(dtype, tensors[0], tensors[1], tensors[2], tensors[4],
                                     static_cast<float *>(tensors[5]), &p, stream);
  if (rc)
    g_last_error = rc;
}

void Bwd(int dtype, void **tensors, void *extra_args, cudaStream_t stream) {
  // tensors: dout, q, k, v, out, softmax_lse, rng_state, dq, dk, dv, d_softmax_sum, dq_accum
  // (flash_api.cu:696)
  const b200_flash_attn_params p = Unpack(extra_args);
  const int rc = b200_flash_attn_bwd(dtype, tensors[0], tensors[1], tensors[2], tensors[3], tensors[4],
                                     static_cast<const float *>(tensors[5]), tensors[7], tensors[8], tensors[9],
                                     static_cast<float *>(tensors[10]), static_cast<float *>(tensors[11]), &p,
                                     stream);
  if (rc)
    g_last_error = rc;
}

void KvCache(int dtype, void **tensors, void *extra_args, cudaStream_t stream) {
  // tensors: q, kcache, vcache, knew, vnew, seqlens_k, out, softmax_lse; 31 packed fields
  // (flash_api.cu:727-811)
  Reader r{static_cast<const char *>(extra_args)};
  b200_flash_kvcache_params p;
  p.q_batch_stride = r.Int();
  p.k_batch_stride = r.Int();
  p.v_batch_stride = r.Int();
  p.knew_batch_stride = r.Int();
  p.vnew_batch_stride = r.Int();
  p.o_batch_stride = r.Int();
  p.q_row_stride = r.Int();
  p.k_row_stride = r.Int();
  p.v_row_stride = r.Int();
  p.knew_row_stride = r.Int();
  p.vnew_row_stride = r.Int();
  p.o_row_stride = r.Int();
  p.q_head_stride = r.Int();
  p.k_head_stride = r.Int();
  p.v_head_stride = r.Int();
  p.knew_head_stride = r.Int();
  p.vnew_head_stride = r.Int();
  p.o_head_stride = r.Int();
  p.b = r.Int();
  p.h = r.Int();
  p.h_k = r.Int();
  p.d = r.Int();
  p.d_rounded = r.Int();
  p.seqlen_knew = r.Int();
  p.softmax_scale = r.Float();
  p.seqlen_q = r.Int();
  p.seqlen_k = r.Int();
  p.seqlen_q_rounded = r.Int();
  p.seqlen_k_rounded = r.Int();
  p.window_size_left = (int32_t)(uint32_t)r.Int();
  p.window_size_right = (int32_t)(uint32_t)r.Int();
  const int rc = b200_flash_attn_kvcache(dtype, tensors[0], tensors[1], tensors[2], tensors[3], tensors[4],
                                         static_cast<const int32_t *>(tensors[5]), tensors[6],
                                         static_cast<float *>(tensors[7]), &p, nullptr, 0, stream);
  if (rc)
    g_last_error = rc;
}

} // namespace

extern "C" {

// the reference's library exports a `const char *VERSION` variable (flash_api.cu:7-9)
const char *VERSION = "2.5.3";

void run_flash_attn_fwd(void **tensors, void *extra_args, cudaStream_t stream) {
  Fwd(B200_F16, tensors, extra_args, stream);
}
void run_flash_attn_bwd(void **tensors, void *extra_args, cudaStream_t stream) {
  Bwd(B200_F16, tensors, extra_args, stream);
}
void run_flash_attn_fwd_bf16(void **tensors, void *extra_args, cudaStream_t stream) {
  Fwd(B200_BF16, tensors, extra_args, stream);
}
void run_flash_attn_bwd_bf16(void **tensors, void *extra_args, cudaStream_t stream) {
  Bwd(B200_BF16, tensors, extra_args, stream);
}
void run_flash_attn_kvcache(void **tensors, void *extra_args, cudaStream_t stream) {
  KvCache(B200_F16, tensors, extra_args, stream);
}
void run_flash_attn_kvcache_bf16(void **tensors, void *extra_args, cudaStream_t stream) {
  KvCache(B200_BF16, tensors, extra_args, stream);
}

int b200_custom_last_error(void) {
  const int e = g_last_error;
  g_last_error = 0;
  return e;
}
}
