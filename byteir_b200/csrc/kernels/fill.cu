// FillOp: every element of a tensor gets the same value (reference:
// tensor_generate/kernels/fill.h, called from tensor_generate/fill.cc:36-62).
// The value's bits are replicated into a 16-byte pattern; the aligned body is
// written with 128-bit stores, the unaligned head and tail element by element.
#include "common.cuh"

namespace b200 {
namespace {

template <typename E>
__global__ void __launch_bounds__(256) fill_kernel(E *__restrict__ out, int64_t n, E value, uint4 pattern,
                                                   int64_t head, int64_t nvec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  constexpr int kPer = 16 / (int)sizeof(E);
  uint4 *body = reinterpret_cast<uint4 *>(out + head);
  for (int64_t v = tid; v < nvec; v += stride)
    body[v] = pattern;
  for (int64_t i = tid; i < head; i += stride) // elements before the first 16-byte boundary
    out[i] = value;
  for (int64_t i = head + nvec * kPer + tid; i < n; i += stride) // and after the last full vector
    out[i] = value;
}

template <typename E> int launch_fill(void *out, int64_t n, uint64_t bits, cudaStream_t stream) {
  E value;
  memcpy(&value, &bits, sizeof(E));
  unsigned char pat[16];
  for (size_t i = 0; i < 16; i += sizeof(E))
    memcpy(pat + i, &value, sizeof(E));
  uint4 pattern;
  memcpy(&pattern, pat, 16);
  constexpr int kPer = 16 / (int)sizeof(E);
  const uintptr_t addr = reinterpret_cast<uintptr_t>(out);
  int64_t head = (int64_t)(((16 - (addr & 15)) & 15) / sizeof(E));
  if (head > n)
    head = n;
  const int64_t nvec = (n - head) / kPer;
  const int64_t work = std::max<int64_t>(nvec, 1);
  const unsigned grid = (unsigned)std::min<int64_t>(ceil_div<int64_t>(work, 256), (int64_t)kNumSMs * 8);
  fill_kernel<E><<<grid, 256, 0, stream>>>(static_cast<E *>(out), n, value, pattern, head, nvec);
  return check_launch();
}

} // namespace
} // namespace b200

using namespace b200;

extern "C" int b200_fill(int elt_bytes, void *out, int64_t n, uint64_t value_bits, cudaStream_t stream) {
  if (n < 0 || (n > 0 && !out))
    return B200_ERR_INVALID_ARG;
  if (n == 0)
    return B200_OK;
  if (reinterpret_cast<uintptr_t>(out) % (uintptr_t)(elt_bytes > 0 ? elt_bytes : 1) != 0)
    return B200_ERR_ALIGNMENT;
  switch (elt_bytes) {
  case 1:
    return launch_fill<uint8_t>(out, n, value_bits, stream);
  case 2:
    return launch_fill<uint16_t>(out, n, value_bits, stream);
  case 4:
    return launch_fill<uint32_t>(out, n, value_bits, stream);
  case 8:
    return launch_fill<uint64_t>(out, n, value_bits, stream);
  default:
    return B200_ERR_INVALID_ARG;
  }
}
