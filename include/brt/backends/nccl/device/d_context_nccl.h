// The context of a collective on device buffers: the stream it is enqueued on
// (runtime/include/brt/backends/nccl/device/d_context_nccl.h).
#pragma once

#include "brt/core/distributed/d_context.h"

struct CUstream_st;

namespace brt {

class CudaContext final : public DContext {
public:
  explicit CudaContext(CUstream_st *stream) : m_stream(stream) {}
  std::string type() const override { return "BRT_CTX_CUDA"; }
  CUstream_st *get_stream() const { return m_stream; }

private:
  CUstream_st *m_stream;
};

} // namespace brt
