// The communicator a DistributedSession hands to its kernels through
// ExecutionContext::distributed_backend
// (runtime/include/brt/core/distributed/distributed_backend.h:22-124).  One object per rank.
//
// The hot path has one exchange step, the all-reduce of the partial sums of a reduction whose reduced
// axis is sharded over devices, so all_reduce is the collective declared here; the reference's
// interface also carries send / recv / scatter / gather / all_to_all / all_gather / reduce_scatter /
// broadcast / reduce and a socket rendezvous, which no op of the path calls.
#pragma once

#include "brt/core/common/enums.h"
#include "brt/core/common/status.h"
#include "brt/core/distributed/d_context.h"
#include "brt/core/framework/dtype.h"
#include <memory>
#include <set>

namespace brt {

class DistributedBackend {
public:
  DistributedBackend(uint32_t nranks, uint32_t rank) : m_nranks(nranks), m_rank(rank) {}
  virtual ~DistributedBackend() = default;

  uint32_t nranks() { return m_nranks; }
  uint32_t rank() { return m_rank; }

  // recvbuff[i] = op over the ranks of replica_group of sendbuff[i], i < len; the same on every rank of
  // the group.  An empty group means all ranks.  Enqueued on ctx's stream for device buffers.
  virtual common::Status all_reduce(const void *sendbuff, void *recvbuff, size_t len, DTypeEnum dtype, ReduceOp op,
                                    std::set<int64_t> replica_group, std::shared_ptr<DContext> ctx) = 0;

  // The sum of f32 vectors delivered in a narrower element type, rounded once after the sum: what
  // nccl.AllReduce followed by a cast computes.  A backend that can do both in one step overrides this;
  // otherwise the caller all-reduces in f32 and casts.
  virtual common::Status all_reduce_sum_f32_rounded(const float *, void *, size_t, DTypeEnum, std::set<int64_t>,
                                                    std::shared_ptr<DContext>) {
    return common::Status(common::StatusCategory::BRT, common::StatusCode::NOT_IMPLEMENTED,
                          "this backend has no fused all-reduce and cast");
  }

protected:
  uint32_t m_nranks;
  uint32_t m_rank;
};

} // namespace brt
