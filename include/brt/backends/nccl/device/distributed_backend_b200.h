// The two communicators of this runtime, in place of the reference's DistributedBackendNCCL
// (runtime/include/brt/backends/nccl/device/distributed_backend_nccl.h; all_reduce at
// runtime/lib/backends/nccl/device/distributed_backend_nccl.cc:175-194, which splits a communicator off
// and destroys it on every call).
#pragma once

#include "brt/core/distributed/distributed_backend.h"
#include <vector>

namespace brt {

// all_reduce handed to the process that owns the communicator.  The host program creates its process
// group once (torch.distributed over NCCL for device buffers, gloo for host buffers) and passes a
// function that runs one all-reduce on it; nothing is created or destroyed per call.
//   fn(user, send, recv, len, dtype (DTypeEnum value), op (ReduceOp value), group, group_len,
//      stream (CUstream_st *, NULL for host buffers)) -> 0 on success
typedef int (*BrtAllReduceFn)(void *user, const void *send, void *recv, uint64_t len, int dtype, int op,
                              const int64_t *group, uint64_t group_len, void *stream);

class DistributedBackendCallback final : public DistributedBackend {
public:
  DistributedBackendCallback(uint32_t nranks, uint32_t rank, BrtAllReduceFn fn, void *user)
      : DistributedBackend(nranks, rank), fn_(fn), user_(user) {}
  common::Status all_reduce(const void *sendbuff, void *recvbuff, size_t len, DTypeEnum dtype, ReduceOp op,
                            std::set<int64_t> replica_group, std::shared_ptr<DContext> ctx) override;

private:
  BrtAllReduceFn fn_;
  void *user_;
};

// The sum of f32 vectors of up to `capacity` elements over ALL ranks as one kernel over NVLink peer
// memory (b200_sharded_sum_finish): every rank stores its vector into every peer's inbox, publishes an
// epoch flag, waits (bounded) for the peers' flags, and adds the vectors in rank order, so that every
// rank holds the same bits; the result may be delivered rounded to f16 / bf16.
//   peer_inbox[p], peer_flags[p]: rank p's inbox (b200_sharded_sum_inbox_bytes(nranks, capacity) bytes)
//   and flag words (nranks * 4 bytes), zeroed once, mapped into this process (symmetric memory);
//   epoch_counter: a zeroed device uint32 of this rank; status: a device int (3 after a wait ran out).
// Every call uses the inbox with the element count it was sized for, so `len` must equal `capacity`.
class DistributedBackendPeer final : public DistributedBackend {
public:
  DistributedBackendPeer(uint32_t nranks, uint32_t rank, size_t capacity, const std::vector<void *> &peer_inbox,
                         const std::vector<void *> &peer_flags, uint32_t *epoch_counter, int *status)
      : DistributedBackend(nranks, rank), capacity_(capacity), inbox_(peer_inbox), flags_(peer_flags),
        epoch_counter_(epoch_counter), status_(status) {}
  common::Status all_reduce(const void *sendbuff, void *recvbuff, size_t len, DTypeEnum dtype, ReduceOp op,
                            std::set<int64_t> replica_group, std::shared_ptr<DContext> ctx) override;
  common::Status all_reduce_sum_f32_rounded(const float *sendbuff, void *recvbuff, size_t len, DTypeEnum out_dtype,
                                            std::set<int64_t> replica_group, std::shared_ptr<DContext> ctx) override;

private:
  common::Status Launch(const float *send, void *recv, size_t len, DTypeEnum out_dtype,
                        const std::set<int64_t> &group, const std::shared_ptr<DContext> &ctx);
  size_t capacity_;
  std::vector<void *> inbox_, flags_;
  uint32_t *epoch_counter_;
  int *status_;
};

} // namespace brt
