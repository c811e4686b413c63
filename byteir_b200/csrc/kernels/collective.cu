// The one exchange step of the hot path: a sum whose reduced axis is sharded over
// GPUs (ReduceSumOp over dim 0 with dim 0 split across devices).  Each device
// reduces its shard to unrounded f32 partials (b200_reduce_sum_to_f32); this kernel
// then does what the reference does with nccl.AllReduce followed by a cast
// (runtime/lib/backends/nccl/providers/all_reduce.cc:44-69), in one launch over
// NVLink peer memory:
//   1. every device pushes its partial vector into a slot of every peer's inbox
//      (plain peer stores; an inbox lives in memory the peers have mapped),
//   2. publishes a monotonically increasing epoch in each peer's flag word,
//   3. waits (bounded) until all peers' epochs have arrived in its own flags,
//   4. adds the world's partials from its own inbox in rank order and rounds once.
// All devices add the same numbers in the same order, so they hold identical
// results.  Inbox slots alternate with the epoch's parity; a device can only be one
// epoch ahead of a peer (it needs the peer's flag to finish an epoch), so a slot is
// never overwritten while a peer still reads it.  No multimem, no TMA, no NCCL.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kMaxWorld = 16;
// One block of 256 threads (at most 64 registers each): it fits into the room of ONE block of the
// reductions it runs beside, whose grids fill every SM exactly (see b200_reduce_reserve_blocks).
constexpr int kExchangeThreads = 256;

struct PeerTable {
  float *inbox[kMaxWorld];      // rank p's inbox: float[2][world][n]
  uint32_t *flags[kMaxWorld];   // rank p's flags: uint32[world], flags[q] = last epoch q published
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

template <typename OutT>
__global__ void __launch_bounds__(kExchangeThreads)
    sharded_sum_finish_kernel(const float *__restrict__ partial, PeerTable peers, int rank, int world,
                              int64_t n, uint32_t *epoch_counter, OutT *__restrict__ out, int *status,
                              uint64_t timeout_ns, int vec4) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_timed_out;
  if (threadIdx.x == 0) {
    s_epoch = *epoch_counter + 1;
    s_timed_out = 0;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int slot = (int)(epoch & 1u);
  // 1. push my partials into slot [slot][rank] of every inbox (mine included): the world x n
  //    elements are spread over all threads, so that the stores to all peers are in flight together
  //    (16 bytes each when the vector allows it)
  const size_t slot_off = ((size_t)slot * world + rank) * n;
  if (vec4) {
    const int64_t nv = n >> 2;
    const float4 *src = reinterpret_cast<const float4 *>(partial);
    for (int64_t idx = threadIdx.x; idx < nv * world; idx += blockDim.x) {
      const int p = (int)(idx / nv);
      const int64_t i = idx - (int64_t)p * nv;
      reinterpret_cast<float4 *>(peers.inbox[p] + slot_off)[i] = src[i];
    }
  } else {
    for (int64_t idx = threadIdx.x; idx < n * world; idx += blockDim.x) {
      const int p = (int)(idx / n);
      const int64_t i = idx - (int64_t)p * n;
      (peers.inbox[p] + slot_off)[i] = partial[i];
    }
  }
  __threadfence_system();
  __syncthreads();
  // 2. publish, 3. wait for everyone (one thread per peer)
  if (threadIdx.x < world) {
    st_release_sys(peers.flags[threadIdx.x] + rank, epoch);
    const uint32_t *mine = peers.flags[rank] + threadIdx.x;
    const uint64_t t0 = global_timer_ns();
    // epochs only grow; compare with wrap-around in mind
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if (global_timer_ns() - t0 > timeout_ns) {
        s_timed_out = 1; // a peer never arrived: report and leave, never spin forever
        break;
      }
    }
  }
  __syncthreads();
  if (s_timed_out) {
    // `out` stays as it was and the epoch does not advance: the caller reads *status before it
    // trusts `out`, and must re-establish the protocol (zeroed flags and counters on every rank)
    // before the next call
    if (threadIdx.x == 0 && status)
      *status = 3;
    return;
  }
  // 4. fold the world's partials in rank order; the inbox was written by other GPUs, read it past L1
  const float *inbox = peers.inbox[rank] + (size_t)slot * world * n;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    float acc = __ldcg(inbox + i);
    for (int p = 1; p < world; ++p)
      acc += __ldcg(inbox + (size_t)p * n + i);
    out[i] = Elt<OutT>::from_f32(acc);
  }
  if (threadIdx.x == 0)
    *epoch_counter = epoch;
}


// The same exchange with the sum taken inside the NVSwitch: every device stores its partials into its
// OWN slot of symmetric memory, publishes its epoch to the peers and waits for theirs as above, and
// then reads the slot through the multicast address with multimem.ld_reduce, which returns the sum of
// all devices' copies.  One flag round and one switch round trip instead of world pushes and a fold;
// the order of the additions is the switch's, the same for every device and every call.
//   own_slots: this device's float[2][n] in symmetric memory; mc_slots: the multicast address of the
//   same range (bound to all `world` devices).
template <typename OutT>
__global__ void __launch_bounds__(kExchangeThreads)
    sharded_sum_finish_nvls_kernel(const float *__restrict__ partial, float *own_slots, const float *mc_slots,
                                   PeerTable peers, int rank, int world, int64_t n, uint32_t *epoch_counter,
                                   OutT *__restrict__ out, int *status, uint64_t timeout_ns) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_timed_out;
  if (threadIdx.x == 0) {
    s_epoch = *epoch_counter + 1;
    s_timed_out = 0;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const size_t slot_off = (size_t)(epoch & 1u) * n;
  const int64_t nv = n >> 2; // n % 4 == 0, checked by the caller
  for (int64_t i = threadIdx.x; i < nv; i += blockDim.x)
    reinterpret_cast<float4 *>(own_slots + slot_off)[i] = reinterpret_cast<const float4 *>(partial)[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) {
    st_release_sys(peers.flags[threadIdx.x] + rank, epoch);
    const uint32_t *mine = peers.flags[rank] + threadIdx.x;
    const uint64_t t0 = global_timer_ns();
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if (global_timer_ns() - t0 > timeout_ns) {
        s_timed_out = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (s_timed_out) {
    if (threadIdx.x == 0 && status)
      *status = 3;
    return;
  }
  for (int64_t i = threadIdx.x; i < nv; i += blockDim.x) {
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(mc_slots + slot_off + 4 * i)
                 : "memory");
    out[4 * i + 0] = Elt<OutT>::from_f32(v.x);
    out[4 * i + 1] = Elt<OutT>::from_f32(v.y);
    out[4 * i + 2] = Elt<OutT>::from_f32(v.z);
    out[4 * i + 3] = Elt<OutT>::from_f32(v.w);
  }
  if (threadIdx.x == 0)
    *epoch_counter = epoch;
}

} // namespace
} // namespace b200

using namespace b200;

extern "C" size_t b200_sharded_sum_inbox_bytes(int world, int64_t n) {
  if (world <= 0 || world > kMaxWorld || n <= 0)
    return 0;
  return (size_t)2 * world * n * sizeof(float);
}

extern "C" int b200_sharded_sum_finish(int dtype, const float *partial, void *const *peer_inbox,
                                       void *const *peer_flags, int rank, int world, int64_t n,
                                       uint32_t *epoch_counter, void *out, int *status, cudaStream_t stream) {
  if (world <= 0 || world > kMaxWorld || rank < 0 || rank >= world || n <= 0 || !partial || !peer_inbox ||
      !peer_flags || !epoch_counter || !out)
    return B200_ERR_INVALID_ARG;
  PeerTable t{};
  for (int p = 0; p < world; ++p) {
    if (!peer_inbox[p] || !peer_flags[p])
      return B200_ERR_INVALID_ARG;
    t.inbox[p] = static_cast<float *>(peer_inbox[p]);
    t.flags[p] = static_cast<uint32_t *>(peer_flags[p]);
  }
  const uint64_t timeout_ns = 2000000000ull; // 2 s
  bool vec = n % 4 == 0 && aligned16(partial);
  for (int p = 0; p < world; ++p)
    vec = vec && aligned16(peer_inbox[p]);
  const int vec4 = vec ? 1 : 0;
  switch (dtype) {
  case B200_F32:
    sharded_sum_finish_kernel<float><<<1, kExchangeThreads, 0, stream>>>(partial, t, rank, world, n, epoch_counter,
                                                              (float *)out, status, timeout_ns, vec4);
    break;
  case B200_F16:
    sharded_sum_finish_kernel<__half><<<1, kExchangeThreads, 0, stream>>>(partial, t, rank, world, n, epoch_counter,
                                                               (__half *)out, status, timeout_ns, vec4);
    break;
  case B200_BF16:
    sharded_sum_finish_kernel<__nv_bfloat16><<<1, kExchangeThreads, 0, stream>>>(partial, t, rank, world, n, epoch_counter,
                                                                      (__nv_bfloat16 *)out, status, timeout_ns, vec4);
    break;
  default:
    return B200_ERR_INVALID_ARG;
  }
  return check_launch();
}


extern "C" int b200_sharded_sum_finish_nvls(int dtype, const float *partial, float *own_slots,
                                            const float *multicast_slots, void *const *peer_flags, int rank,
                                            int world, int64_t n, uint32_t *epoch_counter, void *out, int *status,
                                            cudaStream_t stream) {
  if (world <= 0 || world > kMaxWorld || rank < 0 || rank >= world || n <= 0 || n % 4 != 0 || !partial ||
      !own_slots || !multicast_slots || !peer_flags || !epoch_counter || !out || !aligned16(partial) ||
      !aligned16(own_slots) || !aligned16(multicast_slots))
    return B200_ERR_INVALID_ARG;
  PeerTable t{};
  for (int p = 0; p < world; ++p) {
    if (!peer_flags[p])
      return B200_ERR_INVALID_ARG;
    t.flags[p] = static_cast<uint32_t *>(peer_flags[p]);
  }
  const uint64_t timeout_ns = 2000000000ull; // 2 s
  switch (dtype) {
  case B200_F32:
    sharded_sum_finish_nvls_kernel<float><<<1, kExchangeThreads, 0, stream>>>(partial, own_slots, multicast_slots, t, rank, world, n,
                                                                   epoch_counter, (float *)out, status, timeout_ns);
    break;
  case B200_F16:
    sharded_sum_finish_nvls_kernel<__half><<<1, kExchangeThreads, 0, stream>>>(partial, own_slots, multicast_slots, t, rank, world,
                                                                    n, epoch_counter, (__half *)out, status, timeout_ns);
    break;
  case B200_BF16:
    sharded_sum_finish_nvls_kernel<__nv_bfloat16><<<1, kExchangeThreads, 0, stream>>>(
        partial, own_slots, multicast_slots, t, rank, world, n, epoch_counter, (__nv_bfloat16 *)out, status, timeout_ns);
    break;
  default:
    return B200_ERR_INVALID_ARG;
  }
  return check_launch();
}
