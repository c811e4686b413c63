// extern "C" wrapper over Session / RequestContext (include/brt_c_api.h).
#include "brt_c_api.h"

#include "brt/backends/cpu/providers/default/cpu_provider.h"
#include "brt/backends/cuda/device/cuda_allocator.h"
#include "brt/backends/cuda/device/cuda_work_queue.h"
#include "brt/backends/cuda/providers/default/cuda_provider.h"
#include "brt/backends/nccl/device/distributed_backend_b200.h"
#include "brt/core/common/common.h"
#include "brt/core/distributed/distributed_session.h"
#include "brt/core/framework/execution_provider.h"
#include "brt/core/session/request_context.h"
#include "brt/core/session/session.h"

#include <cstring>
#include <mutex>

using namespace brt;

struct brt_session {
  brt_session() : owned(new Session()), session(*owned) {}
  brt_session(int rank, int nranks) : owned(new DistributedSession(rank, nranks)), session(*owned) {}
  std::unique_ptr<DistributedBackend> backend; // destroyed after the session
  std::unique_ptr<Session> owned;
  Session &session;
};
struct brt_request {
  std::unique_ptr<RequestContext> ctx;
  std::mutex mu;
  std::string trace;
};

namespace {
thread_local std::string g_error;

int Report(const common::Status &s) {
  if (s.IsOK())
    return 0;
  g_error = s.ToString();
  return s.Code() ? s.Code() : 1;
}

template <typename F> int Guard(F &&f) {
  try {
    return Report(f());
  } catch (const std::exception &e) {
    g_error = e.what();
    return common::RUNTIME_EXCEPTION;
  }
}

void CopyStr(const std::string &s, char *dst, size_t cap) {
  if (!dst || cap == 0)
    return;
  const size_t n = std::min(cap - 1, s.size());
  std::memcpy(dst, s.data(), n);
  dst[n] = '\0';
}
} // namespace

extern "C" {

const char *brt_last_error(void) { return g_error.c_str(); }

int brt_register_kernels_from_dynlib(const char *path) {
  return Guard([&] { return ExecutionProvider::StaticRegisterKernelsFromDynlib(path); });
}

brt_session *brt_session_create(void) {
  try {
    return new brt_session();
  } catch (const std::exception &e) {
    g_error = e.what();
    return nullptr;
  }
}
void brt_session_destroy(brt_session *s) { delete s; }

brt_session *brt_session_create_distributed(int rank, int nranks) {
  try {
    return new brt_session(rank, nranks);
  } catch (const std::exception &e) {
    g_error = e.what();
    return nullptr;
  }
}

namespace {
common::Status AsDistributed(brt_session *s, DistributedSession **out) {
  *out = dynamic_cast<DistributedSession *>(s->owned.get());
  if (!*out)
    return common::Status(common::BRT, common::INVALID_ARGUMENT,
                          "not a distributed session (brt_session_create_distributed)");
  return common::Status::OK();
}
} // namespace

int brt_session_set_allreduce_callback(brt_session *s, brt_allreduce_fn fn, void *user) {
  return Guard([&]() -> common::Status {
    DistributedSession *ds = nullptr;
    BRT_RETURN_IF_ERROR(AsDistributed(s, &ds));
    s->backend.reset(new DistributedBackendCallback((uint32_t)ds->GetNRanks(), (uint32_t)ds->GetRank(),
                                                    reinterpret_cast<BrtAllReduceFn>(fn), user));
    ds->SetDistributedBackend(s->backend.get());
    return common::Status::OK();
  });
}

int brt_session_set_allreduce_peer(brt_session *s, uint64_t capacity, void *const *peer_inbox, void *const *peer_flags,
                                   void *epoch_counter, void *status) {
  return Guard([&]() -> common::Status {
    DistributedSession *ds = nullptr;
    BRT_RETURN_IF_ERROR(AsDistributed(s, &ds));
    if (!peer_inbox || !peer_flags || !epoch_counter || capacity == 0)
      return common::Status(common::BRT, common::INVALID_ARGUMENT, "peer tables, counter and capacity are required");
    std::vector<void *> inbox(peer_inbox, peer_inbox + ds->GetNRanks()), flags(peer_flags, peer_flags + ds->GetNRanks());
    s->backend.reset(new DistributedBackendPeer((uint32_t)ds->GetNRanks(), (uint32_t)ds->GetRank(), (size_t)capacity,
                                                inbox, flags, static_cast<uint32_t *>(epoch_counter),
                                                static_cast<int *>(status)));
    ds->SetDistributedBackend(s->backend.get());
    return common::Status::OK();
  });
}

int brt_session_add_cpu(brt_session *s) {
  return Guard([&] { return NaiveCPUExecutionProviderFactory(&s->session); });
}
int brt_session_add_cuda(brt_session *s, int device_id) {
  return Guard([&]() -> common::Status {
    BRT_RETURN_IF_ERROR(CUDAAllocatorFactory(&s->session, device_id));
    return DefaultCUDAExecutionProviderFactory(&s->session);
  });
}
int brt_session_add_cuda_external(brt_session *s, int device_id, void *alloc_fn, void *free_fn) {
  return Guard([&]() -> common::Status {
    BRT_RETURN_IF_ERROR(CUDAExternalAllocatorFactory(&s->session, device_id, alloc_fn, free_fn));
    return DefaultCUDAExecutionProviderFactory(&s->session);
  });
}
int brt_session_load(brt_session *s, const char *path) {
  return Guard([&] { return s->session.Load(path, "byre"); });
}
int brt_session_load_from_memory(brt_session *s, const char *text) {
  return Guard([&] { return s->session.LoadFromMemory(text, "byre"); });
}

int brt_session_load_buffer(brt_session *s, const void *data, size_t size) {
  return Guard([&] { return s->session.LoadFromBuffer(data, size); });
}

int64_t brt_session_arg_num(brt_session *s) { return (int64_t)s->session.GetArgNum(); }
int brt_session_arg_offset(brt_session *s, const char *name) { return s->session.GetGraphArgOffset(name); }

int brt_session_arg_info(brt_session *s, int64_t offset, int *dtype, int *rank, int64_t *shape, char *space,
                         size_t space_cap, int *argtype, char *name, size_t name_cap) {
  return Guard([&]() -> common::Status {
    if (offset < 0 || (size_t)offset >= s->session.GetArgNum())
      return common::Status(common::BRT, common::INVALID_ARGUMENT, "arg offset out of range");
    const auto sh = s->session.GetStaticShape((size_t)offset);
    if (dtype)
      *dtype = (int)s->session.GetDType((size_t)offset);
    if (rank)
      *rank = (int)sh.size();
    if (shape)
      for (size_t i = 0; i < sh.size() && i < 8; ++i)
        shape[i] = sh[i];
    CopyStr(s->session.GetSpace((size_t)offset), space, space_cap);
    int type = 0;
    std::string nm;
    auto find = [&](const std::vector<size_t> &offs, const std::vector<std::string> &names, int bit) {
      for (size_t i = 0; i < offs.size(); ++i)
        if (offs[i] == (size_t)offset) {
          type |= bit;
          nm = names[i];
        }
    };
    find(s->session.GetInputArgOffsets(), s->session.GetInputNames(), 1);
    find(s->session.GetOutputArgOffsets(), s->session.GetOutputNames(), 2);
    find(s->session.GetWeightArgOffsets(), s->session.GetWeightNames(), 4);
    if (argtype)
      *argtype = type;
    CopyStr(nm, name, name_cap);
    return common::Status::OK();
  });
}

brt_request *brt_request_create(brt_session *s, void *cuda_stream) {
  try {
    auto r = std::make_unique<brt_request>();
    WorkQueue *wq = nullptr;
    if (cuda_stream)
      wq = new CUDAExternalStreamWorkQueue(static_cast<CUstream_st *>(cuda_stream));
    common::Status st = s->session.NewRequestContext(&r->ctx, wq);
    if (!st.IsOK()) {
      if (!r->ctx)
        delete wq;
      Report(st);
      return nullptr;
    }
    return r.release();
  } catch (const std::exception &e) {
    g_error = e.what();
    return nullptr;
  }
}
void brt_request_destroy(brt_request *r) { delete r; }

int brt_request_bind_arg(brt_request *r, int64_t offset, void *ptr) {
  return Guard([&] { return r->ctx->BindArg((size_t)offset, ptr, BrtOwnershipType::OwnedByExternal); });
}
void *brt_request_get_arg(brt_request *r, int64_t offset) {
  try {
    return r->ctx->GetArg((size_t)offset);
  } catch (const std::exception &e) {
    g_error = e.what();
    return nullptr;
  }
}
int brt_request_finish_io_binding(brt_request *r) {
  return Guard([&]() -> common::Status {
    r->ctx->FinishIOBinding();
    return common::Status::OK();
  });
}
int brt_session_run(brt_session *s, brt_request *r) {
  return Guard([&] { return s->session.Run(*r->ctx); });
}
int brt_request_sync(brt_request *r) {
  return Guard([&] { return r->ctx->Sync(); });
}
int brt_request_enable_op_trace(brt_request *r) {
  return Guard([&]() -> common::Status {
    r->ctx->AddEventListener<Events::BeforeOpKernelRun>([r](const Events::BeforeOpKernelRun &e) {
      std::lock_guard<std::mutex> lock(r->mu);
      r->trace += e.info.GetByREOpName() + ";";
    });
    return common::Status::OK();
  });
}
int64_t brt_request_op_trace(brt_request *r, char *buf, size_t cap) {
  std::lock_guard<std::mutex> lock(r->mu);
  CopyStr(r->trace, buf, cap);
  return (int64_t)r->trace.size();
}
}
