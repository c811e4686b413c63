// RequestContext: one set of inputs/outputs plus the frame and queue they run on
// (runtime/include/brt/core/session/request_context.h:44-92).  Used by one
// thread at a time.
#pragma once

#include "brt/core/common/status.h"
#include "brt/core/framework/event.h"
#include "brt/core/framework/memory_info.h"
#include "brt/core/session/session.h"
#include <memory>
#include <vector>

namespace brt {

class ExecutionFrame;
class WorkQueue;

class RequestContext {
public:
  // Bind a caller buffer to the arg at `offset`.  OwnedByExternal: borrowed;
  // CopiedByRuntime: not supported for device memory; OwnedByRuntime: the context
  // frees it with the arg's allocator.
  common::Status BindArg(size_t offset, const void *value,
                         BrtOwnershipType owership = BrtOwnershipType::OwnedByExternal);
  // Address of the arg; allocated (and owned) by the context if nothing is bound.
  void *GetArg(size_t offset);
  // Allocate every arg that is still unbound.
  void FinishIOBinding();
  std::vector<int64_t> GetShape(size_t offset);
  common::Status Sync();
  void SetWorkQueue(WorkQueue *wq);
  const Session &GetSession(void) const { return session_; }
  ExecutionFrame *GetExecutionFrame() { return frame_.get(); }
  WorkQueue *GetWorkQueue() { return wq_.get(); }

  template <typename T> void AddEventListener(Events::Listener<T> &&listener) {
    events_->AddEventListener<T>(std::move(listener));
  }
  ~RequestContext();

private:
  friend class Session;
  explicit RequestContext(Session &session);
  Session &session_;
  std::unique_ptr<EventListenerManager> events_;
  std::unique_ptr<ExecutionFrame> frame_;
  std::unique_ptr<WorkQueue> wq_;
};

} // namespace brt
