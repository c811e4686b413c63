// What a kernel gets at run time (runtime/include/brt/core/context/execution_context.h:36-50).
#pragma once

namespace brt {
class ExecutionFrame;
class WorkQueue;
class EventListenerManager;
class DistributedBackend;
namespace ExecutionFrame_ { }

struct ExecutionContext {
  ExecutionFrame *exec_frame;
  WorkQueue *work_queue;
  void *frame_state_info; // brt::ExecutionFrame::StateInfo*
  EventListenerManager *event_listener_manager;
  DistributedBackend *distributed_backend = nullptr;

  ExecutionContext(ExecutionFrame *frame, WorkQueue *wq, void *state_info,
                   EventListenerManager *events, DistributedBackend *backend = nullptr)
      : exec_frame(frame), work_queue(wq), frame_state_info(state_info),
        event_listener_manager(events), distributed_backend(backend) {}
};

} // namespace brt
