// OpKernel: one object per op instance of the loaded module
// (runtime/include/brt/core/framework/op_kernel.h:67-178).
#pragma once

#include "brt/core/common/status.h"
#include "brt/core/context/execution_context.h"
#include "brt/core/framework/event.h"
#include "brt/core/framework/op_kernel_info.h"

namespace brt {

class OpKernel {
public:
  explicit OpKernel(const OpKernelInfo &info, bool prologue_per_session = false,
                    bool epilogue_per_session = false, bool prologue_per_frame = false,
                    bool epilogue_per_frame = false)
      : info_(info), has_prologue_per_session_(prologue_per_session),
        has_epilogue_per_session_(epilogue_per_session), has_prologue_per_frame_(prologue_per_frame),
        has_epilogue_per_frame_(epilogue_per_frame) {}
  virtual ~OpKernel() = default;

  virtual common::Status ProloguePerSession() { return NotImplemented(); }
  virtual common::Status EpiloguePerSession() { return NotImplemented(); }
  // called once per frame, before the first Run on that frame
  virtual common::Status ProloguePerFrame(const ExecutionContext &) { return NotImplemented(); }
  virtual common::Status EpiloguePerFrame(const ExecutionContext &) { return NotImplemented(); }

  // Run only enqueues work on the context's WorkQueue; it may complete later.
  common::Status Run(const ExecutionContext &context) {
    context.event_listener_manager->SignalEvent<Events::BeforeOpKernelRun>({info_});
    auto status = RunImpl(context);
    context.event_listener_manager->SignalEvent<Events::AfterOpKernelRun>({info_});
    return status;
  }
  virtual common::Status RunImpl(const ExecutionContext &) { return NotImplemented(); }

  const OpKernelInfo &GetOpKernelInfo() const { return info_; }
  bool HasProloguePerSession() const { return has_prologue_per_session_; }
  bool HasEpiloguePerSession() const { return has_epilogue_per_session_; }
  bool HasProloguePerFrame() const { return has_prologue_per_frame_; }
  bool HasEpiloguePerFrame() const { return has_epilogue_per_frame_; }

protected:
  const OpKernelInfo info_; // a copy, so the kernel never dangles on its creator's info
  bool has_prologue_per_session_;
  bool has_epilogue_per_session_;
  bool has_prologue_per_frame_;
  bool has_epilogue_per_frame_;

private:
  static common::Status NotImplemented() {
    return common::Status(common::StatusCategory::BRT, common::StatusCode::NOT_IMPLEMENTED,
                          "OpKernel no implemented.");
  }
  OpKernel(const OpKernel &) = delete;
  OpKernel &operator=(const OpKernel &) = delete;
};

} // namespace brt
