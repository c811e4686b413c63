// StaticBRTExecutionPlan, Session and RequestContext
// (runtime/lib/core/framework/execution_plan.cc, runtime/lib/core/session/
// {session,request_context}.cc).
#include "brt/backends/cpu/device/cpu_work_queue.h"
#include "brt/backends/cuda/device/cuda_work_queue.h"
#include "brt/core/common/common.h"
#include "brt/core/framework/execution_plan.h"
#include "brt/core/framework/execution_provider.h"
#include "brt/core/session/request_context.h"
#include "brt/core/session/session.h"

#include <algorithm>

namespace brt {

using common::Status;

namespace {
Status Fail(common::StatusCode code, const std::string &msg) { return Status(common::BRT, code, msg); }

bool IsPlanOnlyOp(const ir::Operation &op) {
  return op.name == "memref.alloc" || op.name == "memref.alloca" || op.name == "func.return";
}
} // namespace

StaticBRTExecutionPlan::StaticBRTExecutionPlan(const ir::ByREHandle &handle, const std::string &ir_path)
    : handle_(handle), ir_path_(ir_path) {}

StaticBRTExecutionPlan::~StaticBRTExecutionPlan() { (void)EpiloguePerSession(); }

Status StaticBRTExecutionPlan::ProloguePerSession(const AllocatorMap &allocators,
                                                  const std::vector<std::unique_ptr<ExecutionProvider>> &providers) {
  const ir::Function &fn = handle_.GetEntryFunc();

  // allocators get a dense index in the frame
  std::unordered_map<std::string, int> alloc_index;
  auto index_of_space = [&](const std::string &space) -> int {
    auto it = alloc_index.find(space);
    if (it != alloc_index.end())
      return it->second;
    auto a = allocators.find(space);
    if (a == allocators.end())
      return -1;
    int idx = (int)frame_info_.allocators.size();
    frame_info_.allocators.push_back(a->second.get());
    frame_info_.intermediate_bytes.push_back(0);
    alloc_index[space] = idx;
    return idx;
  };

  // ---- entry-function arguments (execution_plan.cc:75-157)
  args_.clear();
  frame_info_.args.clear();
  frame_info_.weights.assign(fn.args.size(), nullptr);
  for (size_t i = 0; i < fn.args.size(); ++i) {
    const ir::Value &v = fn.values[fn.args[i]];
    const ir::AttrDict &attrs = fn.arg_attrs[i];
    ArgInfo info;
    auto name_it = attrs.find("byre.argname");
    info.name = name_it != attrs.end() ? name_it->second.s : v.name;
    auto type_it = attrs.find("byre.argtype");
    if (type_it == attrs.end())
      return Fail(common::INVALID_GRAPH, "entry argument " + v.name + " has no byre.argtype");
    info.argtype = (int)type_it->second.i;
    info.type = v.type;
    for (auto d : v.type.shape)
      if (d < 0)
        return Fail(common::NOT_IMPLEMENTED, "dynamic shapes are not supported (argument " + info.name + ")");
    const int ai = index_of_space(v.type.space);
    if (ai < 0)
      return Fail(common::INVALID_GRAPH, "no allocator registered for memory space \"" + v.type.space +
                                             "\" of argument " + info.name);
    ExecutionFrame::ConstructInfo::Arg a;
    a.bytes = v.type.SizeInBytes();
    a.allocator = ai;
    a.is_weight = (info.argtype & ir::kWeight) != 0;
    if (a.is_weight) {
      void *w = frame_info_.allocators[ai]->Alloc(a.bytes ? a.bytes : 1);
      if (!w)
        return Fail(common::FAIL, "allocation of weight " + info.name + " failed");
      owned_weights_.emplace_back(frame_info_.allocators[ai], w);
      frame_info_.weights[i] = w;
    }
    frame_info_.args.push_back(a);
    args_.push_back(info);
  }
  weights_ = frame_info_.weights;

  // ---- tensors: arguments, planned intermediates, aliases (execution_plan.cc:161-241,508-559)
  frame_info_.tensors.resize(fn.values.size());
  uses_cuda_ = false;
  for (const ir::Value &v : fn.values) {
    uses_cuda_ = uses_cuda_ || v.type.space == "cuda";
    auto &loc = frame_info_.tensors[v.id];
    if (v.arg_index >= 0) {
      loc = {ExecutionFrame::ConstructInfo::TensorLoc::kArg, v.arg_index, 0};
      continue;
    }
    const ir::Operation &def = fn.ops[v.defining_op];
    if (def.name == "memref.alloc" || def.name == "memref.alloca") {
      for (auto d : v.type.shape)
        if (d < 0)
          return Fail(common::NOT_IMPLEMENTED, "dynamic shapes are not supported (" + v.name + ")");
      const int ai = index_of_space(v.type.space);
      if (ai < 0)
        return Fail(common::INVALID_GRAPH, "no allocator registered for memory space \"" + v.type.space + "\"");
      size_t &used = frame_info_.intermediate_bytes[ai];
      loc = {ExecutionFrame::ConstructInfo::TensorLoc::kIntermediate, ai, used};
      used += (v.type.SizeInBytes() + kAllocAlignment - 1) / kAllocAlignment * kAllocAlignment;
    } else if (def.name == "byre.alias") {
      if (def.operands.size() != 1)
        return Fail(common::INVALID_GRAPH, "byre.alias takes one operand");
      const ir::Value &src = fn.values[def.operands[0]];
      int64_t offset = 0;
      auto it = def.attrs.find("offset");
      if (it != def.attrs.end())
        offset = it->second.i;
      // the offset counts elements of the SOURCE memref (runtime/lib/core/ir/op_helper.cc:43-52); a view
      // that would start before its source or end behind it is a broken module, not a kernel's problem
      const size_t src_elt = GetDTypeByte(src.type.dtype);
      if (offset < 0 || (size_t)offset * src_elt + v.type.SizeInBytes() > src.type.SizeInBytes())
        return Fail(common::INVALID_GRAPH, "byre.alias " + v.name + " (offset " + std::to_string(offset) + ", " +
                                               std::to_string(v.type.SizeInBytes()) + " bytes) does not fit its source " +
                                               src.name + " (" + std::to_string(src.type.SizeInBytes()) + " bytes)");
      loc = {ExecutionFrame::ConstructInfo::TensorLoc::kAlias, src.id, (size_t)offset * src_elt};
    } else {
      return Fail(common::INVALID_GRAPH, "op " + def.name + " defines a value; only memref.alloc and byre.alias may");
    }
  }

  // ---- a kernel for every ByRE op (execution_plan.cc:314-436)
  kernels_.clear();
  infos_.clear();
  int op_id = 0;
  for (const ir::Operation &op : fn.ops) {
    if (IsPlanOnlyOp(op))
      continue;
    const std::string &key = op.callee;
    if (key.empty())
      return Fail(common::INVALID_GRAPH, "op " + op.name + " at line " + std::to_string(op.line) + " has no callee");
    ExecutionProvider *provider = nullptr;
    for (auto &p : providers) {
      if (p->GetKernelRegistry()->HasKernel(key)) {
        provider = p.get();
        break;
      }
    }
    if (!provider)
      return Fail(common::NOT_IMPLEMENTED, "No providers support Op " + key);
    // the allocator of the memory space of the op's last operand
    IAllocator *last_alloc = nullptr;
    if (!op.operands.empty() || !op.results.empty()) {
      const int last = !op.results.empty() ? op.results.back() : op.operands.back();
      auto a = allocators.find(fn.values[last].type.space);
      if (a != allocators.end())
        last_alloc = a->second.get();
    }
    infos_.push_back(std::make_unique<OpKernelInfo>(*provider, handle_, &op, op_id, allocators, last_alloc,
                                                    weights_, fn.args.size(), ir_path_, std::vector<int>{}));
    std::shared_ptr<OpKernel> kernel;
    try {
      kernel = (*provider->GetKernelRegistry())(key, *infos_.back());
    } catch (const std::exception &e) {
      return Fail(common::INVALID_GRAPH,
                  "building the kernel for " + key + " (line " + std::to_string(op.line) + ") failed: " + e.what());
    }
    if (!kernel)
      return Fail(common::FAIL, "the registry returned no kernel for " + key);
    kernels_.push_back(std::move(kernel));
    ++op_id;
  }
  for (auto &k : kernels_)
    if (k->HasProloguePerSession())
      BRT_RETURN_IF_ERROR(k->ProloguePerSession());
  return Status::OK();
}

Status StaticBRTExecutionPlan::EpiloguePerSession() {
  for (auto &k : kernels_)
    if (k->HasEpiloguePerSession())
      (void)k->EpiloguePerSession();
  kernels_.clear();
  for (auto &w : owned_weights_)
    w.first->Free(w.second);
  owned_weights_.clear();
  return Status::OK();
}

Status StaticBRTExecutionPlan::ProloguePerFrame(const ExecutionContext &ctx) {
  for (auto &k : kernels_)
    if (k->HasProloguePerFrame())
      BRT_RETURN_IF_ERROR(k->ProloguePerFrame(ctx));
  return Status::OK();
}

Status StaticBRTExecutionPlan::EpiloguePerFrame(const ExecutionContext &ctx) {
  Status first = Status::OK();
  for (auto &k : kernels_)
    if (k->HasEpiloguePerFrame()) {
      Status s = k->EpiloguePerFrame(ctx);
      if (first.IsOK() && !s.IsOK())
        first = s;
    }
  return first;
}

Status StaticBRTExecutionPlan::Run(const ExecutionContext &ctx) {
  ctx.event_listener_manager->SignalEvent<Events::BeforeExecutionPlanRun>({});
  BRT_RETURN_IF_ERROR(ctx.exec_frame->AllocIntermediate());
  for (auto &k : kernels_) {
    Status s;
    try {
      s = k->Run(ctx);
    } catch (const std::exception &e) {
      s = Fail(common::RUNTIME_EXCEPTION, std::string("op ") + k->GetOpKernelInfo().GetByREOpName() + ": " + e.what());
    }
    if (!s.IsOK())
      return s;
  }
  ctx.event_listener_manager->SignalEvent<Events::AfterExecutionPlanRun>({});
  return Status::OK();
}

void StaticBRTExecutionPlan::CreateExecutinFrame(std::unique_ptr<ExecutionFrame> *frame) {
  frame->reset(new ExecutionFrame(frame_info_));
}

void StaticBRTExecutionPlan::CreateWorkQueue(std::unique_ptr<WorkQueue> *wq, int rank) {
  // the reference always makes a single-stream CUDA queue in a CUDA build (execution_plan.cc:592-601);
  // here any value in device memory asks for one, whichever memory space the first argument is in
  if (uses_cuda_)
    wq->reset(new CUDASingleStreamWorkQueue(rank));
  else
    wq->reset(new cpu::CPUNaiveWorkQueue());
}

// =============================================================================
// Session
// =============================================================================
Session::Session() = default;
Session::~Session() {
  execution_plan_.reset(); // kernels and weights go before allocators and providers
}

Status Session::AddExecutionProvider(std::unique_ptr<ExecutionProvider> provider) {
  exec_providers_.push_back(std::move(provider));
  return Status::OK();
}

Status Session::AddAllocator(std::unique_ptr<IAllocator> allocator) {
  const std::string key = allocator->Info().key;
  allocators_.emplace(key, std::move(allocator)); // first registration of a memory space wins
  return Status::OK();
}

IAllocator *Session::GetAllocator(const std::string &key) {
  auto it = allocators_.find(key);
  return it == allocators_.end() ? nullptr : it->second.get();
}

Status Session::BuildPlan(const std::string &ir_path) {
  execution_plan_.reset(new StaticBRTExecutionPlan(*ir_handle_, ir_path));
  Status s = execution_plan_->ProloguePerSession(allocators_, exec_providers_);
  if (!s.IsOK()) {
    execution_plan_.reset();
    return s;
  }
  weight_names_.clear(), input_names_.clear(), output_names_.clear();
  weight_offsets_.clear(), input_offsets_.clear(), output_offsets_.clear();
  const auto &args = execution_plan_->GetArgs();
  for (size_t i = 0; i < args.size(); ++i) {
    if (args[i].argtype & ir::kWeight) {
      weight_names_.push_back(args[i].name);
      weight_offsets_.push_back(i);
    }
    if (args[i].argtype & ir::kInput) {
      input_names_.push_back(args[i].name);
      input_offsets_.push_back(i);
    }
    if (args[i].argtype & ir::kOutput) {
      output_names_.push_back(args[i].name);
      output_offsets_.push_back(i);
    }
  }
  return Status::OK();
}

Status Session::Load(const std::string &url, const std::string &fmt) {
  auto handle = std::make_unique<ir::ByREHandle>();
  BRT_RETURN_IF_ERROR(handle->Load(url, fmt));
  execution_plan_.reset();
  ir_handle_ = std::move(handle);
  return BuildPlan(url);
}

Status Session::LoadFromMemory(const void *ptr, const std::string &fmt) {
  auto handle = std::make_unique<ir::ByREHandle>();
  BRT_RETURN_IF_ERROR(handle->LoadFromMemory(ptr, fmt));
  execution_plan_.reset();
  ir_handle_ = std::move(handle);
  return BuildPlan("");
}

Status Session::LoadFromBuffer(const void *data, size_t size) {
  auto handle = std::make_unique<ir::ByREHandle>();
  BRT_RETURN_IF_ERROR(handle->LoadFromBuffer(data, size));
  execution_plan_.reset();
  ir_handle_ = std::move(handle);
  return BuildPlan("");
}

Status Session::LoadWeights(const std::string &, const std::string &) {
  return Status(common::BRT, common::NOT_IMPLEMENTED, "LoadWeights is not implemented"); // as the reference
}

void *Session::GetWeightAsyncValue(size_t offset) {
  BRT_ENFORCE(execution_plan_, "no model loaded");
  return execution_plan_->GetWeight(offset);
}

Status Session::NewRequestContext(std::unique_ptr<RequestContext> *request_ctx, WorkQueue *work_queue) {
  if (!execution_plan_)
    return Status(common::BRT, common::NO_MODEL, "NewRequestContext before a model is loaded");
  std::unique_ptr<RequestContext> ctx(new RequestContext(*this));
  execution_plan_->CreateExecutinFrame(&ctx->frame_);
  if (work_queue) {
    ctx->wq_.reset(work_queue);
  } else {
    try {
      execution_plan_->CreateWorkQueue(&ctx->wq_);
    } catch (const std::exception &e) {
      return Status(common::BRT, common::FAIL, std::string("creating the work queue failed: ") + e.what());
    }
  }
  *request_ctx = std::move(ctx);
  return Status::OK();
}

Status Session::Run(RequestContext &request) {
  if (!execution_plan_)
    return Status(common::BRT, common::NO_MODEL, "Run before a model is loaded");
  ExecutionContext ctx(request.frame_.get(), request.wq_.get(), &request.frame_->GetStateInfo(), request.events_.get(),
                       distributed_backend_);
  try {
    request.frame_->FinishIOBinding();
    if (!request.frame_->IsPrologued()) {
      BRT_RETURN_IF_ERROR(execution_plan_->ProloguePerFrame(ctx));
      request.frame_->SetPrologued();
    }
    return execution_plan_->Run(ctx);
  } catch (const std::exception &e) {
    return Status(common::BRT, common::RUNTIME_EXCEPTION, e.what());
  }
}

void Session::Cleanup(RequestContext &request) noexcept {
  if (!execution_plan_ || !request.frame_ || !request.frame_->IsPrologued())
    return;
  try {
    ExecutionContext ctx(request.frame_.get(), request.wq_.get(), &request.frame_->GetStateInfo(),
                         request.events_.get(), distributed_backend_);
    (void)execution_plan_->EpiloguePerFrame(ctx);
  } catch (...) {
  }
}

int Session::GetGraphArgOffset(const std::string &name) {
  if (!execution_plan_)
    return -1;
  const auto &args = execution_plan_->GetArgs();
  for (size_t i = 0; i < args.size(); ++i)
    if (args[i].name == name)
      return (int)i;
  return -1;
}

size_t Session::GetArgNum() { return execution_plan_ ? execution_plan_->GetArgs().size() : 0; }
size_t Session::GetWeightNum() { return weight_offsets_.size(); }
const std::vector<std::string> &Session::GetWeightNames() { return weight_names_; }
const std::vector<std::string> &Session::GetInputNames() { return input_names_; }
const std::vector<std::string> &Session::GetOutputNames() { return output_names_; }
const std::vector<size_t> &Session::GetWeightArgOffsets() { return weight_offsets_; }
const std::vector<size_t> &Session::GetInputArgOffsets() { return input_offsets_; }
const std::vector<size_t> &Session::GetOutputArgOffsets() { return output_offsets_; }

const std::vector<int64_t> Session::GetStaticShape(size_t id) {
  BRT_ENFORCE(execution_plan_ && id < execution_plan_->GetArgs().size(), "arg offset out of range");
  return execution_plan_->GetArgs()[id].type.shape;
}
DTypeEnum Session::GetDType(size_t id) {
  BRT_ENFORCE(execution_plan_ && id < execution_plan_->GetArgs().size(), "arg offset out of range");
  return execution_plan_->GetArgs()[id].type.dtype;
}
std::string Session::GetSpace(size_t id) {
  BRT_ENFORCE(execution_plan_ && id < execution_plan_->GetArgs().size(), "arg offset out of range");
  return execution_plan_->GetArgs()[id].type.space;
}

// =============================================================================
// RequestContext
// =============================================================================
RequestContext::RequestContext(Session &session) : session_(session), events_(new EventListenerManager()) {}

RequestContext::~RequestContext() {
  try { // a device that went away must not turn the destructor into std::terminate
    if (wq_)
      (void)wq_->Sync();
    session_.Cleanup(*this);
  } catch (const std::exception &) {
  }
}

Status RequestContext::BindArg(size_t offset, const void *value, BrtOwnershipType ownership) {
  return frame_->BindArg(offset, value, ownership);
}
void *RequestContext::GetArg(size_t offset) { return frame_->GetArg(offset); }
void RequestContext::FinishIOBinding() { frame_->FinishIOBinding(); }
std::vector<int64_t> RequestContext::GetShape(size_t offset) { return session_.GetStaticShape(offset); }
Status RequestContext::Sync() { return wq_ ? wq_->Sync() : Status::OK(); }
void RequestContext::SetWorkQueue(WorkQueue *wq) { wq_.reset(wq); }

} // namespace brt
