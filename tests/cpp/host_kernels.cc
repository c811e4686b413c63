// A kernel plug-in for the host ("CPU", "BRT") provider, loaded by the tests with
// ExecutionProvider::StaticRegisterKernelsFromDynlib, the way the reference's test
// binary loads lib/libexternal_kernels.so (runtime/test/unittest_main/test_main.cc:33-35,
// runtime/test/external_kernels/cpu/kernels.cc).
#include "brt/backends/common.h"
#include "brt/core/context/execution_frame.h"
#include "brt/core/framework/kernel_registry.h"
#include "brt/core/framework/op_accessor.h"

using namespace brt;

namespace {

// AddOp_f32f32_f32(a, b, out): out = a + b
class HostAdd final : public OpKernel {
public:
  explicit HostAdd(const OpKernelInfo &info) : OpKernel(info) {
    OpAccessor a(info_);
    BRT_ENFORCE(a.GetNumArgs() == 3, "AddOp takes 3 operands");
    BRT_ENFORCE(a.GetArgShape(0) == a.GetArgShape(2) && a.GetArgShape(1) == a.GetArgShape(2), "shape mismatch");
    n_ = OpAccessor::GetNumElementsOfShape(a.GetArgShape(0));
  }
  common::Status RunImpl(const ExecutionContext &ctx) override {
    OpAccessor a(info_, ctx.exec_frame);
    const float *x = static_cast<const float *>(a.GetArgAsyncValueRef(0));
    const float *y = static_cast<const float *>(a.GetArgAsyncValueRef(1));
    float *z = static_cast<float *>(a.GetArgAsyncValueRef(2));
    for (int64_t i = 0; i < n_; ++i)
      z[i] = x[i] + y[i];
    return common::Status::OK();
  }

private:
  int64_t n_;
};

// ScaleOp_f32_f32(in, out) {factor = 2.0 : f32, shift = 1 : i64, dims = dense<..>}: out = in * factor + shift
class HostScale final : public OpKernel {
public:
  explicit HostScale(const OpKernelInfo &info) : OpKernel(info) {
    OpAccessor a(info_);
    factor_ = a.GetAttrAsFloat("factor");
    shift_ = a.HasAttr("shift") ? a.GetAttrAsInt("shift") : 0;
    n_ = OpAccessor::GetNumElementsOfShape(a.GetArgShape(0));
  }
  common::Status RunImpl(const ExecutionContext &ctx) override {
    OpAccessor a(info_, ctx.exec_frame);
    const float *x = static_cast<const float *>(a.GetArgAsyncValueRef(0));
    float *z = static_cast<float *>(a.GetArgAsyncValueRef(1));
    for (int64_t i = 0; i < n_; ++i)
      z[i] = x[i] * factor_ + (float)shift_;
    return common::Status::OK();
  }

private:
  float factor_;
  int64_t shift_, n_;
};

// AlwaysFailOp: RunImpl returns an error Status (host-side failure injection)
class HostFail final : public OpKernel {
public:
  explicit HostFail(const OpKernelInfo &info) : OpKernel(info) {}
  common::Status RunImpl(const ExecutionContext &) override {
    return common::Status(common::BRT, common::FAIL, "injected failure");
  }
};

// LLVMJITOp stand-in: checks at construction that the attributes of the reference's bytecode
// fixture (LLJIT/Case0) arrived, then does nothing
class HostJitStub final : public OpKernel {
public:
  explicit HostJitStub(const OpKernelInfo &info) : OpKernel(info) {
    OpAccessor a(info_);
    BRT_ENFORCE(a.GetAttrAsString("device") == "cpu", "device");
    BRT_ENFORCE(a.GetAttrAsString("llvm_file_name").rfind("host_kernels", 0) == 0, "llvm_file_name");
    BRT_ENFORCE(a.GetAttrAsString("kernel_name").rfind("Unknown", 0) == 0, "kernel_name");
    const std::vector<int64_t> want = {1, 1, 1, 1, 2, 2};
    BRT_ENFORCE(a.GetAttrAsIntArray("memory_effects") == want, "memory_effects");
    BRT_ENFORCE(a.GetNumArgs() == 6, "operands");
  }
  common::Status RunImpl(const ExecutionContext &) override { return common::Status::OK(); }
};

BRT_STATIC_KERNEL_REGISTRATION(DeviceKind::CPU, ProviderType::BRT, [](KernelRegistry *registry) {
  registry->Register("LLVMJITOp", [](const OpKernelInfo &info) -> std::shared_ptr<OpKernel> {
    return std::make_shared<HostJitStub>(info);
  });
  registry->Register("AddOp_f32f32_f32", [](const OpKernelInfo &info) -> std::shared_ptr<OpKernel> {
    return std::make_shared<HostAdd>(info);
  });
  registry->Register("ScaleOp_f32_f32", [](const OpKernelInfo &info) -> std::shared_ptr<OpKernel> {
    return std::make_shared<HostScale>(info);
  });
  registry->Register("AlwaysFailOp", [](const OpKernelInfo &info) -> std::shared_ptr<OpKernel> {
    return std::make_shared<HostFail>(info);
  });
})

} // namespace
