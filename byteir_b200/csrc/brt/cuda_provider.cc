// The default CUDA provider and its op kernels for the ByRE compute ops
// ReduceSumOp / ReduceMaxOp / IndexSelectOp / IndexPutOp / TransposeOp and the
// byre.custom bridge.  Each kernel parses its op at construction (shapes and
// attributes, as the reference's Impl constructors do) and at run time hands raw
// pointers and the queue's stream to the sm_100a kernels behind b200_kernels.h.
#include "b200_kernels.h"
#include "brt/backends/common.h"
#include "brt/backends/cuda/device/utils/op_kernel_impl_helpers.h"
#include "brt/backends/cuda/providers/default/copy/op_registration.h"
#include "brt/backends/cuda/providers/default/cuda_provider.h"
#include "brt/backends/cuda/providers/default/custom/op_registration.h"
#include "brt/backends/cuda/providers/default/indexing/op_registration.h"
#include "brt/backends/cuda/providers/default/reduction/op_registration.h"
#include "brt/backends/cuda/providers/default/tensor_generate/op_registration.h"
#include "brt/backends/cuda/providers/default/tensor_manipulate/op_registration.h"
#include "brt/core/common/common.h"
#include "brt/core/session/session.h"

#include <algorithm>
#include <cstring>
#include <dlfcn.h>

namespace brt {
namespace cuda {

namespace {

common::Status FromRc(int rc, const char *what) {
  if (rc == B200_OK)
    return common::Status::OK();
  std::string msg = std::string(what) + ": " + b200_error_string(rc);
  if (rc == B200_ERR_CUDA)
    msg += " (cudaError " + std::to_string(b200_last_cuda_error()) + ")";
  return common::Status(common::BRT, common::FAIL, msg);
}

int KernelDType(DTypeEnum dt) {
  switch (dt) {
  case DTypeEnum::Float32: return B200_F32;
  case DTypeEnum::Float16: return B200_F16;
  case DTypeEnum::BFloat16: return B200_BF16;
  default: BRT_THROW("element type ", DTypeName(dt), " is not supported by this op");
  }
}

// =============================================================================
// ReduceSumOp / ReduceMaxOp   (reduction/reduce_impl.h:28-107)
// =============================================================================
std::vector<int64_t> DeduceReduceShape(const std::vector<int64_t> &shape, std::vector<int64_t> dims) {
  std::sort(dims.begin(), dims.end());
  std::vector<int64_t> out;
  for (size_t i = 0; i < shape.size(); ++i)
    if (!std::binary_search(dims.begin(), dims.end(), (int64_t)i))
      out.push_back(shape[i]);
  return out;
}

// Dimensions of size 1 reduce nothing; the rest form groups of consecutive dimensions.  One group is one
// A x B x C reduction, as in the reference, which stops there ("Only consecutive dimensions ..."
// reduce_impl.h:40-42).  Several groups are reduced one after the other, last group first, through f32
// intermediates in the workspace (for a sum of 16-bit values, so that the result is rounded once).
// The target may also be f32 for a 16-bit source (ReduceSumOp_f16_f32): the unrounded sum, which is what a
// device contributes when the reduced axis is sharded over devices and an all-reduce follows.
template <int OP> class ReduceImpl {
public:
  explicit ReduceImpl(const OpAccessor &accessor) {
    auto shape = accessor.GetArgShape(0);
    auto tshape = accessor.GetArgShape(1);
    std::vector<int64_t> dimensions = accessor.GetAttrAsIntArray("dimensions");
    for (auto d : dimensions)
      BRT_ENFORCE(d >= 0 && d < (int64_t)shape.size(), "reduce dimension out of range");
    BRT_ENFORCE(tshape == DeduceReduceShape(shape, dimensions), "output shape does not match input minus dimensions");
    in_dtype_ = KernelDType(accessor.GetArgDTypeEnum(0));
    out_dtype_ = KernelDType(accessor.GetArgDTypeEnum(1));
    BRT_ENFORCE(in_dtype_ == out_dtype_ || (OP == B200_REDUCE_SUM && out_dtype_ == B200_F32),
                "input and output types differ (only a sum may be delivered as f32)");
    // dims of size 1 reduce nothing (reduce_impl.h:81-90)
    dimensions.erase(std::remove_if(dimensions.begin(), dimensions.end(), [&](int64_t d) { return shape[d] == 1; }),
                     dimensions.end());
    std::sort(dimensions.begin(), dimensions.end());
    dimensions.erase(std::unique(dimensions.begin(), dimensions.end()), dimensions.end());
    total_ = OpAccessor::GetNumElementsOfShape(shape);
    // Dimensions of size 1 are taken out of the shape altogether, so that reduced dimensions with only such
    // dimensions between them form one group (f16 [128, 2, 1, 21] over all four is one pass, not two).
    std::vector<int64_t> cur, renumber(shape.size(), -1);
    for (size_t i = 0; i < shape.size(); ++i)
      if (shape[i] != 1) {
        renumber[i] = (int64_t)cur.size();
        cur.push_back(shape[i]);
      }
    for (auto &d : dimensions)
      d = renumber[d];
    // groups of consecutive dimensions, taken from the back so that the indices in front stay valid
    for (size_t hi = dimensions.size(); hi > 0;) {
      size_t lo = hi - 1;
      while (lo > 0 && dimensions[lo] - dimensions[lo - 1] == 1)
        --lo;
      Pass p{1, 1, 1};
      for (int64_t i = 0; i < dimensions[lo]; ++i)
        p.A *= cur[i];
      for (size_t k = lo; k < hi; ++k)
        p.B *= cur[dimensions[k]];
      for (size_t i = dimensions[hi - 1] + 1; i < cur.size(); ++i)
        p.C *= cur[i];
      passes_.push_back(p);
      cur.erase(cur.begin() + dimensions[lo], cur.begin() + dimensions[hi - 1] + 1);
      hi = lo;
    }
    // bytes: [kernel workspace, the largest any pass needs][two intermediates of the first pass's output]
    const int mid = MidDType();
    kernel_ws_ = 0;
    for (size_t i = 0; i < passes_.size(); ++i) {
      const Pass &p = passes_[i];
      if (p.A && p.B && p.C)
        kernel_ws_ = std::max(kernel_ws_, b200_reduce_workspace_bytes(OP, i == 0 ? in_dtype_ : mid, p.A, p.B, p.C));
    }
    kernel_ws_ = (kernel_ws_ + 255) & ~(size_t)255;
    mid_bytes_ = 0;
    const bool cast_at_end = passes_.size() > 1 && mid != out_dtype_;
    if (passes_.size() > 1 || cast_at_end)
      mid_bytes_ = ((size_t)(passes_[0].A * passes_[0].C) * ElemBytes(mid) + 255) & ~(size_t)255;
  }

  common::Status Execute(const void *input, void *output, void *workspace, cudaStream_t stream) {
    if (passes_.empty()) { // nothing to reduce: a copy (reduce_impl.h:70-73)
      return FromRc(b200_reduce(OP, in_dtype_, input, output, 0, 0, total_, nullptr, 0, stream), "b200_reduce");
    }
    char *ws = static_cast<char *>(workspace);
    if (passes_.size() == 1) {
      const Pass &p = passes_[0];
      if (out_dtype_ == in_dtype_)
        return FromRc(b200_reduce(OP, in_dtype_, input, output, p.A, p.B, p.C, ws, kernel_ws_, stream), "b200_reduce");
      return FromRc(b200_reduce_sum_to_f32(in_dtype_, input, static_cast<float *>(output), p.A, p.B, p.C, ws, kernel_ws_,
                                           stream),
                    "b200_reduce_sum_to_f32");
    }
    // several groups: in -> mid[0] -> mid[1] -> ... -> out, the intermediates in f32 for a sum
    const int mid = MidDType();
    void *bufs[2] = {ws + kernel_ws_, ws + kernel_ws_ + mid_bytes_};
    const void *src = input;
    for (size_t i = 0; i < passes_.size(); ++i) {
      const Pass &p = passes_[i];
      const bool last = i + 1 == passes_.size();
      void *dst = (last && mid == out_dtype_) ? output : bufs[i & 1];
      int rc;
      if (i == 0 && mid != in_dtype_)
        rc = b200_reduce_sum_to_f32(in_dtype_, src, static_cast<float *>(dst), p.A, p.B, p.C, ws, kernel_ws_, stream);
      else
        rc = b200_reduce(OP, i == 0 ? in_dtype_ : mid, src, dst, p.A, p.B, p.C, ws, kernel_ws_, stream);
      if (rc)
        return FromRc(rc, "b200_reduce");
      src = dst;
    }
    if (mid != out_dtype_) {
      const Pass &p = passes_.back();
      return FromRc(b200_cast_from_f32(out_dtype_, static_cast<const float *>(src), output, p.A * p.C, stream),
                    "b200_cast_from_f32");
    }
    return common::Status::OK();
  }

  size_t GetWorkspaceSize(const ExecutionContext &) const { return kernel_ws_ + 2 * mid_bytes_; }

private:
  struct Pass {
    int64_t A, B, C;
  };
  static size_t ElemBytes(int dt) { return dt == B200_F32 ? 4 : 2; }
  // element type between the passes of a multi-group reduction
  int MidDType() const { return (OP == B200_REDUCE_SUM && in_dtype_ != B200_F32) ? B200_F32 : in_dtype_; }
  std::vector<Pass> passes_; // in execution order
  int64_t total_;
  int in_dtype_, out_dtype_;
  size_t kernel_ws_, mid_bytes_;
};

template <int OP>
using Reduce = CudaOpKernelWithWorkspace<ReduceImpl<OP>, TypedOperand<const void *, 0>, TypedOperand<void *, 1>>;

// =============================================================================
// IndexSelectOp   (indexing/index_select.h:26-51)
// =============================================================================
class IndexSelectImpl {
public:
  explicit IndexSelectImpl(const OpAccessor &accessor) {
    auto shape = accessor.GetArgShape(0);
    const int64_t ndim = (int64_t)shape.size();
    const int64_t dim = accessor.GetAttrAsInt("dim");
    BRT_ENFORCE(dim >= 0 && dim < ndim, "dim out of range");
    BRT_ENFORCE(accessor.GetArgShape(1).size() == 1, "the index must be one-dimensional");
    A = C = 1;
    for (int64_t i = 0; i < dim; ++i)
      A *= shape[i];
    IB = shape[dim];
    OB = accessor.GetArgShape(1)[0];
    for (int64_t i = dim + 1; i < ndim; ++i)
      C *= shape[i];
    auto out = accessor.GetArgShape(2);
    auto want = shape;
    want[dim] = OB;
    BRT_ENFORCE(out == want, "output shape does not match");
    elt_bytes_ = (int)GetDTypeByte(accessor.GetArgDTypeEnum(0));
    idx_bytes_ = (int)GetDTypeByte(accessor.GetArgDTypeEnum(1));
    BRT_ENFORCE(idx_bytes_ == 4 || idx_bytes_ == 8, "index must be ui32 or i64");
  }
  common::Status Execute(const void *input, const void *index, void *output, cudaStream_t stream) {
    return FromRc(b200_index_select(elt_bytes_, idx_bytes_, input, index, output, A, IB, OB, C, nullptr, stream),
                  "b200_index_select");
  }

private:
  int64_t A, IB, OB, C;
  int elt_bytes_, idx_bytes_;
};
using IndexSelect = CudaOpKernel<IndexSelectImpl, TypedOperand<const void *, 0>, TypedOperand<const void *, 1>,
                                 TypedOperand<void *, 2>>;

// =============================================================================
// IndexPutOp (accumulate)   (indexing/index_put.h:26-66)
// =============================================================================
class IndexPutImpl {
public:
  explicit IndexPutImpl(const OpAccessor &accessor) {
    auto shape = accessor.GetArgShape(0);
    const int64_t ndim = (int64_t)shape.size();
    const int64_t dim = accessor.GetAttrAsInt("dim");
    BRT_ENFORCE(dim >= 0 && dim < ndim, "dim out of range");
    rows_ = 1;
    for (int64_t i = 0; i <= dim; ++i)
      rows_ *= shape[i];
    index_count_ = accessor.GetArgShape(1)[0];
    feature_ = 1;
    for (int64_t i = dim + 1; i < ndim; ++i)
      feature_ *= shape[i];
    BRT_ENFORCE(accessor.GetArgDTypeEnum(1) == DTypeEnum::Int64, "index must be i64");
    BRT_ENFORCE(accessor.GetArgShape(3) == shape, "output shape does not match the input");
    dtype_ = KernelDType(accessor.GetArgDTypeEnum(0));
  }
  common::Status Execute(const void *input, const void *index, const void *update, void *output, void *workspace,
                         cudaStream_t stream) {
    return FromRc(b200_index_put_add(dtype_, input, static_cast<const int64_t *>(index), update, output, rows_,
                                     index_count_, feature_, workspace, Bytes(), nullptr, stream),
                  "b200_index_put_add");
  }
  size_t GetWorkspaceSize(const ExecutionContext &) const { return Bytes(); }

private:
  size_t Bytes() const { return b200_index_put_workspace_bytes(dtype_, rows_, index_count_, feature_); }
  int64_t rows_, index_count_, feature_;
  int dtype_;
};
using IndexPut = CudaOpKernelWithWorkspace<IndexPutImpl, TypedOperand<const void *, 0>, TypedOperand<const void *, 1>,
                                           TypedOperand<const void *, 2>, TypedOperand<void *, 3>>;

// =============================================================================
// TransposeOp   (tensor_manipulate/transpose.{h,cc}): any rank and permutation
// =============================================================================
class TransposeImpl {
public:
  explicit TransposeImpl(const OpAccessor &accessor) {
    shape_ = accessor.GetArgShape(0);
    perm_ = accessor.GetAttrAsIntArray("permutation");
    BRT_ENFORCE(perm_.size() == shape_.size(), "permutation rank does not match the input");
    BRT_ENFORCE(shape_.size() >= 1 && shape_.size() <= 8, "unsupported transpose");
    std::vector<int64_t> want;
    for (auto p : perm_) {
      BRT_ENFORCE(p >= 0 && p < (int64_t)shape_.size(), "bad permutation");
      want.push_back(shape_[p]);
    }
    BRT_ENFORCE(accessor.GetArgShape(1) == want, "output shape does not match the permuted input");
    elt_bytes_ = (int)GetDTypeByte(accessor.GetArgDTypeEnum(0));
  }
  common::Status Execute(const void *input, void *output, cudaStream_t stream) {
    return FromRc(b200_permute(elt_bytes_, input, output, (int)shape_.size(), shape_.data(), perm_.data(), stream),
                  "b200_permute");
  }

private:
  std::vector<int64_t> shape_, perm_;
  int elt_bytes_;
};
using Transpose = CudaOpKernel<TransposeImpl, TypedOperand<const void *, 0>, TypedOperand<void *, 1>>;

// =============================================================================
// byre.custom bridge   (custom/custom.{h,cc})
// =============================================================================
// dlopen(lib_path), dlsym(api_name), call f(void **tensors, void *extra_args, stream).
// Differences from the reference, on purpose: the packed extra_args blob is built
// once at construction instead of malloc'd per run; the VERSION symbol is compared
// as the string it points to and a mismatch only warns; and for the three
// flash-attention entry points, bf16 operands select the sibling symbol
// `<api_name>_bf16` when the library exports it (the custom-call ABI itself
// carries no element type).
class CustomOpKernel final : public OpKernel {
public:
  explicit CustomOpKernel(const OpKernelInfo &info) : OpKernel(info) {
    OpAccessor accessor(info_);
    const std::string lib_path = accessor.GetAttrAsString("lib_path");
    std::string api_name = accessor.GetAttrAsString("api_name");
    const std::string version = accessor.HasAttr("version") ? accessor.GetAttrAsString("version") : "";
    handle_ = dlopen(lib_path.c_str(), RTLD_LAZY | RTLD_GLOBAL);
    BRT_ENFORCE(handle_ != nullptr, "Custom lib ", lib_path, " load failed: ", dlerror());
    const bool flash = api_name == "run_flash_attn_fwd" || api_name == "run_flash_attn_bwd" ||
                       api_name == "run_flash_attn_kvcache";
    if (flash && accessor.GetNumArgs() > 0 && accessor.GetArgDTypeEnum(0) == DTypeEnum::BFloat16) {
      if (dlsym(handle_, (api_name + "_bf16").c_str()))
        api_name += "_bf16";
      else
        BRT_THROW("custom library ", lib_path, " has no bf16 variant of ", api_name);
    }
    run_func_ = reinterpret_cast<RunFn>(dlsym(handle_, api_name.c_str()));
    BRT_ENFORCE(run_func_ != nullptr, "Couldn't find function: ", api_name);
    void *sym = dlsym(handle_, "VERSION");
    BRT_ENFORCE(sym != nullptr, "Version doesn't exist in custom library!");
    const char *lib_version = *static_cast<const char *const *>(sym);
    if (!version.empty() && lib_version && version != lib_version)
      BRT_LOGS_DEFAULT(WARNING) << "custom library " << lib_path << " reports version " << lib_version
                                << ", the module asks for " << version;
    last_error_ = reinterpret_cast<LastErrorFn>(dlsym(handle_, "b200_custom_last_error"));
    if (accessor.HasAttr("extra_args")) {
      size_t n = 0;
      void *blob = accessor.GetAttrAsVoidPtr("extra_args", &n);
      extra_args_.assign(static_cast<char *>(blob), static_cast<char *>(blob) + n);
      free(blob);
    }
    num_args_ = accessor.GetNumArgs();
  }

  ~CustomOpKernel() override {
    if (handle_)
      dlclose(handle_);
  }

  common::Status RunImpl(const ExecutionContext &ctx) override {
    OpAccessor accessor(info_, ctx.exec_frame);
    std::vector<void *> tensors(num_args_);
    for (size_t i = 0; i < num_args_; ++i)
      tensors[i] = accessor.GetArgAsyncValueRef(i);
    cudaStream_t stream = detail::StreamOf(ctx);
    // the callee may read extra_args only during the call, as in the reference
    std::vector<char> args = extra_args_;
    run_func_(tensors.data(), args.data(), stream);
    if (last_error_) {
      if (int rc = last_error_())
        return common::Status(common::BRT, common::FAIL,
                              "custom call " + info_.GetByREOpName() + " failed with code " + std::to_string(rc));
    }
    return BRT_CUDA_CALL(cudaGetLastError());
  }

private:
  using RunFn = void (*)(void **, void *, cudaStream_t);
  using LastErrorFn = int (*)();
  void *handle_ = nullptr;
  RunFn run_func_ = nullptr;
  LastErrorFn last_error_ = nullptr;
  std::vector<char> extra_args_;
  size_t num_args_ = 0;
};

// byre.copy with callee cuda2cuda (copy/copy.cc): a device-to-device copy on the queue's stream
class Cuda2CudaCopy final : public OpKernel {
public:
  explicit Cuda2CudaCopy(const OpKernelInfo &info) : OpKernel(info) {
    OpAccessor accessor(info_);
    bytes_ = (size_t)OpAccessor::GetNumElementsOfShape(accessor.GetArgShape(0)) *
             GetDTypeByte(accessor.GetArgDTypeEnum(0));
  }
  common::Status RunImpl(const ExecutionContext &ctx) override {
    OpAccessor accessor(info_, ctx.exec_frame);
    cudaStream_t stream = detail::StreamOf(ctx);
    return BRT_CUDA_CALL(cudaMemcpyAsync(accessor.GetArgAsyncValueRef(1), accessor.GetArgAsyncValueRef(0), bytes_,
                                         cudaMemcpyDeviceToDevice, stream));
  }

private:
  size_t bytes_;
};

// byre.compute @cpu2cuda / @cuda2cpu (copy/copy.cc:38-72, copy/op_registration.cc): host <-> device
// copies routed through the work queue's copy tasks, as the reference does
class HostDeviceCopy final : public OpKernel {
public:
  HostDeviceCopy(const OpKernelInfo &info, int task_type) : OpKernel(info), task_type_(task_type) {
    OpAccessor accessor(info_);
    bytes_ = (size_t)OpAccessor::GetNumElementsOfShape(accessor.GetArgShape(0)) *
             GetDTypeByte(accessor.GetArgDTypeEnum(0));
  }
  common::Status RunImpl(const ExecutionContext &ctx) override {
    OpAccessor accessor(info_, ctx.exec_frame);
    void *src = accessor.GetArgAsyncValueRef(0), *dst = accessor.GetArgAsyncValueRef(1);
    if (src == dst)
      return common::Status::OK();
    void *args[3] = {&dst, &src, &bytes_};
    return ctx.work_queue->AddTask(task_type_, nullptr, args, info_.GetOpId(), info_.GetDependency());
  }

private:
  int task_type_;
  size_t bytes_;
};

// 16-bit storage formats of a host double, round to nearest even
uint16_t ToF16Bits(double d) {
  const float f = (float)d;
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff)
    return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31)
    return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10)
      return (uint16_t)sign;
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t half = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1)))
      ++half;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((uint32_t)exp << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1)))
    ++half;
  return (uint16_t)(sign | half);
}
uint16_t ToBF16Bits(double d) {
  const float f = (float)d;
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u)
    return (uint16_t)((x >> 16) | 0x40u);
  x += 0x7fffu + ((x >> 16) & 1u);
  return (uint16_t)(x >> 16);
}

// byre.compute @FillOp (tensor_generate/fill.cc:36-95): attribute `value` is a dense constant of the
// tensor's type; a splat fills on the device, anything else is copied from the host
class FillOpKernel final : public OpKernel {
public:
  explicit FillOpKernel(const OpKernelInfo &info) : OpKernel(info) {
    OpAccessor accessor(info_);
    dtype_ = accessor.GetArgDTypeEnum(0);
    count_ = OpAccessor::GetNumElementsOfShape(accessor.GetArgShape(0));
    elt_ = GetDTypeByte(dtype_);
    BRT_ENFORCE(accessor.HasAttr("value"), "FillOp needs a `value` attribute");
    splat_ = accessor.HasAttrOfSplatValue<double>("value");
    const std::vector<double> vals =
        splat_ ? std::vector<double>{accessor.GetAttrAsSplatValue<double>("value")} : accessor.GetAttrAsVector<double>("value");
    BRT_ENFORCE(splat_ || (int64_t)vals.size() == count_, "FillOp: `value` has ", vals.size(), " elements, the tensor ",
                count_);
    host_.resize(vals.size() * elt_);
    for (size_t i = 0; i < vals.size(); ++i)
      Encode(vals[i], host_.data() + i * elt_);
  }
  common::Status RunImpl(const ExecutionContext &ctx) override {
    OpAccessor accessor(info_, ctx.exec_frame);
    cudaStream_t stream = detail::StreamOf(ctx);
    void *out = accessor.GetArgAsyncValueRef(0);
    if (splat_) {
      uint64_t bits = 0;
      std::memcpy(&bits, host_.data(), elt_);
      return FromRc(b200_fill((int)elt_, out, count_, bits, stream), "FillOp");
    }
    return BRT_CUDA_CALL(cudaMemcpyAsync(out, host_.data(), host_.size(), cudaMemcpyHostToDevice, stream));
  }

private:
  void Encode(double v, char *dst) const {
    switch (dtype_) {
    case DTypeEnum::Float32: { const float f = (float)v; std::memcpy(dst, &f, 4); break; }
    case DTypeEnum::Float64: std::memcpy(dst, &v, 8); break;
    case DTypeEnum::Float16: { const uint16_t h = ToF16Bits(v); std::memcpy(dst, &h, 2); break; }
    case DTypeEnum::BFloat16: { const uint16_t h = ToBF16Bits(v); std::memcpy(dst, &h, 2); break; }
    case DTypeEnum::Int64: case DTypeEnum::UInt64: { const int64_t i = (int64_t)v; std::memcpy(dst, &i, 8); break; }
    case DTypeEnum::Int32: case DTypeEnum::UInt32: { const int32_t i = (int32_t)v; std::memcpy(dst, &i, 4); break; }
    case DTypeEnum::Int16: case DTypeEnum::UInt16: { const int16_t i = (int16_t)v; std::memcpy(dst, &i, 2); break; }
    case DTypeEnum::Int8: case DTypeEnum::UInt8: case DTypeEnum::Bool: { const int8_t i = (int8_t)v; std::memcpy(dst, &i, 1); break; }
    default: BRT_THROW("FillOp: element type ", DTypeName(dtype_), " is not supported");
    }
  }
  DTypeEnum dtype_;
  int64_t count_;
  size_t elt_;
  bool splat_;
  std::vector<char> host_; // the value(s) in the tensor's storage format; lives as long as the kernel
};

template <typename K> KernelCreateFn Creator() {
  return [](const OpKernelInfo &info) -> std::shared_ptr<OpKernel> { return std::make_shared<K>(info); };
}

} // namespace

// keys are <Name>_<operand element types>_<result element types>, as the compiler's
// getByreKey builds them (compiler/lib/Dialect/Byre/IR/Common.cpp:35-99)
void RegisterReductionOps(KernelRegistry *registry) {
  for (const char *t : {"f16_f16", "f32_f32", "bf16_bf16"}) { // reference: f16 and f32 sum, f32 and f16 max
    registry->Register(std::string("ReduceSumOp_") + t, Creator<Reduce<B200_REDUCE_SUM>>());
    registry->Register(std::string("ReduceMaxOp_") + t, Creator<Reduce<B200_REDUCE_MAX>>());
  }
  // the unrounded sum of 16-bit values, for a sum that an all-reduce over devices continues
  for (const char *t : {"f16_f32", "bf16_f32"})
    registry->Register(std::string("ReduceSumOp_") + t, Creator<Reduce<B200_REDUCE_SUM>>());
}

void RegisterIndexingOps(KernelRegistry *registry) {
  // reference: IndexSelectOp_{f32ui32_f32, f32i64_f32, f16i64_f16}, IndexPutOp_f32i64f32_f32
  for (const char *t : {"f32", "f16", "bf16"}) {
    for (const char *i : {"ui32", "i64", "i32"})
      registry->Register(std::string("IndexSelectOp_") + t + i + "_" + t, Creator<IndexSelect>());
    registry->Register(std::string("IndexPutOp_") + t + "i64" + t + "_" + t, Creator<IndexPut>());
  }
}

void RegisterTensorManipulateOps(KernelRegistry *registry) {
  for (const char *t : {"f16_f16", "f32_f32", "bf16_bf16", "i32_i32", "i64_i64", "i8_i8", "ui8_ui8", "i16_i16", "f64_f64"})
    registry->Register(std::string("TransposeOp_") + t, Creator<Transpose>());
}

void RegisterCustomOps(KernelRegistry *registry) { registry->Register("custom", Creator<CustomOpKernel>()); }

// the ops on either side of the compute ops in host-driven modules
void RegisterCopyOps(KernelRegistry *registry) { // copy/op_registration.cc
  registry->Register("cpu2cuda", [](const OpKernelInfo &info) -> std::shared_ptr<OpKernel> {
    return std::make_shared<HostDeviceCopy>(info, (int)kH2D);
  });
  registry->Register("cuda2cpu", [](const OpKernelInfo &info) -> std::shared_ptr<OpKernel> {
    return std::make_shared<HostDeviceCopy>(info, (int)kD2H);
  });
  registry->Register("cuda2cuda", Creator<Cuda2CudaCopy>());
}

void RegisterTensorGenerateOps(KernelRegistry *registry) { // tensor_generate/op_registration.cc: FillOp only
  registry->Register("FillOp", Creator<FillOpKernel>());
}

} // namespace cuda

namespace {
// the provider's own kernels are registered like a plug-in's would be
BRT_STATIC_KERNEL_REGISTRATION(DeviceKind::CUDA, ProviderType::BRT, [](KernelRegistry *registry) {
  cuda::RegisterReductionOps(registry);
  cuda::RegisterIndexingOps(registry);
  cuda::RegisterTensorManipulateOps(registry);
  cuda::RegisterCustomOps(registry);
  cuda::RegisterCopyOps(registry);
  cuda::RegisterTensorGenerateOps(registry);
  RegisterCommonBuiltinOps(registry);
})
} // namespace

CUDAExecutionProvider::CUDAExecutionProvider(const std::string &name) : ExecutionProvider(DeviceKind::CUDA, name) {}

common::Status DefaultCUDAExecutionProviderFactory(Session *session) {
  return session->AddExecutionProvider(std::make_unique<CUDAExecutionProvider>(ProviderType::BRT));
}

} // namespace brt
