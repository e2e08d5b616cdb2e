// Minimal tensor view and exception helpers of the B200 operator layer.
//
// Plays the role `ms::Tensor`, `GetTensorOrEmpty` and `GetValueFromTensor`
// play in the reference (ops/framework/utils.h:64-107): optional tensors
// become empty views, host-resident int32 vectors are read directly.
#ifndef MS_CUSTOM_OPS_B200_FRAMEWORK_TENSOR_H_
#define MS_CUSTOM_OPS_B200_FRAMEWORK_TENSOR_H_

#include <cstdint>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "ms_custom_ops_c.h"

namespace ms_custom_ops {

// Exceptions carry the kind the reference would have raised; the C ABI maps
// them to (status code, kind, message).
class OpError : public std::runtime_error {
 public:
  OpError(int kind, int code, const std::string &msg) : std::runtime_error(msg), kind_(kind), code_(code) {}
  int kind() const { return kind_; }
  int code() const { return code_; }

 private:
  int kind_;
  int code_;
};

// Stream-style message builder: `throw ValueError() << "text " << v;`
class ErrorBuilder {
 public:
  ErrorBuilder(int kind, int code) : kind_(kind), code_(code) {}
  template <typename T> ErrorBuilder &operator<<(const T &v) {
    os_ << v;
    return *this;
  }
  [[noreturn]] void Throw() const { throw OpError(kind_, code_, os_.str()); }

 private:
  int kind_, code_;
  std::ostringstream os_;
};
struct Raise {
  [[noreturn]] void operator&(const ErrorBuilder &b) const { b.Throw(); }
};
#define MS_VALUE_ERROR ::ms_custom_ops::Raise() & ::ms_custom_ops::ErrorBuilder(MS_ERR_KIND_VALUE, MSCO_ERR_INVALID_ARG)
#define MS_TYPE_ERROR ::ms_custom_ops::Raise() & ::ms_custom_ops::ErrorBuilder(MS_ERR_KIND_TYPE, MSCO_ERR_INVALID_ARG)
#define MS_RUNTIME_ERROR ::ms_custom_ops::Raise() & ::ms_custom_ops::ErrorBuilder(MS_ERR_KIND_RUNTIME, MSCO_ERR_INTERNAL)
#define MS_UNSUPPORTED ::ms_custom_ops::Raise() & ::ms_custom_ops::ErrorBuilder(MS_ERR_KIND_UNSUPPORTED, MSCO_ERR_UNSUPPORTED)

inline const char *DTypeName(int32_t dt) {
  switch (dt) {
    case MSCO_DTYPE_F16: return "Float16";
    case MSCO_DTYPE_BF16: return "BFloat16";
    case MSCO_DTYPE_I8: return "Int8";
    case MSCO_DTYPE_F32: return "Float32";
    case MSCO_DTYPE_I32: return "Int32";
    case MSCO_DTYPE_I64: return "Int64";
    default: return "Unknown";
  }
}

inline int64_t DTypeSize(int32_t dt) {
  switch (dt) {
    case MSCO_DTYPE_F16:
    case MSCO_DTYPE_BF16: return 2;
    case MSCO_DTYPE_I8: return 1;
    case MSCO_DTYPE_F32:
    case MSCO_DTYPE_I32: return 4;
    case MSCO_DTYPE_I64: return 8;
    default: return 0;
  }
}

// Non-owning view; `defined() == false` stands for an absent optional tensor.
class Tensor {
 public:
  Tensor() = default;
  explicit Tensor(const MsTensorDesc *d) : d_(d) {}
  bool defined() const { return d_ != nullptr; }
  void *data() const { return d_ ? d_->data : nullptr; }
  int32_t dtype() const { return d_ ? d_->dtype : -1; }
  bool on_host() const { return d_ && d_->on_host != 0; }
  size_t rank() const { return d_ ? static_cast<size_t>(d_->ndim) : 0; }
  int64_t dim(size_t i) const { return d_->shape[i]; }
  std::vector<int64_t> shape() const {
    return d_ ? std::vector<int64_t>(d_->shape, d_->shape + d_->ndim) : std::vector<int64_t>();
  }
  int64_t numel() const {
    if (!d_) return 0;
    int64_t n = 1;
    for (int i = 0; i < d_->ndim; ++i) n *= d_->shape[i];
    return n;
  }
  bool has_zero_dim() const {
    if (!d_) return false;
    for (int i = 0; i < d_->ndim; ++i)
      if (d_->shape[i] == 0) return true;
    return false;
  }
  // Row-major contiguity (dimensions of extent 1 may carry any stride).
  bool is_contiguous() const {
    if (!d_) return true;
    int64_t expect = 1;
    for (int i = d_->ndim - 1; i >= 0; --i) {
      if (d_->shape[i] != 1 && d_->strides[i] != expect) return false;
      expect *= d_->shape[i];
    }
    return true;
  }
  const MsTensorDesc *desc() const { return d_; }

 private:
  const MsTensorDesc *d_ = nullptr;
};

inline Tensor GetTensorOrEmpty(const MsTensorDesc *opt) { return Tensor(opt); }

// Host-resident int32 vector (context_lens, q_seq_lens, batch_run_status).
inline std::vector<int32_t> GetInt32VectorFromHostTensor(const Tensor &t, const std::string &op_name,
                                                         const std::string &tensor_name) {
  if (t.dtype() != MSCO_DTYPE_I32) {
    MS_RUNTIME_ERROR << "For " << op_name << ", the data_type of " << tensor_name << " must be Int32, but got: "
                     << DTypeName(t.dtype());
  }
  if (!t.on_host()) {
    MS_RUNTIME_ERROR << "For " << op_name << ", " << tensor_name
                     << " must be a CPU tensor (move it to CPU before the call): its values are read on the host.";
  }
  if (t.data() == nullptr && t.numel() != 0) {
    MS_RUNTIME_ERROR << "For " << op_name << ", the data ptr of " << tensor_name << " can not be nullptr.";
  }
  const int32_t *p = static_cast<const int32_t *>(t.data());
  return std::vector<int32_t>(p, p + t.numel());
}

// The reference rejects non-contiguous device tensors at launch
// (internal_kernel_mod.cc:314-331, internal_pyboost_runner.cc:151-163).
inline void CheckContiguous(const Tensor &t, const std::string &op_name, const std::string &tensor_name) {
  if (t.defined() && !t.is_contiguous()) {
    MS_RUNTIME_ERROR << "For " << op_name << ", the tensor " << tensor_name << " must be contiguous.";
  }
}

}  // namespace ms_custom_ops
#endif  // MS_CUSTOM_OPS_B200_FRAMEWORK_TENSOR_H_
