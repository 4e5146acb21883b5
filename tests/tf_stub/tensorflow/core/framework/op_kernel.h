// TEST INFRASTRUCTURE ONLY: declarations of the handful of TensorFlow C++ names that
// v1_glif_model_b200/tf_shim/v1g_tf_ops.cc uses, so that the shim can be type-checked against
// include/v1g.h with `g++ -fsyntax-only` on a machine without TensorFlow.  Nothing here has a body
// worth linking; the real headers come from tf.sysconfig when the shim is built.
#pragma once
#include <cstdint>
#include <initializer_list>
#include <string>

namespace Eigen {
struct GpuDevice {
  void* stream() const { return nullptr; }
};
}  // namespace Eigen

namespace tensorflow {
typedef long long int64;  // TensorFlow's own 64-bit integer type
typedef std::int32_t int32;
typedef std::int8_t int8;
typedef std::uint8_t uint8;

class Status {
 public:
  bool ok() const { return true; }
  void IgnoreError() const {}
};
inline Status OkStatus() { return Status(); }
namespace errors {
template <typename... A> Status InvalidArgument(A...) { return Status(); }
template <typename... A> Status ResourceExhausted(A...) { return Status(); }
template <typename... A> Status Internal(A...) { return Status(); }
}  // namespace errors

class TensorShape {
 public:
  TensorShape() {}
  TensorShape(std::initializer_list<int64>) {}
};

template <typename T>
struct FlatView {
  T* data() const { return nullptr; }
  int64 size() const { return 0; }
};

class Tensor {
 public:
  template <typename T> FlatView<T> flat() { return FlatView<T>(); }
  template <typename T> FlatView<const T> flat() const { return FlatView<const T>(); }
  int64 dim_size(int) const { return 0; }
  int dims() const { return 0; }
  int64 NumElements() const { return 0; }
  const TensorShape& shape() const { return shape_; }

 private:
  TensorShape shape_;
};

class OpKernelConstruction {
 public:
  template <typename T> Status GetAttr(const char*, T*) const { return Status(); }
  void CtxFailure(const Status&) {}
  void CtxFailure(const char*, int, const Status&) {}
};

class OpKernelContext {
 public:
  const Tensor& input(int) { return t_; }
  Status allocate_output(int, const TensorShape&, Tensor**) { return Status(); }
  template <typename D> const D& eigen_device() const { static D d; return d; }
  void CtxFailure(const Status&) {}
  void CtxFailure(const char*, int, const Status&) {}

 private:
  Tensor t_;
};

class OpKernel {
 public:
  explicit OpKernel(OpKernelConstruction*) {}
  virtual ~OpKernel() {}
  virtual void Compute(OpKernelContext*) = 0;
};

extern const char* const DEVICE_GPU;

struct KernelDefBuilder {
  KernelDefBuilder& Device(const char*) { return *this; }
  KernelDefBuilder& HostMemory(const char*) { return *this; }
};
inline KernelDefBuilder Name(const char*) { return KernelDefBuilder(); }
}  // namespace tensorflow

#define OP_REQUIRES(CTX, EXP, STATUS) \
  do {                                \
    if (!(EXP)) {                     \
      (CTX)->CtxFailure((STATUS));    \
      return;                         \
    }                                 \
  } while (0)
#define OP_REQUIRES_OK(CTX, ...)                     \
  do {                                               \
    ::tensorflow::Status s_(__VA_ARGS__);            \
    if (!s_.ok()) {                                  \
      (CTX)->CtxFailure(s_);                         \
      return;                                        \
    }                                                \
  } while (0)
#define TF_RETURN_IF_ERROR(...)                      \
  do {                                               \
    ::tensorflow::Status s_(__VA_ARGS__);            \
    if (!s_.ok()) return s_;                         \
  } while (0)
#define V1G_STUB_CAT2(a, b) a##b
#define V1G_STUB_CAT(a, b) V1G_STUB_CAT2(a, b)
#define REGISTER_KERNEL_BUILDER(BUILDER, ...)                                       \
  static ::tensorflow::KernelDefBuilder V1G_STUB_CAT(v1g_stub_kernel_, __COUNTER__) = \
      (::tensorflow::BUILDER);                                                      \
  static_assert(sizeof(__VA_ARGS__) > 0, "kernel class must be complete")
