// TEST INFRASTRUCTURE ONLY: see op_kernel.h in this directory.
#pragma once
#include "tensorflow/core/framework/op_kernel.h"
#include "tensorflow/core/framework/shape_inference.h"

namespace tensorflow {
struct OpDefBuilderStub {
  OpDefBuilderStub& Attr(const char*) { return *this; }
  OpDefBuilderStub& Input(const char*) { return *this; }
  OpDefBuilderStub& Output(const char*) { return *this; }
  OpDefBuilderStub& Doc(const char*) { return *this; }
  template <typename F> OpDefBuilderStub& SetShapeFn(F f) {
    Status (*check)(shape_inference::InferenceContext*) = f;  // the signature TensorFlow expects
    (void)check;
    return *this;
  }
};
}  // namespace tensorflow
#define REGISTER_OP(NAME) \
  static ::tensorflow::OpDefBuilderStub V1G_STUB_CAT(v1g_stub_op_, __COUNTER__) = ::tensorflow::OpDefBuilderStub()
