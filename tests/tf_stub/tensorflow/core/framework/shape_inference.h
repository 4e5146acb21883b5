// TEST INFRASTRUCTURE ONLY: see op_kernel.h in this directory.
#pragma once
#include "tensorflow/core/framework/op_kernel.h"

namespace tensorflow {
namespace shape_inference {
struct ShapeHandle {};
class InferenceContext {
 public:
  void set_output(int, ShapeHandle) {}
  ShapeHandle input(int) { return ShapeHandle(); }
  ShapeHandle UnknownShape() { return ShapeHandle(); }
  ShapeHandle UnknownShapeOfRank(int) { return ShapeHandle(); }
};
}  // namespace shape_inference
}  // namespace tensorflow
