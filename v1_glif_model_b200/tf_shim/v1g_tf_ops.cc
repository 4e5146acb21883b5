// TensorFlow custom ops over the C ABI of include/v1g.h: the drop-in for the TensorFlow-level
// callables of the reference's recurrent cell (v1_model_utils/models.py).
//
//   V1GSynCurrents      calculate_synaptic_currents forward                 models.py:103-169
//                       calculate_input_current_from_spikes / noise current  models.py:814-940
//   V1GSynCurrentsGrad  its custom gradient (d rec_z_buf, dense dW)          models.py:174-261
//   V1GStep             update_psc + _dense_update_impl + spike + shift      models.py:979-1028, 1099-1117
//   V1GStepGrad         adjoint of the above                                 models.py:58-64, 994, 1010-1018
//   V1GCompactSpikes    tf.where(x > 0)                                      models.py:128, 826, 890
//   V1GRollout          the Keras RNN loop over V1Column.call                models.py:1317-1322
//   V1GRolloutGrad      tape.gradient over it                                multi_training.py:493
//
// Every Compute() takes the GPU stream TensorFlow runs the op on and passes it to the library, so the
// kernels are ordered with the rest of the graph.  Outputs are allocated by TensorFlow; the only entry
// point that needs scratch memory inside a single op call and must not call cudaMalloc behind
// TensorFlow's allocator is the compaction, which therefore uses v1g_compact_spikes_noalloc.
// A library handle (one V1Column on one GPU) is created in Python through ctypes and reaches the ops
// as an int64 attribute holding its address.
//
// Built by build_tf_shim.py, and only where `import tensorflow` succeeds (TensorFlow 2.15 is the
// reference's version, environment.yml:22).
#define EIGEN_USE_GPU
#include "tensorflow/core/framework/op.h"
#include "tensorflow/core/framework/op_kernel.h"
#include "tensorflow/core/framework/shape_inference.h"
#include <cuda_runtime.h>

#include "v1g.h"

namespace tf = tensorflow;
using GPUDevice = Eigen::GpuDevice;

namespace {

V1GHandle* HandleOf(tf::OpKernelConstruction* c) {
  tf::int64 address = 0;
  c->GetAttr("handle", &address).IgnoreError();
  return reinterpret_cast<V1GHandle*>(address);
}

void* StreamOf(tf::OpKernelContext* ctx) { return (void*)ctx->eigen_device<GPUDevice>().stream(); }

// library status -> TensorFlow status with the library's message (the reference raises ValueError
// for bad inputs, models.py:299-315; a failed op raises from session.run / the eager call)
tf::Status Check(V1GHandle* h, int rc) {
  if (rc == V1G_OK) return tf::OkStatus();
  const char* msg = v1g_last_error(h);
  if (rc == V1G_EINVAL) return tf::errors::InvalidArgument(msg);
  if (rc == V1G_ENOMEM) return tf::errors::ResourceExhausted(msg);
  return tf::errors::Internal(msg);
}

class HandleOp : public tf::OpKernel {
 public:
  explicit HandleOp(tf::OpKernelConstruction* c) : tf::OpKernel(c), h_(HandleOf(c)) {
    OP_REQUIRES(c, h_ != nullptr, tf::errors::InvalidArgument("attribute `handle` is not a V1GHandle address"));
  }

 protected:
  V1GHandle* h_;
};

}  // namespace

REGISTER_OP("V1GSynCurrents")
    .Attr("handle: int").Attr("source: int").Attr("n_neurons: int").Attr("n_receptors: int")
    .Input("x: float")            // [B, n_source_cols]: z_buf, LGN spikes or background counts
    .Output("i_flat: float")      // [B * N, R]
    .SetShapeFn([](tf::shape_inference::InferenceContext* c) {
      c->set_output(0, c->UnknownShapeOfRank(2));
      return tf::OkStatus();
    });

class SynCurrentsOp : public HandleOp {
 public:
  explicit SynCurrentsOp(tf::OpKernelConstruction* c) : HandleOp(c) {
    OP_REQUIRES_OK(c, c->GetAttr("source", &source_));
    OP_REQUIRES_OK(c, c->GetAttr("n_neurons", &n_));
    OP_REQUIRES_OK(c, c->GetAttr("n_receptors", &r_));
  }
  void Compute(tf::OpKernelContext* ctx) override {
    const tf::Tensor& x = ctx->input(0);
    const int batch = (int)x.dim_size(0);
    tf::Tensor* out = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, tf::TensorShape({(tf::int64)batch * n_, r_}), &out));
    OP_REQUIRES_OK(ctx, Check(h_, v1g_syn_currents_fwd(h_, source_, x.flat<float>().data(), batch,
                                                       out->flat<float>().data(), StreamOf(ctx))));
  }

 private:
  int source_, n_, r_;
};
REGISTER_KERNEL_BUILDER(Name("V1GSynCurrents").Device(tf::DEVICE_GPU), SynCurrentsOp);

REGISTER_OP("V1GSynCurrentsGrad")
    .Attr("handle: int").Attr("source: int").Attr("nnz: int")
    .Input("x: float").Input("dy: float")   // x as in the forward op, dy [B * N, R]
    .Output("d_x: float")                   // [B, n_source_cols], dense over ALL synapses (models.py:187-202)
    .Output("d_w: float");                  // [nnz], dense, reference synapse order (models.py:226-241)

class SynCurrentsGradOp : public HandleOp {
 public:
  explicit SynCurrentsGradOp(tf::OpKernelConstruction* c) : HandleOp(c) {
    OP_REQUIRES_OK(c, c->GetAttr("source", &source_));
    OP_REQUIRES_OK(c, c->GetAttr("nnz", &nnz_));
  }
  void Compute(tf::OpKernelContext* ctx) override {
    const tf::Tensor& x = ctx->input(0);
    const tf::Tensor& dy = ctx->input(1);
    tf::Tensor *d_x = nullptr, *d_w = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, x.shape(), &d_x));
    OP_REQUIRES_OK(ctx, ctx->allocate_output(1, tf::TensorShape({nnz_}), &d_w));
    OP_REQUIRES_OK(ctx, Check(h_, v1g_syn_currents_bwd(h_, source_, x.flat<float>().data(), dy.flat<float>().data(),
                                                       (int)x.dim_size(0), d_x->flat<float>().data(),
                                                       d_w->flat<float>().data(), StreamOf(ctx))));
  }

 private:
  int source_;
  tf::int64 nnz_;
};
REGISTER_KERNEL_BUILDER(Name("V1GSynCurrentsGrad").Device(tf::DEVICE_GPU), SynCurrentsGradOp);

// state tensors in the reference's order and dtypes (models.py:1030-1056): z_buf, v, r (int8), asc,
// psc_rise, psc
static V1GState StateOf(tf::OpKernelContext* ctx, int first) {
  V1GState s;
  s.z_buf = const_cast<float*>(ctx->input(first + 0).flat<float>().data());
  s.v = const_cast<float*>(ctx->input(first + 1).flat<float>().data());
  s.r = const_cast<int8_t*>(reinterpret_cast<const int8_t*>(ctx->input(first + 2).flat<tf::int8>().data()));
  s.asc = const_cast<float*>(ctx->input(first + 3).flat<float>().data());
  s.psc_rise = const_cast<float*>(ctx->input(first + 4).flat<float>().data());
  s.psc = const_cast<float*>(ctx->input(first + 5).flat<float>().data());
  s.noise_step = nullptr;
  return s;
}

static tf::Status AllocState(tf::OpKernelContext* ctx, int first_in, int first_out, V1GState* s) {
  tf::Tensor* t[6];
  for (int i = 0; i < 6; ++i) TF_RETURN_IF_ERROR(ctx->allocate_output(first_out + i, ctx->input(first_in + i).shape(), &t[i]));
  s->z_buf = t[0]->flat<float>().data();
  s->v = t[1]->flat<float>().data();
  s->r = reinterpret_cast<int8_t*>(t[2]->flat<tf::int8>().data());
  s->asc = t[3]->flat<float>().data();
  s->psc_rise = t[4]->flat<float>().data();
  s->psc = t[5]->flat<float>().data();
  s->noise_step = nullptr;
  return tf::OkStatus();
}

REGISTER_OP("V1GStep")
    .Attr("handle: int")
    .Input("z_buf: float").Input("v: float").Input("r: int8").Input("asc: float")
    .Input("psc_rise: float").Input("psc: float").Input("rec_inputs: float")
    .Output("new_z_buf: float").Output("new_v: float").Output("new_r: int8").Output("new_asc: float")
    .Output("new_psc_rise: float").Output("new_psc: float").Output("z: float");

class StepOp : public HandleOp {
 public:
  using HandleOp::HandleOp;
  void Compute(tf::OpKernelContext* ctx) override {
    V1GState in = StateOf(ctx, 0), out;
    OP_REQUIRES_OK(ctx, AllocState(ctx, 0, 0, &out));
    const tf::Tensor& v = ctx->input(1);
    tf::Tensor* z = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(6, v.shape(), &z));
    OP_REQUIRES_OK(ctx, Check(h_, v1g_step_fwd(h_, (int)v.dim_size(0), &in, ctx->input(6).flat<float>().data(), &out,
                                               z->flat<float>().data(), StreamOf(ctx))));
  }
};
REGISTER_KERNEL_BUILDER(Name("V1GStep").Device(tf::DEVICE_GPU), StepOp);

REGISTER_OP("V1GStepGrad")
    .Attr("handle: int")
    .Input("g_z_buf: float").Input("g_v: float").Input("g_r: int8").Input("g_asc: float")
    .Input("g_psc_rise: float").Input("g_psc: float")            // dL/d(new state); g_r is ignored
    .Input("g_z: float").Input("g_v_out: float")                 // dL/d(outputs z, v)
    .Input("new_v: float").Input("new_r: int8")                  // forward results
    .Output("d_z_buf: float").Output("d_v: float").Output("d_r: int8").Output("d_asc: float")
    .Output("d_psc_rise: float").Output("d_psc: float").Output("d_rec_inputs: float");

class StepGradOp : public HandleOp {
 public:
  using HandleOp::HandleOp;
  void Compute(tf::OpKernelContext* ctx) override {
    V1GState g_out = StateOf(ctx, 0), g_in;
    OP_REQUIRES_OK(ctx, AllocState(ctx, 0, 0, &g_in));
    tf::Tensor* d_rec = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(6, ctx->input(5).shape(), &d_rec));
    OP_REQUIRES_OK(ctx, Check(h_, v1g_step_bwd(h_, (int)ctx->input(1).dim_size(0), &g_out,
                                               ctx->input(6).flat<float>().data(), ctx->input(7).flat<float>().data(),
                                               ctx->input(8).flat<float>().data(),
                                               reinterpret_cast<const int8_t*>(ctx->input(9).flat<tf::int8>().data()),
                                               &g_in, d_rec->flat<float>().data(), StreamOf(ctx))));
  }
};
REGISTER_KERNEL_BUILDER(Name("V1GStepGrad").Device(tf::DEVICE_GPU), StepGradOp);

REGISTER_OP("V1GCompactSpikes")
    .Input("x: float")          // [rows, cols]
    .Output("coords: int64")    // [rows * cols, 2]; the first `count` rows are tf.where(x > 0)
    .Output("count: int32");    // [1]

class CompactSpikesOp : public tf::OpKernel {
 public:
  using tf::OpKernel::OpKernel;
  void Compute(tf::OpKernelContext* ctx) override {
    const tf::Tensor& x = ctx->input(0);
    const tf::int64 rows = x.dim_size(0), cols = x.dim_size(1);
    tf::Tensor *coords = nullptr, *count = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, tf::TensorShape({rows * cols, 2}), &coords));
    OP_REQUIRES_OK(ctx, ctx->allocate_output(1, tf::TensorShape({1}), &count));
    // no handle and no allocation inside the library: all memory of this op comes from TensorFlow
    OP_REQUIRES_OK(ctx, Check(nullptr, v1g_compact_spikes_noalloc(
                                           x.flat<float>().data(), (int32_t)rows, cols,
                                           reinterpret_cast<int64_t*>(coords->flat<tf::int64>().data()), rows * cols,
                                           count->flat<tf::int32>().data(), StreamOf(ctx))));
  }
};
REGISTER_KERNEL_BUILDER(Name("V1GCompactSpikes").Device(tf::DEVICE_GPU), CompactSpikesOp);

REGISTER_OP("V1GRollout")
    .Attr("handle: int").Attr("n_neurons: int").Attr("save_for_bwd: bool = true")
    .Input("x: uint8")             // [B, T, n_lgn] LGN spikes
    .Input("bkg_counts: int32")    // [B, T, n_bkg]; an empty tensor: drawn on the device (models.py:865-887)
    .Output("z: uint8").Output("v: float");   // [B, T, N] each; from the zero state

class RolloutOp : public HandleOp {
 public:
  explicit RolloutOp(tf::OpKernelConstruction* c) : HandleOp(c) {
    OP_REQUIRES_OK(c, c->GetAttr("n_neurons", &n_));
    OP_REQUIRES_OK(c, c->GetAttr("save_for_bwd", &save_));
  }
  void Compute(tf::OpKernelContext* ctx) override {
    const tf::Tensor& x = ctx->input(0);
    const tf::Tensor& counts = ctx->input(1);
    const tf::int64 batch = x.dim_size(0), steps = x.dim_size(1);
    tf::Tensor *z = nullptr, *v = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, tf::TensorShape({batch, steps, n_}), &z));
    OP_REQUIRES_OK(ctx, ctx->allocate_output(1, tf::TensorShape({batch, steps, n_}), &v));
    const int32_t* c = counts.NumElements() ? counts.flat<tf::int32>().data() : nullptr;
    OP_REQUIRES_OK(ctx, Check(h_, v1g_rollout_fwd(h_, (int)batch, (int)steps, x.flat<tf::uint8>().data(), c, nullptr,
                                                  z->flat<tf::uint8>().data(), v->flat<float>().data(), save_ ? 1 : 0,
                                                  StreamOf(ctx))));
  }

 private:
  int n_;
  bool save_;
};
REGISTER_KERNEL_BUILDER(Name("V1GRollout").Device(tf::DEVICE_GPU), RolloutOp);

REGISTER_OP("V1GRolloutGrad")
    .Attr("handle: int").Attr("nnz_rec: int").Attr("nnz_lgn: int").Attr("nnz_bkg: int")
    .Input("g_z: float").Input("g_v: float")   // [B, T, N] gradients of the two outputs
    .Output("d_w_rec: float").Output("d_w_lgn: float").Output("d_w_bkg: float");

class RolloutGradOp : public HandleOp {
 public:
  explicit RolloutGradOp(tf::OpKernelConstruction* c) : HandleOp(c) {
    OP_REQUIRES_OK(c, c->GetAttr("nnz_rec", &nnz_[0]));
    OP_REQUIRES_OK(c, c->GetAttr("nnz_lgn", &nnz_[1]));
    OP_REQUIRES_OK(c, c->GetAttr("nnz_bkg", &nnz_[2]));
  }
  void Compute(tf::OpKernelContext* ctx) override {
    tf::Tensor* d[3];
    for (int i = 0; i < 3; ++i) {
      OP_REQUIRES_OK(ctx, ctx->allocate_output(i, tf::TensorShape({nnz_[i]}), &d[i]));
      // the library accumulates into the gradient buffers
      OP_REQUIRES(ctx, cudaMemsetAsync(d[i]->flat<float>().data(), 0, sizeof(float) * nnz_[i],
                                       (cudaStream_t)StreamOf(ctx)) == cudaSuccess,
                  tf::errors::Internal("cudaMemsetAsync failed"));
    }
    OP_REQUIRES_OK(ctx, Check(h_, v1g_rollout_bwd(h_, nullptr, ctx->input(0).flat<float>().data(),
                                                  ctx->input(1).flat<float>().data(), d[0]->flat<float>().data(),
                                                  d[1]->flat<float>().data(), d[2]->flat<float>().data(), nullptr,
                                                  StreamOf(ctx))));
  }

 private:
  tf::int64 nnz_[3];
};
REGISTER_KERNEL_BUILDER(Name("V1GRolloutGrad").Device(tf::DEVICE_GPU), RolloutGradOp);
