// ExponentiatedAdam dense update (optimizers.py:353-376) fused with the gradient scaling that
// follows the data-parallel sum and with the SignedConstraint (models.py:419-427).
#include <math.h>

#include "v1g_internal.h"

namespace {

__global__ void __launch_bounds__(256) expadam_kernel(float* __restrict__ w,
                                                      const float* __restrict__ grad,
                                                      float* __restrict__ m, float* __restrict__ v,
                                                      const uint8_t* __restrict__ positive,
                                                      int64_t n, float alpha, float one_m_b1,
                                                      float one_m_b2, float eps, float grad_scale) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const float g = grad[i] * grad_scale;
    float mi = m[i], vi = v[i];
    mi = mi + (g - mi) * one_m_b1;
    vi = vi + (g * g - vi) * one_m_b2;
    m[i] = mi;
    v[i] = vi;
    const float adam = mi / (sqrtf(vi) + eps);
    float wi = w[i];
    const float sgn = (wi < 0.f) ? -1.f : 1.f;  // sign(0) counts as +1
    wi = wi * expf((-alpha * adam) * sgn);
    // SignedConstraint: where(positive, relu(w), -relu(-w))
    if (positive) wi = positive[i] ? fmaxf(wi, 0.f) : -fmaxf(-wi, 0.f);
    w[i] = wi;
  }
}

}  // namespace

extern "C" int v1g_expadam_update(float* w, const float* grad, float* m, float* v,
                                  const uint8_t* positive, int64_t n, float lr, float beta1,
                                  float beta2, float eps, int64_t step, float grad_scale,
                                  void* stream) {
  if (!w || !grad || !m || !v || n < 0 || step < 1) return V1G_EINVAL;
  if (n == 0) return V1G_OK;
  // alpha = lr * sqrt(1 - beta2^t) / (1 - beta1^t) in fp32, as the reference computes it
  const float b1p = powf(beta1, (float)step), b2p = powf(beta2, (float)step);
  const float alpha = lr * sqrtf(1.f - b2p) / (1.f - b1p);
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  expadam_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(w, grad, m, v, positive, n, alpha,
                                                           1.f - beta1, 1.f - beta2, eps, grad_scale);
  v1g_count_launches(1);
  return cudaGetLastError() == cudaSuccess ? V1G_OK : V1G_ECUDA;
}
