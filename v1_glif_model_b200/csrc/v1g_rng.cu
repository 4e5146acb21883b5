// Device-side samplers for the two stochastic inputs of the cell, so that a rollout needs no input
// from the host beyond seeds:
//   * background spike counts ~ Poisson(bkg_firing_rate * 0.001) per node, trial and step, keyed by
//     (noise_seed + replica * 1000003, step) exactly as calculate_noise_current keys its
//     tf.random.stateless_poisson call (models.py:865-887; noise_seed is advanced once per rollout by
//     tf_utils.py:235-237, which is what makes a recomputed rollout see the same noise);
//   * LGN spikes u < 1 - exp(-rate / 1000) per unit, trial and step from a table of firing rates
//     (stim_dataset.py:182-193).
// The generator is Philox-4x32-10 used as a pure function of (key, counter): any (trial, step,
// unit) can be evaluated anywhere and any number of times with the same result, so chunked rollouts,
// the two passes of the ordered compaction and a replayed backward pass all see the same draws.
// TensorFlow's own streams are not reproduced (its counter layout and Poisson algorithm belong to
// TensorFlow 2.15 and are not part of the reference's sources); what is kept is the keying.
#include <math.h>

#include "v1g_rng.cuh"

namespace {

struct PoissonTable {
  float cdf[V1G_POISSON_TABLE];
};

__global__ void __launch_bounds__(256) sample_bkg_kernel(int B, int T, int n_bkg, unsigned key0,
                                                         const int32_t* __restrict__ step0_dev, int step0,
                                                         PoissonTable tab, int32_t* __restrict__ out) {
  const int64_t n = (int64_t)B * T * n_bkg;
  const int base_step = step0 + (step0_dev ? step0_dev[0] : 0);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int j = (int)(i % n_bkg);
    const int64_t bt = i / n_bkg;
    const int t = (int)(bt % T), b = (int)(bt / T);
    // key = (seed + replica * 1000003, step); counter = (node / 4, trial, 0, stream tag)
    const uint4 r = v1g_philox4x32(make_uint4((unsigned)(j >> 2), (unsigned)b, 0u, V1G_RNG_STREAM_BKG),
                                   make_uint2(key0, (unsigned)(base_step + t)));
    const unsigned w = (j & 3) == 0 ? r.x : (j & 3) == 1 ? r.y : (j & 3) == 2 ? r.z : r.w;
    const float u = v1g_u01(w);
    int k = 0;
#pragma unroll
    for (int q = 0; q < V1G_POISSON_TABLE; ++q) k += (u >= tab.cdf[q]) ? 1 : 0;
    out[i] = k;
  }
}

__global__ void __launch_bounds__(256) sample_lgn_kernel(int B, int T, int n_lgn, const float* __restrict__ rates,
                                                         int64_t batch_stride, unsigned key0, unsigned key1,
                                                         uint8_t* __restrict__ out) {
  const int64_t n = (int64_t)B * T * n_lgn;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % n_lgn);
    const int64_t bt = i / n_lgn;
    const int t = (int)(bt % T), b = (int)(bt / T);
    const float rate = rates[(int64_t)b * batch_stride + (int64_t)t * n_lgn + c];
    out[i] = v1g_lgn_spike(rate, b, t, c, key0, key1) ? 1 : 0;
  }
}

__global__ void advance_noise_step_kernel(int32_t* noise_step, int B, int T) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) noise_step[b] += T;
}

int poisson_table(V1GHandle* h, float lam, PoissonTable* tab) {
  if (!(lam >= 0.f) || lam > 8.f)
    return v1g_fail(h, V1G_ERANGE, "Poisson rate per step %g outside 0..8 (bkg_firing_rate * dt / 1000)", (double)lam);
  double p = exp(-(double)lam), c = 0.0;
  for (int k = 0; k < V1G_POISSON_TABLE; ++k) {
    c += p;
    tab->cdf[k] = (float)fmin(c, 1.0);
    p *= (double)lam / (double)(k + 1);
  }
  tab->cdf[V1G_POISSON_TABLE - 1] = 2.f;  // the count never exceeds the table
  return V1G_OK;
}

}  // namespace

int v1g_sample_bkg_internal(V1GHandle* h, int B, int T, const int32_t* step0_dev, int step0, int32_t* out,
                            cudaStream_t st) {
  PoissonTable tab;
  const float lam = h->cfg.bkg_firing_rate * 0.001f * h->cfg.dt;
  int rc = poisson_table(h, lam, &tab);
  if (rc) return rc;
  const int64_t n = (int64_t)B * T * h->cfg.n_bkg;
  if (n == 0) return V1G_OK;
  const unsigned key0 = (unsigned)(h->noise_seed + (int64_t)h->noise_replica * 1000003LL);
  const int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)h->n_sms * 8);
  sample_bkg_kernel<<<blocks, 256, 0, st>>>(B, T, h->cfg.n_bkg, key0, step0_dev, step0, tab, out);
  v1g_count_launches(1);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

int v1g_advance_noise_step(V1GHandle* h, int32_t* noise_step, int B, int T, cudaStream_t st) {
  if (!noise_step) return V1G_OK;
  advance_noise_step_kernel<<<1, 32, 0, st>>>(noise_step, B, T);
  v1g_count_launches(1);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

extern "C" int v1g_set_noise_seed(V1GHandle* h, int64_t noise_seed, int32_t replica_id) {
  if (!h) return V1G_EINVAL;
  h->noise_seed = noise_seed;
  h->noise_replica = replica_id;
  return V1G_OK;
}

extern "C" int v1g_sample_bkg_counts(V1GHandle* h, int32_t batch, int32_t n_steps, int32_t first_step,
                                     int32_t* counts_out, void* stream) {
  if (!h) return V1G_EINVAL;
  if (batch <= 0 || n_steps < 0 || !counts_out)
    return v1g_fail(h, V1G_EINVAL, "v1g_sample_bkg_counts: bad argument");
  return v1g_sample_bkg_internal(h, batch, n_steps, nullptr, first_step, counts_out, (cudaStream_t)stream);
}

extern "C" int v1g_sample_lgn_spikes(V1GHandle* h, int32_t batch, int32_t n_steps, const float* rates,
                                     int64_t rates_batch_stride, int64_t seed, uint8_t* x_out, void* stream) {
  if (!h) return V1G_EINVAL;
  if (batch <= 0 || n_steps < 0 || !rates || !x_out || rates_batch_stride < 0)
    return v1g_fail(h, V1G_EINVAL, "v1g_sample_lgn_spikes: bad argument");
  const int64_t n = (int64_t)batch * n_steps * h->cfg.n_lgn;
  if (n == 0) return V1G_OK;
  const int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)h->n_sms * 16);
  sample_lgn_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(batch, n_steps, h->cfg.n_lgn, rates,
                                                              rates_batch_stride, (unsigned)seed,
                                                              (unsigned)((uint64_t)seed >> 32), x_out);
  v1g_count_launches(1);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}
