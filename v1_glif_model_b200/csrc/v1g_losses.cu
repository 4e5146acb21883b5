// Firing-rate distribution target of the reference (SpikeRateDistributionTarget.__call__,
// loss_functions.py:873-889; compute_spike_rate_target_loss / compute_spike_rate_distribution_loss /
// huber_quantile_loss, :626-681) evaluated on the spikes saved by the forward rollout.
//
// rates[n] = mean of z[b, t, n] over the batch and the steps [pre_delay, T - post_delay).  For every
// population the rates of its neurons are sorted and compared rank by rank with the population's
// sorted target sample: u_i = rate_(i) - target_i, tau_i = (i+1)/n, penalty
//   |tau - [u <= 0]| * (u^2 / (2 kappa)   if |u| <= kappa,   |u| - kappa/2   otherwise);
// the loss is rate_cost * (sum over all populations) / (neurons covered).  Its gradient with respect to
// z[b, t, n] is the same for all (b, t) inside the window, so the backward rollout only needs one
// coefficient per neuron.
//
// The sort is a stable radix sort of (population, spike count) keys: neurons with equal rates keep the
// order in which the population lists them (the reference shuffles them at random before sorting; the
// loss value does not depend on that choice).
#include <cub/device/device_radix_sort.cuh>

#include "v1g_internal.h"

namespace {

// count[n] = spikes of neuron n over all batch rows and the steps [t0, t1) of the saved rollout
__global__ void __launch_bounds__(256) window_count_kernel(const uint8_t* __restrict__ zr, int B, int N,
                                                           int t0, int t1, int32_t* __restrict__ count) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  int c = 0;
  for (int t = t0; t < t1; ++t)
    for (int b = 0; b < B; ++b) c += zr[((int64_t)t * B + b) * N + n] & 1;
  count[n] = c;
}

__global__ void __launch_bounds__(256) rate_keys_kernel(const int32_t* __restrict__ offsets, int G,
                                                        const int32_t* __restrict__ neurons,
                                                        const int32_t* __restrict__ count, int M,
                                                        unsigned long long* __restrict__ keys,
                                                        int32_t* __restrict__ vals) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= M) return;
  int lo = 0, hi = G;  // population of position p: offsets[g] <= p < offsets[g+1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (offsets[mid] <= p) lo = mid; else hi = mid;
  }
  keys[p] = ((unsigned long long)lo << 32) | (unsigned)count[neurons[p]];
  vals[p] = p;
}

// one thread per sorted position q; sorted positions of population g occupy the same range
// [offsets[g], offsets[g+1]) as its unsorted ones because the population is the leading key
__global__ void __launch_bounds__(256) rate_distribution_kernel(
    const unsigned long long* __restrict__ keys, const int32_t* __restrict__ vals,
    const int32_t* __restrict__ offsets, const int32_t* __restrict__ neurons,
    const float* __restrict__ targets, int M, float inv_bt, float kappa, float scale,
    float* __restrict__ rate_coef, float* __restrict__ loss_acc) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  float loss = 0.f;
  if (q < M) {
    const unsigned long long key = keys[q];
    const int g = (int)(key >> 32);
    const float rate = (float)(unsigned)(key & 0xffffffffull) * inv_bt;
    const int o0 = offsets[g], ng = offsets[g + 1] - o0;
    const float tau = (float)(q - o0 + 1) / (float)ng;
    const float u = rate - targets[q];
    const float num = fabsf(tau - (u <= 0.f ? 1.f : 0.f));
    const float au = fabsf(u);
    float du;
    if (au <= kappa) {
      loss = num / (2.f * kappa) * u * u;
      du = num / kappa * u;
    } else {
      loss = num * (au - 0.5f * kappa);
      du = u > 0.f ? num : -num;
    }
    atomicAdd(rate_coef + neurons[vals[q]], scale * du * inv_bt);
  }
  for (int o = 16; o > 0; o >>= 1) loss += __shfl_down_sync(0xffffffffu, loss, o);
  if ((threadIdx.x & 31) == 0 && loss != 0.f) atomicAdd(loss_acc, loss * scale);
}

}  // namespace

// rate_coef[n] += d loss / d z[b, t, n] for (b, t) in the window; loss_acc += loss.  `count` holds the
// spikes per neuron inside the window, or NULL to count them here from the saved spikes.
int v1g_rate_distribution_loss(V1GHandle* h, const V1GLossSpec* ls, const int32_t* count, int B, int T,
                               float* rate_coef, float* loss_acc, cudaStream_t st) {
  const int N = h->cfg.n_neurons, G = ls->n_rate_groups, M = ls->n_rate_neurons;
  if (G <= 0 || M <= 0) return V1G_OK;
  if (!ls->rate_group_offsets || !ls->rate_group_neurons || !ls->rate_group_targets)
    return v1g_fail(h, V1G_EINVAL, "rate populations: null offsets / neurons / targets");
  const int t0 = std::max(ls->rate_pre_delay, 0), t1 = T - std::max(ls->rate_post_delay, 0);
  if (t1 <= t0) return v1g_fail(h, V1G_EINVAL, "rate window [%d, %d) is empty", t0, t1);
  int rc;
  // scratch: count[N] | vals_in[M] | vals_out[M] | keys_in[M] | keys_out[M] | cub storage
  size_t cub_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, (const unsigned long long*)nullptr,
                                  (unsigned long long*)nullptr, (const int32_t*)nullptr, (int32_t*)nullptr, M,
                                  0, 64, st);
  const int64_t words = (int64_t)N + 2 * (int64_t)M + 4 * (int64_t)M + 2 + (int64_t)(cub_bytes + 3) / 4;
  if ((rc = v1g_reserve(h, &h->rate_scratch, &h->rate_scratch_cap, words))) return rc;
  int32_t* cnt = h->rate_scratch;
  int32_t* vals_in = cnt + N;
  int32_t* vals_out = vals_in + M;
  unsigned long long* keys_in = (unsigned long long*)(((uintptr_t)(vals_out + M) + 7) & ~(uintptr_t)7);
  unsigned long long* keys_out = keys_in + M;
  void* cub_tmp = keys_out + M;
  if (!count || t0 != 0 || t1 != T) {
    window_count_kernel<<<(N + 255) / 256, 256, 0, st>>>(h->tape_zr, B, N, t0, t1, cnt);
    v1g_count_launches(1);
    count = cnt;
  }
  rate_keys_kernel<<<(M + 255) / 256, 256, 0, st>>>(ls->rate_group_offsets, G, ls->rate_group_neurons, count, M,
                                                    keys_in, vals_in);
  int key_bits = 33;
  while ((1 << (key_bits - 32)) < G) ++key_bits;
  V1G_CUDA(h, cub::DeviceRadixSort::SortPairs(cub_tmp, cub_bytes, keys_in, keys_out, vals_in, vals_out, M, 0,
                                              key_bits, st));
  const float inv_bt = 1.f / ((float)B * (float)(t1 - t0));
  const float scale = ls->rate_cost * ls->loss_scale / (float)M;
  rate_distribution_kernel<<<(M + 255) / 256, 256, 0, st>>>(keys_out, vals_out, ls->rate_group_offsets,
                                                            ls->rate_group_neurons, ls->rate_group_targets, M,
                                                            inv_bt, ls->rate_kappa > 0.f ? ls->rate_kappa : 0.002f,
                                                            scale, rate_coef, loss_acc);
  v1g_count_launches(3);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}
