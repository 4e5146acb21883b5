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

// The saved rollout is one word per (step, batch row, neuron): the voltage with its two lowest mantissa
// bits replaced by (spiked, refractory).
// count[n] = spikes of neuron n over all batch rows and the steps [t0, t1) of the saved rollout
__global__ void __launch_bounds__(256) window_count_kernel(const uint32_t* __restrict__ zr, int B, int N,
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
    window_count_kernel<<<(N + 255) / 256, 256, 0, st>>>((const uint32_t*)h->tape_v, B, N, t0, t1, cnt);
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

// ---------------------------------------------------------------------------------------------
// Synchrony target of the reference in full (SynchronizationLoss.__call__ and pop_fano_tf,
// loss_functions.py:964-1044) for given samples.  A sample is one trial (batch row) and a set of
// neurons; pop[s][t] is its population spike count at step t of the window [t0, t0 + W).  For every
// bin size smaller than W/2 the counts are summed in non-overlapping bins (incomplete last bin
// dropped), Fano = biased variance / max(mean, 1e-7) per sample, averaged over the samples; the loss
// is sync_cost * mean_k (target_k - Fano_k)^2.  g[s][t] = d loss / d pop[s][t] is what the backward
// rollout adds to dL/dz of the sample's members in the sample's trial.
namespace {

constexpr int SYNC_MAX_BINS = 32;
constexpr float SYNC_EPS = 1e-7f;

struct SyncBins {
  int n;                       // bin sizes in use (already restricted to those below W/2)
  int size[SYNC_MAX_BINS];
  float target[SYNC_MAX_BINS];
};

// membership lists: first[n] -> position -> next[position]; pos_sample[position] = sample
__global__ void __launch_bounds__(256) sync_members_kernel(const int32_t* __restrict__ offsets, int S,
                                                           const int32_t* __restrict__ neurons, int P,
                                                           int32_t* first, int32_t* __restrict__ next,
                                                           int32_t* __restrict__ pos_sample) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= P) return;
  int lo = 0, hi = S;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (offsets[mid] <= p) lo = mid; else hi = mid;
  }
  pos_sample[p] = lo;
  next[p] = atomicExch(first + neurons[p], p);
}

// pop[s][t - t0] = spikes of the sample's neurons in its trial at step t
__global__ void __launch_bounds__(256) sync_pop_kernel(const uint32_t* __restrict__ zr, int B, int N,
                                                       const int32_t* __restrict__ trial,
                                                       const int32_t* __restrict__ offsets,
                                                       const int32_t* __restrict__ neurons, int t0, int W,
                                                       float* __restrict__ pop) {
  const int s = blockIdx.x;
  const int b = trial[s], p0 = offsets[s], p1 = offsets[s + 1];
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const uint32_t* row = zr + ((int64_t)(t0 + i) * B + b) * N;
    int c = 0;
    for (int p = p0; p < p1; ++p) c += row[neurons[p]] & 1;
    pop[(int64_t)s * W + i] = (float)c;
  }
}

__device__ __forceinline__ float block_sum(float v, float* ws) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += ws[w];
  return t;
}

// pass 0: stats[s][k] = (mean, variance) of the bin counts, fano_mean[k] += Fano / S
// pass 1: g[s][t] = sum_k dL/dFano_k * dFano_sk / d pop[s][t]
__global__ void __launch_bounds__(256) sync_fano_kernel(const float* __restrict__ pop, int S, int W, SyncBins bins,
                                                        int pass, float cost, float2* __restrict__ stats,
                                                        float* __restrict__ fano_mean, float* __restrict__ g) {
  extern __shared__ float cnt_s[];  // bin counts of one bin size [W]
  __shared__ float ws[8];
  const int s = blockIdx.x;
  const float* ps = pop + (int64_t)s * W;
  for (int k = 0; k < bins.n; ++k) {
    const int bs = bins.size[k], nb = W / bs;
    __syncthreads();
    for (int j = threadIdx.x; j < nb; j += blockDim.x) {
      float c = 0.f;
      for (int i = 0; i < bs; ++i) c += ps[j * bs + i];
      cnt_s[j] = c;
    }
    __syncthreads();
    if (pass == 0) {
      float a = 0.f;
      for (int j = threadIdx.x; j < nb; j += blockDim.x) a += cnt_s[j];
      const float mean = block_sum(a, ws) / (float)nb;
      float q = 0.f;
      for (int j = threadIdx.x; j < nb; j += blockDim.x) q += (cnt_s[j] - mean) * (cnt_s[j] - mean);
      const float var = block_sum(q, ws) / (float)nb;
      if (threadIdx.x == 0) {
        stats[(int64_t)s * bins.n + k] = make_float2(mean, var);
        atomicAdd(fano_mean + k, var / fmaxf(mean, SYNC_EPS) / (float)S);
      }
    } else {
      const float2 mv = stats[(int64_t)s * bins.n + k];
      const float dldf = cost * 2.f * (fano_mean[k] - bins.target[k]) / (float)bins.n / (float)S;
      const float m = fmaxf(mv.x, SYNC_EPS);
      // d(var/m)/dc_j = 2 (c_j - mean) / (nb m) - [mean > eps] var / (m^2 nb)
      const float k1 = 2.f / ((float)nb * m), k0 = mv.x > SYNC_EPS ? mv.y / (m * m * (float)nb) : 0.f;
      for (int i = threadIdx.x; i < nb * bs; i += blockDim.x)
        g[(int64_t)s * W + i] += dldf * (k1 * (cnt_s[i / bs] - mv.x) - k0);
    }
  }
}

__global__ void sync_loss_value_kernel(const float* __restrict__ fano_mean, SyncBins bins, float cost,
                                       float* __restrict__ loss_acc) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    float a = 0.f;
    for (int k = 0; k < bins.n; ++k) a += (bins.target[k] - fano_mean[k]) * (bins.target[k] - fano_mean[k]);
    if (bins.n > 0) atomicAdd(loss_acc, cost * a / (float)bins.n);
  }
}

}  // namespace

// Fills h->sync_* (membership lists and g) for the backward rollout; loss_acc += loss.
int v1g_sync_samples_loss(V1GHandle* h, const V1GLossSpec* ls, int B, int T, float* loss_acc,
                          V1GSyncTables* out, cudaStream_t st) {
  const int N = h->cfg.n_neurons, S = ls->n_sync_samples, P = ls->n_sync_members;
  out->first = nullptr;
  if (S <= 0 || P <= 0) return V1G_OK;
  if (!ls->sync_sample_trial || !ls->sync_sample_offsets || !ls->sync_sample_neurons ||
      (ls->n_sync_bins > 0 && (!ls->sync_bin_sizes || !ls->sync_bin_targets)))
    return v1g_fail(h, V1G_EINVAL, "synchrony samples: null trial / offsets / neurons / bins");
  const int t0 = std::max(ls->sync_t_start, 0), t1 = ls->sync_t_end > 0 ? std::min(ls->sync_t_end, T) : T;
  const int W = t1 - t0;
  if (W < 2) return v1g_fail(h, V1G_EINVAL, "synchrony window [%d, %d) is too short", t0, t1);
  SyncBins bins;
  bins.n = 0;
  for (int k = 0; k < ls->n_sync_bins; ++k) {  // host arrays
    const int bs = ls->sync_bin_sizes[k];
    if (bs < 1) return v1g_fail(h, V1G_EINVAL, "synchrony bin size %d", bs);
    if (!(bs < W / 2)) continue;
    if (bins.n == SYNC_MAX_BINS) return v1g_fail(h, V1G_ERANGE, "more than %d synchrony bin sizes", SYNC_MAX_BINS);
    bins.size[bins.n] = bs;
    bins.target[bins.n] = ls->sync_bin_targets[k];
    ++bins.n;
  }
  const float cost = ls->sync_cost * ls->loss_scale;
  // scratch (4-byte words): first[N] | next[P] | pos_sample[P] | fano_mean[32] | stats[S*32*2] | pop[S*W] | g[S*W]
  const int64_t words = (int64_t)N + 2 * (int64_t)P + SYNC_MAX_BINS + (int64_t)S * SYNC_MAX_BINS * 2 + 2 * (int64_t)S * W + 2;
  int rc;
  if ((rc = v1g_reserve(h, &h->sync_scratch, &h->sync_scratch_cap, words))) return rc;
  int32_t* first = h->sync_scratch;
  int32_t* next = first + N;
  int32_t* pos_sample = next + P;
  float* fano_mean = (float*)(pos_sample + P);
  float2* stats = (float2*)(((uintptr_t)(fano_mean + SYNC_MAX_BINS) + 7) & ~(uintptr_t)7);
  float* pop = (float*)(stats + (int64_t)S * SYNC_MAX_BINS);
  float* g = pop + (int64_t)S * W;
  V1G_CUDA(h, cudaMemsetAsync(first, 0xff, (size_t)N * sizeof(int32_t), st));  // -1: in no sample
  V1G_CUDA(h, cudaMemsetAsync(fano_mean, 0, SYNC_MAX_BINS * sizeof(float), st));
  V1G_CUDA(h, cudaMemsetAsync(g, 0, (size_t)S * W * sizeof(float), st));
  sync_members_kernel<<<(P + 255) / 256, 256, 0, st>>>(ls->sync_sample_offsets, S, ls->sync_sample_neurons, P,
                                                       first, next, pos_sample);
  sync_pop_kernel<<<S, 256, 0, st>>>((const uint32_t*)h->tape_v, B, N, ls->sync_sample_trial, ls->sync_sample_offsets,
                                     ls->sync_sample_neurons, t0, W, pop);
  const size_t smem = (size_t)W * sizeof(float);
  if (smem > 200 * 1024) return v1g_fail(h, V1G_ERANGE, "synchrony window of %d steps is too long", W);
  if (smem > 48 * 1024)
    V1G_CUDA(h, cudaFuncSetAttribute(sync_fano_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  sync_fano_kernel<<<S, 256, smem, st>>>(pop, S, W, bins, 0, cost, stats, fano_mean, g);
  sync_fano_kernel<<<S, 256, smem, st>>>(pop, S, W, bins, 1, cost, stats, fano_mean, g);
  sync_loss_value_kernel<<<1, 32, 0, st>>>(fano_mean, bins, cost, loss_acc);
  v1g_count_launches(5);
  V1G_CUDA(h, cudaGetLastError());
  out->first = first;
  out->next = next;
  out->pos_sample = pos_sample;
  out->trial = ls->sync_sample_trial;
  out->g = g;
  out->t0 = t0;
  out->W = W;
  return V1G_OK;
}

// ---------------------------------------------------------------------------------------------
// Population OSI/DSI target of the reference (OrientationSelectivityLoss with method "crowd_osi":
// __call__, crowd_osi_loss, _compute_osi_dsi_core; loss_functions.py:1340-1440).
// rates[b, n] = mean of the spikes over the steps [t0, t1), optionally divided by
// max(normalizer[n], 0.0005); delta = (angle[b] - tuning[n]) pi / 180.  Per trial and cell type:
// den = max(mean_n rates, 0.0005), osi = mean_n(rates cos 2 delta) / den, dsi = mean_n(rates cos delta) /
// den; both averaged over the trials; loss = cost * sum_type count ((osi - osi_t)^2 + (dsi - dsi_t)^2) /
// sum_type count.  The gradient with respect to z[b, t, n] is one coefficient per (b, n) for all steps
// of the window.
namespace {

constexpr int OSI_MAX_TYPES = 64;
constexpr float OSI_MIN_RATE = 0.0005f;

__global__ void __launch_bounds__(256) osi_count_kernel(const uint32_t* __restrict__ zr, int B, int N, int t0,
                                                        int t1, int32_t* __restrict__ cnt /*[B][N]*/) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (n >= N) return;
  int c = 0;
  for (int t = t0; t < t1; ++t) c += zr[((int64_t)t * B + b) * N + n] & 1;
  cnt[(int64_t)b * N + n] = c;
}

__device__ __forceinline__ float osi_rate(int c, float inv_w, const float* normalizer, int n) {
  float r = (float)c * inv_w;
  if (normalizer) r = r / fmaxf(normalizer[n], OSI_MIN_RATE);
  return r;
}

// seg[b][ty] = (sum rates, sum rates cos 2 delta, sum rates cos delta); seg_n[ty] = neurons of the type
__global__ void __launch_bounds__(256) osi_segment_kernel(const int32_t* __restrict__ cnt, int B, int N,
                                                          float inv_w, const float* __restrict__ normalizer,
                                                          const float* __restrict__ angle,
                                                          const float* __restrict__ tuning,
                                                          const int32_t* __restrict__ type_ids, int n_types,
                                                          float* __restrict__ seg, float* __restrict__ seg_n) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (n >= N) return;
  const int ty = type_ids[n];
  if (b == 0) atomicAdd(seg_n + ty, 1.f);
  const int c = cnt[(int64_t)b * N + n];
  if (c == 0) return;
  const float r = osi_rate(c, inv_w, normalizer, n);
  const float d = (angle[b] - tuning[n]) * (3.14159265358979323846f / 180.f);
  float* o = seg + ((int64_t)b * n_types + ty) * 3;
  atomicAdd(o, r);
  atomicAdd(o + 1, r * cosf(2.f * d));
  atomicAdd(o + 2, r * cosf(d));
}

struct OsiTargets {
  int n;
  float osi[OSI_MAX_TYPES], dsi[OSI_MAX_TYPES], count[OSI_MAX_TYPES];
};

// one block: loss value and, per (b, type), the three coefficients of d loss / d rates[b, n]:
//   d = ca * cos 2 delta + cb * cos delta + cc
__global__ void osi_type_kernel(const float* __restrict__ seg, const float* __restrict__ seg_n, int B,
                                OsiTargets tg, float cost, float* __restrict__ coef3, float* __restrict__ loss_acc) {
  __shared__ float osi_s[OSI_MAX_TYPES], dsi_s[OSI_MAX_TYPES];
  const int ty = threadIdx.x;
  float csum = 0.f;
  for (int k = 0; k < tg.n; ++k) csum += tg.count[k];
  if (ty < tg.n) {
    const float nn = fmaxf(seg_n[ty], 1.f);
    float so = 0.f, sd = 0.f;
    for (int b = 0; b < B; ++b) {
      const float* o = seg + ((int64_t)b * tg.n + ty) * 3;
      const float den = fmaxf(o[0] / nn, OSI_MIN_RATE);
      so += (o[1] / nn) / den;
      sd += (o[2] / nn) / den;
    }
    osi_s[ty] = so / (float)B;
    dsi_s[ty] = sd / (float)B;
    const float dl_osi = cost * tg.count[ty] * 2.f * (osi_s[ty] - tg.osi[ty]) / csum / (float)B;
    const float dl_dsi = cost * tg.count[ty] * 2.f * (dsi_s[ty] - tg.dsi[ty]) / csum / (float)B;
    for (int b = 0; b < B; ++b) {
      const float* o = seg + ((int64_t)b * tg.n + ty) * 3;
      const float mean = o[0] / nn, den = fmaxf(mean, OSI_MIN_RATE);
      float* c3 = coef3 + ((int64_t)b * tg.n + ty) * 3;
      c3[0] = dl_osi / (nn * den);
      c3[1] = dl_dsi / (nn * den);
      c3[2] = mean > OSI_MIN_RATE ? -(dl_osi * (o[1] / nn) + dl_dsi * (o[2] / nn)) / (den * den * nn) : 0.f;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f;
    for (int k = 0; k < tg.n; ++k)
      a += tg.count[k] * ((osi_s[k] - tg.osi[k]) * (osi_s[k] - tg.osi[k]) + (dsi_s[k] - tg.dsi[k]) * (dsi_s[k] - tg.dsi[k]));
    atomicAdd(loss_acc, cost * a / csum);
  }
}

// coef[b][n] = d loss / d z[b, t, n] for t in the window
__global__ void __launch_bounds__(256) osi_coef_kernel(int B, int N, float inv_w, const float* __restrict__ normalizer,
                                                       const float* __restrict__ angle, const float* __restrict__ tuning,
                                                       const int32_t* __restrict__ type_ids, int n_types,
                                                       const float* __restrict__ coef3, float* __restrict__ coef) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (n >= N) return;
  const float* c3 = coef3 + ((int64_t)b * n_types + type_ids[n]) * 3;
  const float d = (angle[b] - tuning[n]) * (3.14159265358979323846f / 180.f);
  float g = c3[0] * cosf(2.f * d) + c3[1] * cosf(d) + c3[2];
  if (normalizer) g = g / fmaxf(normalizer[n], OSI_MIN_RATE);
  coef[(int64_t)b * N + n] = g * inv_w;
}

}  // namespace

// *coef_out = [B][N] table of d loss / d z[b, t, n] for t in [*t0_out, *t1_out) (NULL: term off); loss_acc += loss.
int v1g_osi_dsi_loss(V1GHandle* h, const V1GLossSpec* ls, int B, int T, float* loss_acc, const float** coef_out,
                     int* t0_out, int* t1_out, cudaStream_t st) {
  *coef_out = nullptr;
  const int N = h->cfg.n_neurons, n_types = ls->n_osi_types;
  if (ls->osi_cost == 0.f || n_types <= 0) return V1G_OK;
  if (n_types > OSI_MAX_TYPES) return v1g_fail(h, V1G_ERANGE, "more than %d OSI/DSI cell types", OSI_MAX_TYPES);
  if (!ls->osi_angle || !ls->osi_tuning_angle || !ls->osi_type_ids || !ls->osi_targets || !ls->dsi_targets ||
      !ls->osi_type_counts)
    return v1g_fail(h, V1G_EINVAL, "OSI/DSI target: null angle / tuning / types / targets");
  const int t0 = std::max(ls->osi_pre_delay, 0), t1 = T - std::max(ls->osi_post_delay, 0);
  if (t1 <= t0) return v1g_fail(h, V1G_EINVAL, "OSI/DSI window [%d, %d) is empty", t0, t1);
  OsiTargets tg;
  tg.n = n_types;
  for (int k = 0; k < n_types; ++k) {  // host arrays
    tg.osi[k] = ls->osi_targets[k];
    tg.dsi[k] = ls->dsi_targets[k];
    tg.count[k] = ls->osi_type_counts[k];
  }
  // scratch (4-byte words): cnt[B*N] | coef[B*N] | seg[B*types*3] | coef3[B*types*3] | seg_n[types]
  const int64_t bn = (int64_t)B * N, bt3 = (int64_t)B * n_types * 3;
  int rc;
  if ((rc = v1g_reserve(h, &h->osi_scratch, &h->osi_scratch_cap, 2 * bn + 2 * bt3 + n_types))) return rc;
  int32_t* cnt = (int32_t*)h->osi_scratch;
  float* coef = h->osi_scratch + bn;
  float* seg = coef + bn;
  float* coef3 = seg + bt3;
  float* seg_n = coef3 + bt3;
  V1G_CUDA(h, cudaMemsetAsync(seg, 0, (size_t)(2 * bt3 + n_types) * sizeof(float), st));
  const dim3 grid((N + 255) / 256, B);
  const float inv_w = 1.f / (float)(t1 - t0);
  osi_count_kernel<<<grid, 256, 0, st>>>((const uint32_t*)h->tape_v, B, N, t0, t1, cnt);
  osi_segment_kernel<<<grid, 256, 0, st>>>(cnt, B, N, inv_w, ls->osi_normalizer, ls->osi_angle, ls->osi_tuning_angle,
                                           ls->osi_type_ids, n_types, seg, seg_n);
  osi_type_kernel<<<1, OSI_MAX_TYPES, 0, st>>>(seg, seg_n, B, tg, ls->osi_cost * ls->loss_scale, coef3, loss_acc);
  osi_coef_kernel<<<grid, 256, 0, st>>>(B, N, inv_w, ls->osi_normalizer, ls->osi_angle, ls->osi_tuning_angle,
                                        ls->osi_type_ids, n_types, coef3, coef);
  v1g_count_launches(4);
  V1G_CUDA(h, cudaGetLastError());
  *coef_out = coef;
  *t0_out = t0;
  *t1_out = t1;
  return V1G_OK;
}
