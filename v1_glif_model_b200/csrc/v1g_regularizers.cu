// Weight regularisers of the reference, evaluated on the [nnz] weight vector next to the optimiser
// pass (value and gradient; the gradient is ACCUMULATED into the buffer the Exp-Adam kernel reads):
//   * MeanStiffRegularizer (loss_functions.py:171-220): the mean weight of every edge type is held
//     to its initial mean - mean over types of (mean_g - target_g)^2, or with
//     penalize_relative_change sqrt(mean_g ((mean_g - target_g) / denominator_g)^2);
//   * EarthMoversDistanceRegularizer (loss_functions.py:536-601): per edge type the sorted current
//     weights against the sorted initial weights, mean |sort(x_g) - y_g|, averaged over types.
// Both need the weights grouped by an integer id per synapse; any synapse order is fine as long as
// weights, ids and gradient use the same one.
#include <cub/cub.cuh>

#include "v1g_internal.h"

namespace {

// sum[g] += w, cnt[g] += 1.  The sums are kept in double precision: the penalty is built on the small
// difference between a group's mean and its target, which float atomics in arbitrary order would
// blur (and a sign-normalised optimiser step would then follow the noise).
__global__ void __launch_bounds__(256) group_sum_kernel(const float* __restrict__ w, const int32_t* __restrict__ gid,
                                                        int64_t n, double* __restrict__ sum, double* __restrict__ cnt) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int g = gid[i];
    atomicAdd(sum + g, (double)w[i]);
    atomicAdd(cnt + g, 1.0);
  }
}

// coef[g] = d loss / d mean_g / count_g; loss_out[0] += loss  (one block)
__global__ void __launch_bounds__(256) mean_stiff_coef_kernel(const double* __restrict__ sum, const double* __restrict__ cnt,
                                                              const float* __restrict__ target,
                                                              const float* __restrict__ denom, int G, float strength,
                                                              float* __restrict__ coef, float* loss_out) {
  __shared__ float red[256];
  float acc = 0.f;
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    const float c = fmaxf((float)cnt[g], 1.f);   // unsorted_segment_mean: empty segments have mean 0
    float d = (float)(sum[g] / (double)c - (double)target[g]);
    if (denom) d /= denom[g];
    acc += d * d;
  }
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  const float ms = red[0] / (float)G;
  const float loss = denom ? sqrtf(ms) : ms;
  // d loss / d d_g: plain 2 d_g / G; relative d_g / (G sqrt(ms))
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    const float c = fmaxf((float)cnt[g], 1.f);
    float d = (float)(sum[g] / (double)c - (double)target[g]);
    float dd;
    if (denom) {
      d /= denom[g];
      dd = loss > 0.f ? d / ((float)G * loss) / denom[g] : 0.f;
    } else {
      dd = 2.f * d / (float)G;
    }
    coef[g] = strength * dd / c;
  }
  if (threadIdx.x == 0 && loss_out) atomicAdd(loss_out, strength * loss);
}

__global__ void __launch_bounds__(256) add_group_coef_kernel(const int32_t* __restrict__ gid, const float* __restrict__ coef,
                                                             int64_t n, float* __restrict__ grad) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    grad[i] += coef[gid[i]];
}

// sortable key: group in the high word, the float's bits mapped to an order-preserving unsigned
__global__ void __launch_bounds__(256) emd_keys_kernel(const float* __restrict__ w, const int32_t* __restrict__ gid,
                                                       int64_t n, unsigned long long* __restrict__ keys,
                                                       int32_t* __restrict__ vals) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const unsigned u = __float_as_uint(w[i]);
    const unsigned s = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    keys[i] = ((unsigned long long)(unsigned)gid[i] << 32) | s;
    vals[i] = (int32_t)i;
  }
}

// position q of the sorted list holds the rank-(q - offsets[g]) weight of group g; its partner is the
// initial weight of the same rank
__global__ void __launch_bounds__(256) emd_kernel(const unsigned long long* __restrict__ keys,
                                                  const int32_t* __restrict__ vals, const float* __restrict__ w,
                                                  const float* __restrict__ sorted_initial,
                                                  const int32_t* __restrict__ offsets, int G, int64_t n, float strength,
                                                  float* __restrict__ grad, float* loss_out) {
  float loss = 0.f;
  for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < n; q += (int64_t)gridDim.x * blockDim.x) {
    const int g = (int)(keys[q] >> 32);
    const int ng = offsets[g + 1] - offsets[g];
    const int j = vals[q];
    const float d = w[j] - sorted_initial[q];
    const float scale = strength / ((float)G * (float)ng);
    loss += fabsf(d) * scale;
    grad[j] += d > 0.f ? scale : (d < 0.f ? -scale : 0.f);
  }
  for (int o = 16; o > 0; o >>= 1) loss += __shfl_down_sync(0xffffffffu, loss, o);
  if ((threadIdx.x & 31) == 0 && loss != 0.f && loss_out) atomicAdd(loss_out, loss);
}

}  // namespace

extern "C" int v1g_weight_regularizer(V1GHandle* h, int32_t kind, const float* w, const int32_t* group_ids, int64_t n,
                                      int32_t n_groups, const float* target, const int32_t* group_offsets,
                                      const float* denominator, float strength, float* loss_out, float* grad,
                                      void* stream) {
  if (!h) return V1G_EINVAL;
  if (kind < 0 || kind > 1 || !w || !group_ids || !target || !grad || n < 0 || n_groups <= 0 || n > 0x7fffffffLL)
    return v1g_fail(h, V1G_EINVAL, "v1g_weight_regularizer: bad argument");
  if (kind == 1 && !group_offsets) return v1g_fail(h, V1G_EINVAL, "v1g_weight_regularizer: the EMD form needs group_offsets");
  if (n == 0) return V1G_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)h->n_sms * 16);
  int rc;
  if (kind == 0) {
    // scratch: sum[G] | cnt[G] (double) | coef[G] (float)
    if ((rc = v1g_reserve(h, &h->reg_scratch, &h->reg_scratch_cap, 5 * (int64_t)n_groups + 2))) return rc;
    double* sum = (double*)(((uintptr_t)h->reg_scratch + 7) & ~(uintptr_t)7);
    double* cnt = sum + n_groups;
    float* coef = (float*)(cnt + n_groups);
    V1G_CUDA(h, cudaMemsetAsync(sum, 0, sizeof(double) * 2 * n_groups, st));
    group_sum_kernel<<<blocks, 256, 0, st>>>(w, group_ids, n, sum, cnt);
    mean_stiff_coef_kernel<<<1, 256, 0, st>>>(sum, cnt, target, denominator, n_groups, strength, coef, loss_out);
    add_group_coef_kernel<<<blocks, 256, 0, st>>>(group_ids, coef, n, grad);
    v1g_count_launches(3);
  } else {
    size_t cub_bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, (const unsigned long long*)nullptr, (unsigned long long*)nullptr,
                                    (const int32_t*)nullptr, (int32_t*)nullptr, (int)n, 0, 64, st);
    // scratch (4-byte words): vals_in[n] | vals_out[n] | keys_in[2n] | keys_out[2n] | cub storage
    const int64_t words = 2 * n + 4 * n + 4 + (int64_t)(cub_bytes + 3) / 4;
    if ((rc = v1g_reserve(h, &h->reg_scratch, &h->reg_scratch_cap, words))) return rc;
    int32_t* vals_in = h->reg_scratch;
    int32_t* vals_out = vals_in + n;
    unsigned long long* keys_in = (unsigned long long*)(((uintptr_t)(vals_out + n) + 7) & ~(uintptr_t)7);
    unsigned long long* keys_out = keys_in + n;
    void* cub_tmp = keys_out + n;
    emd_keys_kernel<<<blocks, 256, 0, st>>>(w, group_ids, n, keys_in, vals_in);
    int key_bits = 33;
    while ((1LL << (key_bits - 32)) < n_groups) ++key_bits;
    V1G_CUDA(h, cub::DeviceRadixSort::SortPairs(cub_tmp, cub_bytes, keys_in, keys_out, vals_in, vals_out, (int)n, 0,
                                                key_bits, st));
    emd_kernel<<<blocks, 256, 0, st>>>(keys_out, vals_out, w, target, group_offsets, n_groups, n, strength, grad,
                                       loss_out);
    v1g_count_launches(3);
  }
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

extern "C" int v1g_get_internal_order(V1GHandle* h, int source, int32_t* perm_out_host) {
  if (!h || !perm_out_host) return V1G_EINVAL;
  if (source < 0 || source >= V1G_NSRC) return v1g_fail(h, V1G_EINVAL, "unknown source %d", source);
  const V1GSource& s = h->src[source];
  if (!s.rowptr) return v1g_fail(h, V1G_ESTATE, "connectivity of source %d not set", source);
  if (s.nnz == 0) return V1G_OK;
  if (source == V1G_SRC_BKG) {
    if (s.in_perm)
      V1G_CUDA(h, cudaMemcpy(perm_out_host, s.in_perm, (size_t)s.nnz * sizeof(int32_t), cudaMemcpyDeviceToHost));
    else
      for (int64_t i = 0; i < s.nnz; ++i) perm_out_host[i] = (int32_t)i;
    return V1G_OK;
  }
  V1G_CUDA(h, cudaMemcpy(perm_out_host, s.perm, (size_t)s.nnz * sizeof(int32_t), cudaMemcpyDeviceToHost));
  return V1G_OK;
}

extern "C" int v1g_internal_weights(V1GHandle* h, int source, const float** w_out) {
  if (!h || !w_out) return V1G_EINVAL;
  if (source < 0 || source >= V1G_NSRC) return v1g_fail(h, V1G_EINVAL, "unknown source %d", source);
  const V1GSource& s = h->src[source];
  if (!s.rowptr) return v1g_fail(h, V1G_ESTATE, "connectivity of source %d not set", source);
  *w_out = (source == V1G_SRC_BKG) ? s.gather_w() : s.w;
  return V1G_OK;
}
