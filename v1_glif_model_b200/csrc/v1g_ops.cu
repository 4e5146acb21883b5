// Operator-level kernels: one launch group per TensorFlow-level callable of the reference cell.
// These are the functional (state in -> state out) forms used for per-step parity and by the
// TensorFlow op shim; the throughput path is the fused rollout.
#include <algorithm>

#include "v1g_internal.h"

namespace {

struct DenseConsts {
  float sd[V1G_MAX_RECEPTORS], pinit[V1G_MAX_RECEPTORS], dtsd[V1G_MAX_RECEPTORS];
  float vd_keep, vd_drop, damp, width, gauss_std;
  int N, R, D, hard_reset, gauss;
};

// ------------------------------------------------------------------------------------------
// spike -> current scatter over a compacted active list (models.py:134-169, 833-857, 896-934)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) scatter_fwd_kernel(
    const int64_t* __restrict__ coords, const int32_t* __restrict__ count,
    const int32_t* __restrict__ rowptr, const int32_t* __restrict__ post,
    const float* __restrict__ w, const uint8_t* __restrict__ sid, const float* __restrict__ basis,
    const float* __restrict__ x, int64_t n_cols, int N, int R, int S, int D, int n_src, int is_bkg,
    float* __restrict__ i_flat) {
  extern __shared__ float basis_s[];
  for (int i = threadIdx.x; i < S * R; i += blockDim.x) basis_s[i] = basis[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t n_act = *count;
  for (int64_t e = gw; e < n_act; e += nw) {
    const int64_t b = coords[2 * e], col = coords[2 * e + 1];
    const int64_t row = (D > 1) ? (col % n_src) * D + col / n_src : col;
    const float mult = is_bkg ? x[b * n_cols + col] : 1.f;
    const int j1 = rowptr[row + 1];
    for (int j = rowptr[row] + lane; j < j1; j += 32) {
      float wv = w[j];
      if (is_bkg) wv = wv * mult;  // (w * n_pre_spikes) * basis, models.py:931
      const float* bs = basis_s + (int)sid[j] * R;
      float* dst = i_flat + (b * N + post[j]) * R;
      for (int r = 0; r < R; ++r) {
        const float c = wv * bs[r];
        if (c != 0.f) atomicAdd(dst + r, c);
      }
    }
  }
}

// d_x[b, col] = sum over the synapses of column col of w * sum_r basis[sid,r]*dy[b,post,r]
// (models.py:187-202; every synapse, active or not).
__global__ void __launch_bounds__(256) gather_dx_kernel(
    const int32_t* __restrict__ rowptr, const int32_t* __restrict__ post,
    const float* __restrict__ w, const uint8_t* __restrict__ sid, const float* __restrict__ basis,
    const float* __restrict__ dy, int64_t n_cols, int B, int N, int R, int S, int D, int n_src,
    float* __restrict__ d_x) {
  extern __shared__ float basis_s[];
  for (int i = threadIdx.x; i < S * R; i += blockDim.x) basis_s[i] = basis[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t total = (int64_t)B * n_cols;
  for (int64_t e = gw; e < total; e += nw) {
    const int64_t b = e / n_cols, col = e - b * n_cols;
    const int64_t row = (D > 1) ? (col % n_src) * D + col / n_src : col;
    const int j1 = rowptr[row + 1];
    float acc = 0.f;
    for (int j = rowptr[row] + lane; j < j1; j += 32) {
      const float* bs = basis_s + (int)sid[j] * R;
      const float* g = dy + (b * N + post[j]) * R;
      const float wv = w[j];
      float s = 0.f;
      for (int r = 0; r < R; ++r) s += g[r] * (wv * bs[r]);
      acc += s;
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if (lane == 0) d_x[e] = acc;
  }
}

// d_w[syn] += sum_r dy[b,post,r]*basis[sid,r] for the synapses of active columns
// (models.py:226-240); the background source carries the Poisson count (autodiff of :931).
__global__ void __launch_bounds__(256) scatter_dw_kernel(
    const int64_t* __restrict__ coords, const int32_t* __restrict__ count,
    const int32_t* __restrict__ rowptr, const int32_t* __restrict__ post,
    const uint8_t* __restrict__ sid, const int32_t* __restrict__ perm,
    const float* __restrict__ basis, const float* __restrict__ x, const float* __restrict__ dy,
    int64_t n_cols, int N, int R, int S, int D, int n_src, int is_bkg, float* __restrict__ d_w) {
  extern __shared__ float basis_s[];
  for (int i = threadIdx.x; i < S * R; i += blockDim.x) basis_s[i] = basis[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t n_act = *count;
  for (int64_t e = gw; e < n_act; e += nw) {
    const int64_t b = coords[2 * e], col = coords[2 * e + 1];
    const int64_t row = (D > 1) ? (col % n_src) * D + col / n_src : col;
    const float mult = is_bkg ? x[b * n_cols + col] : 1.f;
    const int j1 = rowptr[row + 1];
    for (int j = rowptr[row] + lane; j < j1; j += 32) {
      const float* bs = basis_s + (int)sid[j] * R;
      const float* g = dy + (b * N + post[j]) * R;
      float s = 0.f;
      for (int r = 0; r < R; ++r) s += g[r] * bs[r];
      if (is_bkg) s = s * mult;
      atomicAdd(d_w + perm[j], s);
    }
  }
}

// ------------------------------------------------------------------------------------------
// dense update (models.py:979-1028) + spike, refractory gate and buffer shift (:1105-1117)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) step_fwd_kernel(
    DenseConsts k, int B, const float* __restrict__ decay, const float* __restrict__ cf,
    const float* __restrict__ asc_decay, const float* __restrict__ asc_amps,
    const int32_t* __restrict__ tref, V1GState in, const float* __restrict__ rec_inputs,
    V1GState out, float* __restrict__ z_out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int N = k.N, R = k.R, D = k.D;
  if (i >= (int64_t)B * N) return;
  const int b = (int)(i / N), n = (int)(i - (int64_t)b * N);
  const float* zb = in.z_buf + (int64_t)b * D * N;
  const float prev_z = zb[n];
  float csum = 0.f;
  const int64_t o = i * R;
  for (int r = 0; r < R; ++r) {
    const float I = rec_inputs[o + r], pr = in.psc_rise[o + r], p = in.psc[o + r];
    out.psc_rise[o + r] = pr * k.sd[r] + I * k.pinit[r];
    out.psc[o + r] = p * k.sd[r] + k.dtsd[r] * pr;
    csum = (r == 0) ? p : csum + p;
  }
  const float a0 = in.asc[i * 2], a1 = in.asc[i * 2 + 1];
  out.asc[i * 2] = asc_decay[n * 2] * a0 + prev_z * asc_amps[n * 2];
  out.asc[i * 2 + 1] = asc_decay[n * 2 + 1] * a1 + prev_z * asc_amps[n * 2 + 1];
  const float c1 = csum + (a0 + a1);
  const float v = in.v[i];
  const float dv = v * k.vd_keep + v * k.vd_drop;
  float nv = (decay[n] * dv + cf[n] * c1) - prev_z;
  int nr = (int)in.r[i] + (int)prev_z * tref[n] - 1;
  nr = nr > 0 ? nr : 0;
  if (k.hard_reset && nr > 0) nv = 0.f;
  float z = ((nv - 1.f) > 0.f) ? 1.f : 0.f;
  if (nr > 0) z = 0.f;
  out.v[i] = nv;
  out.r[i] = (int8_t)nr;
  float* zo = out.z_buf + (int64_t)b * D * N;
  zo[n] = z;
  for (int d = 1; d < D; ++d) zo[(int64_t)d * N + n] = zb[(int64_t)(d - 1) * N + n];
  if (z_out) z_out[i] = z;
}

__device__ __forceinline__ float pseudo_h(float vs, const DenseConsts& k) {
  if (k.gauss) return expf(-(vs * vs) / (k.gauss_std * k.gauss_std)) * k.damp;
  float a = fabsf(vs);
  if (k.width != 1.f) a = a / k.width;
  return k.damp * fmaxf(1.f - a, 0.f);
}

__global__ void __launch_bounds__(256) step_bwd_kernel(
    DenseConsts k, int B, const float* __restrict__ decay, const float* __restrict__ cf,
    const float* __restrict__ asc_decay, V1GState g_out, const float* __restrict__ g_z,
    const float* __restrict__ g_v_out, const float* __restrict__ new_v,
    const int8_t* __restrict__ new_r, V1GState g_in, float* __restrict__ g_rec_inputs) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int N = k.N, R = k.R, D = k.D;
  if (i >= (int64_t)B * N) return;
  const int b = (int)(i / N), n = (int)(i - (int64_t)b * N);
  const float* gzb = g_out.z_buf ? g_out.z_buf + (int64_t)b * D * N : nullptr;
  float gz = g_z ? g_z[i] : 0.f;
  if (gzb) gz += gzb[n];
  const bool free_ = new_r[i] == 0;
  float gnv = (g_out.v ? g_out.v[i] : 0.f) + (g_v_out ? g_v_out[i] : 0.f);
  if (free_) gnv += gz * pseudo_h(new_v[i] - 1.f, k);
  if (k.hard_reset && !free_) gnv = 0.f;
  g_in.v[i] = decay[n] * k.vd_keep * gnv;
  const float gc1 = cf[n] * gnv;
  const int64_t o = i * R;
  for (int r = 0; r < R; ++r) {
    const float gpr = g_out.psc_rise ? g_out.psc_rise[o + r] : 0.f;
    const float gp = g_out.psc ? g_out.psc[o + r] : 0.f;
    g_in.psc[o + r] = k.sd[r] * gp + gc1;
    g_in.psc_rise[o + r] = k.sd[r] * gpr + k.dtsd[r] * gp;
    g_rec_inputs[o + r] = k.pinit[r] * gpr;
  }
  for (int q = 0; q < 2; ++q) {
    const float ga = g_out.asc ? g_out.asc[i * 2 + q] : 0.f;
    g_in.asc[i * 2 + q] = asc_decay[n * 2 + q] * ga + gc1;
  }
  if (g_in.z_buf) {
    float* go = g_in.z_buf + (int64_t)b * D * N;
    for (int d = 0; d < D - 1; ++d) go[(int64_t)d * N + n] = gzb ? gzb[(int64_t)(d + 1) * N + n] : 0.f;
    go[(int64_t)(D - 1) * N + n] = 0.f;
  }
}

DenseConsts make_consts(const V1GHandle* h) {
  DenseConsts k;
  const V1GConfig& c = h->cfg;
  for (int r = 0; r < V1G_MAX_RECEPTORS; ++r) {
    k.sd[r] = r < c.n_receptors ? h->syn_decay[r] : 0.f;
    k.pinit[r] = r < c.n_receptors ? h->psc_initial[r] : 0.f;
    k.dtsd[r] = c.dt * k.sd[r];
  }
  k.vd_keep = h->vd_keep;
  k.vd_drop = h->vd_drop;
  k.damp = c.dampening_factor;
  k.width = c.pseudo_width;
  k.gauss_std = c.gauss_std;
  k.N = c.n_neurons;
  k.R = c.n_receptors;
  k.D = c.max_delay;
  k.hard_reset = (c.flags & V1G_FLAG_HARD_RESET) ? 1 : 0;
  k.gauss = (c.flags & V1G_FLAG_PSEUDO_GAUSS) ? 1 : 0;
  return k;
}

int check_source(V1GHandle* h, int source, int batch) {
  if (source < 0 || source >= V1G_NSRC) return v1g_fail(h, V1G_EINVAL, "unknown source %d", source);
  if (!h->src[source].rowptr) return v1g_fail(h, V1G_ESTATE, "connectivity of source %d not set", source);
  if (!h->params_set) return v1g_fail(h, V1G_ESTATE, "neuron parameters not set");
  if (batch <= 0) return v1g_fail(h, V1G_EINVAL, "batch must be > 0");
  return V1G_OK;
}

// compaction of x[B, n_cols] > 0 into h->coords / h->d_count
int compact_active(V1GHandle* h, const float* x, int batch, int64_t n_cols, cudaStream_t st) {
  const int nseg = (int)((n_cols + V1G_SEG - 1) / V1G_SEG);
  int rc;
  if ((rc = v1g_reserve(h, &h->seg_counts, &h->seg_cap, (int64_t)batch * nseg + 1))) return rc;
  if ((rc = v1g_reserve(h, &h->coords, &h->coords_cap, 2 * (int64_t)batch * n_cols))) return rc;
  if ((rc = v1g_compact_count_scan(h, V1G_COMPACT_F32_COORDS, x, batch, n_cols, 0, h->seg_counts,
                                   nullptr, st)))
    return rc;
  return v1g_compact_fill(h, V1G_COMPACT_F32_COORDS, x, batch, n_cols, 0, h->seg_counts, h->coords,
                          (int64_t)batch * n_cols, st);
}

}  // namespace

extern "C" int v1g_syn_currents_fwd(V1GHandle* h, int source, const float* x, int32_t batch,
                                    float* i_flat, void* stream) {
  if (!h) return V1G_EINVAL;
  int rc = check_source(h, source, batch);
  if (rc) return rc;
  if (!x || !i_flat) return v1g_fail(h, V1G_EINVAL, "v1g_syn_currents_fwd: null argument");
  cudaStream_t st = (cudaStream_t)stream;
  const V1GSource& s = h->src[source];
  const int N = h->cfg.n_neurons, R = h->cfg.n_receptors, S = h->cfg.n_syn_types;
  V1G_CUDA(h, cudaMemsetAsync(i_flat, 0, (size_t)batch * N * R * sizeof(float), st));
  if (s.nnz == 0) return V1G_OK;
  if ((rc = compact_active(h, x, batch, s.n_cols, st))) return rc;
  scatter_fwd_kernel<<<h->n_sms * 4, 256, S * R * sizeof(float), st>>>(
      h->coords, h->d_count, s.rowptr, s.post, s.w, s.sid, h->basis, x, s.n_cols, N, R, S, s.delays,
      s.n_src, source == V1G_SRC_BKG, i_flat);
  v1g_count_launches(1);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

extern "C" int v1g_syn_currents_bwd(V1GHandle* h, int source, const float* x, const float* dy,
                                    int32_t batch, float* d_x, float* d_w, void* stream) {
  if (!h) return V1G_EINVAL;
  int rc = check_source(h, source, batch);
  if (rc) return rc;
  if (!x || !dy) return v1g_fail(h, V1G_EINVAL, "v1g_syn_currents_bwd: null argument");
  cudaStream_t st = (cudaStream_t)stream;
  const V1GSource& s = h->src[source];
  const int N = h->cfg.n_neurons, R = h->cfg.n_receptors, S = h->cfg.n_syn_types;
  if (d_x) {
    gather_dx_kernel<<<h->n_sms * 8, 256, S * R * sizeof(float), st>>>(
        s.rowptr, s.post, s.w, s.sid, h->basis, dy, s.n_cols, batch, N, R, S, s.delays, s.n_src, d_x);
    V1G_CUDA(h, cudaGetLastError());
  }
  if (d_w && s.nnz > 0) {
    V1G_CUDA(h, cudaMemsetAsync(d_w, 0, (size_t)s.nnz * sizeof(float), st));
    if ((rc = compact_active(h, x, batch, s.n_cols, st))) return rc;
    scatter_dw_kernel<<<h->n_sms * 4, 256, S * R * sizeof(float), st>>>(
        h->coords, h->d_count, s.rowptr, s.post, s.sid, s.perm, h->basis, x, dy, s.n_cols, N, R, S,
        s.delays, s.n_src, source == V1G_SRC_BKG, d_w);
    V1G_CUDA(h, cudaGetLastError());
  }
  return V1G_OK;
}

static bool state_complete(const V1GState* s) {
  return s && s->z_buf && s->v && s->r && s->asc && s->psc_rise && s->psc;
}

extern "C" int v1g_step_fwd(V1GHandle* h, int32_t batch, const V1GState* in,
                            const float* rec_inputs, V1GState* out, float* z_out, void* stream) {
  if (!h) return V1G_EINVAL;
  if (!h->params_set) return v1g_fail(h, V1G_ESTATE, "neuron parameters not set");
  if (batch <= 0 || !state_complete(in) || !state_complete(out) || !rec_inputs)
    return v1g_fail(h, V1G_EINVAL, "v1g_step_fwd: bad argument");
  const int64_t total = (int64_t)batch * h->cfg.n_neurons;
  step_fwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      make_consts(h), batch, h->decay, h->cf, h->asc_decay, h->asc_amps, h->tref, *in, rec_inputs,
      *out, z_out);
  v1g_count_launches(1);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

extern "C" int v1g_step_bwd(V1GHandle* h, int32_t batch, const V1GState* g_out, const float* g_z,
                            const float* g_v_out, const float* new_v, const int8_t* new_r,
                            V1GState* g_in, float* g_rec_inputs, void* stream) {
  if (!h) return V1G_EINVAL;
  if (!h->params_set) return v1g_fail(h, V1G_ESTATE, "neuron parameters not set");
  if (batch <= 0 || !g_out || !g_in || !new_v || !new_r || !g_rec_inputs || !g_in->v ||
      !g_in->asc || !g_in->psc || !g_in->psc_rise)
    return v1g_fail(h, V1G_EINVAL, "v1g_step_bwd: bad argument");
  const int64_t total = (int64_t)batch * h->cfg.n_neurons;
  step_bwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      make_consts(h), batch, h->decay, h->cf, h->asc_decay, *g_out, g_z, g_v_out, new_v, new_r,
      *g_in, g_rec_inputs);
  v1g_count_launches(1);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}
