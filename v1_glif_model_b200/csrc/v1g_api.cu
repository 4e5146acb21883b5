// Handle life cycle, connectivity layout build, parameter upload.
#include <stdarg.h>
#include <string.h>

#include <algorithm>

#include "v1g_internal.h"

int v1g_fail(const V1GHandle* h, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (h) h->err = buf;
  return code;
}

static std::string g_create_err;

#include <atomic>
static std::atomic<long long> g_launches{0};
void v1g_count_launches(int n) { g_launches += n; }
void v1g_set_global_error(const char* msg) { g_create_err = msg ? msg : ""; }
extern "C" long long v1g_launch_count(void) { return g_launches.load(); }

extern "C" const char* v1g_version(void) { return "v1g-sm100a-1"; }

extern "C" const char* v1g_last_error(const V1GHandle* h) {
  return h ? h->err.c_str() : g_create_err.c_str();
}

extern "C" int v1g_create(const V1GConfig* cfg, V1GHandle** out) {
  if (!cfg || !out) {
    g_create_err = "v1g_create: null argument";
    return V1G_EINVAL;
  }
  *out = nullptr;
  if (cfg->n_neurons <= 0 || cfg->n_receptors <= 0 || cfg->n_receptors > V1G_MAX_RECEPTORS ||
      cfg->n_syn_types <= 0 || cfg->n_syn_types > 256 || cfg->max_delay <= 0 ||
      cfg->max_delay > V1G_MAX_DELAY || cfg->n_lgn <= 0 || cfg->n_bkg <= 0 ||
      cfg->n_lgn >= (1 << 24)) {
    g_create_err =
        "v1g_create: sizes out of range (need N>0, 0<R<=8, 0<S<=256, 0<D<=8, 0<n_lgn<2^24, "
        "n_bkg>0)";
    return V1G_EINVAL;
  }
  if (!(cfg->pseudo_width > 0.f)) {
    g_create_err = "v1g_create: pseudo_width must be > 0";
    return V1G_EINVAL;
  }
  V1GHandle* h = new V1GHandle();
  h->cfg = *cfg;
  cudaError_t e = cudaGetDevice(&h->device);
  if (e != cudaSuccess) {
    g_create_err = std::string("v1g_create: no CUDA device: ") + cudaGetErrorString(e);
    delete h;
    return V1G_ECUDA;
  }
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, h->device);
  if (e != cudaSuccess) {
    g_create_err = std::string("v1g_create: ") + cudaGetErrorString(e);
    delete h;
    return V1G_ECUDA;
  }
  h->n_sms = prop.multiProcessorCount;
  h->smem_optin = (int)prop.sharedMemPerBlockOptin;
  // straight_through_dampen (models.py:284-296): d = clip(dampening, 0, 1); forward uses
  // x*(1-d) + x*d, backward scales by (1-d).  The recurrent path is called with 1 - rd.
  float d = fminf(fmaxf(cfg->voltage_gradient_dampening, 0.f), 1.f);
  h->vd_keep = 1.f - d;
  h->vd_drop = d;
  float dr = fminf(fmaxf(1.f - cfg->recurrent_dampening, 0.f), 1.f);
  h->rec_grad_factor = 1.f - dr;
  int rc = V1G_OK;
  auto chk = [&](cudaError_t ce) {
    if (ce != cudaSuccess && rc == V1G_OK) {
      g_create_err = std::string("v1g_create: ") + cudaGetErrorString(ce);
      rc = V1G_ECUDA;
    }
  };
  chk(cudaMalloc((void**)&h->d_count, 4 * sizeof(int32_t)));
  chk(cudaMallocHost((void**)&h->h_count, 4 * sizeof(int32_t)));
  chk(cudaMalloc((void**)&h->barrier, 8 * 16 * sizeof(unsigned long long)));
  chk(cudaMalloc((void**)&h->dev_status, 4 * sizeof(int32_t)));
  chk(cudaMalloc((void**)&h->counters, sizeof(V1GCounters)));
  for (int i = 0; i < 4; ++i) chk(cudaEventCreate(&h->ev[i]));
  if (rc == V1G_OK) {
    chk(cudaMemset(h->dev_status, 0, 4 * sizeof(int32_t)));
    chk(cudaMemset(h->counters, 0, sizeof(V1GCounters)));
  }
  if (rc != V1G_OK) {
    v1g_destroy(h);
    return rc;
  }
  *out = h;
  return V1G_OK;
}

static void free_source(V1GSource& s) {
  cudaFree(s.rowptr);
  cudaFree(s.post);
  cudaFree(s.w);
  cudaFree(s.sid);
  cudaFree(s.perm);
  cudaFree(s.syn8);
  cudaFree(s.pos_int);
  cudaFree(s.in_ptr);
  cudaFree(s.in_pre);
  cudaFree(s.in_sid);
  cudaFree(s.in_perm);
  cudaFree(s.w_in);
  cudaFree(s.w_ref);
  for (int p = 0; p < 2; ++p) {
    cudaFree(s.pair_ptr[p]);
    cudaFree(s.pair_rec[p]);
    cudaFree(s.pair_j[p]);
  }
  s = V1GSource();
}

extern "C" int v1g_destroy(V1GHandle* h) {
  if (!h) return V1G_OK;
  for (int i = 0; i < V1G_NSRC; ++i) {
    free_source(h->src[i]);
    cudaFree(h->dw_csr[i]);
  }
  cudaFree(h->decay);
  cudaFree(h->cf);
  cudaFree(h->asc_decay);
  cudaFree(h->asc_amps);
  cudaFree(h->tref);
  cudaFree(h->basis);
  cudaFree(h->seg_counts);
  cudaFree(h->coords);
  cudaFree(h->d_count);
  if (h->h_count) cudaFreeHost(h->h_count);
  cudaFree(h->lgn_entries);
  cudaFree(h->lgn_ent4);
  cudaFree(h->tape_stats);
  cudaFree(h->fwd_slice);
  cudaFree(h->rate_scratch);
  cudaFree(h->reg_scratch);
  cudaFree(h->sync_scratch);
  cudaFree(h->osi_scratch);
  cudaFree(h->lgn_offsets);
  cudaFree(h->ring);
  cudaFree(h->state_ws);
  cudaFree(h->barrier);
  cudaFree(h->dev_status);
  cudaFree(h->counters);
  cudaFree(h->tape_v);
  cudaFree(h->tape_hist0);
  cudaFree(h->tape_counts_buf);
  cudaFree(h->dy_ring);
  cudaFree(h->loss_scratch);
  cudaFree(h->stage_x);
  cudaFree(h->stage_counts);
  cudaFree(h->stage_z);
  cudaFree(h->stage_v);
  cudaFree(h->stage_bits);
  cudaFree(h->pipe_state);
  if (h->pipe_in) cudaStreamDestroy(h->pipe_in);
  if (h->pipe_out) cudaStreamDestroy(h->pipe_out);
  for (int i = 0; i < 6; ++i)
    if (h->pipe_ev[i]) cudaEventDestroy(h->pipe_ev[i]);
  cudaFree(h->phase_ns);
  for (int i = 0; i < 4; ++i)
    if (h->ev[i]) cudaEventDestroy(h->ev[i]);
  delete h;
  return V1G_OK;
}

template <typename T>
static int upload(V1GHandle* h, T** dst, const T* src, size_t n) {
  if (*dst) {
    cudaFree(*dst);
    *dst = nullptr;
  }
  V1G_CUDA(h, cudaMalloc((void**)dst, std::max<size_t>(n, 1) * sizeof(T)));
  if (n) V1G_CUDA(h, cudaMemcpy(*dst, src, n * sizeof(T), cudaMemcpyHostToDevice));
  return V1G_OK;
}

extern "C" int v1g_set_connectivity(V1GHandle* h, int source, int64_t nnz,
                                    const int64_t* indices_host, const uint8_t* syn_ids_host,
                                    int64_t n_source_cols) {
  if (!h) return V1G_EINVAL;
  if (source < 0 || source >= V1G_NSRC) return v1g_fail(h, V1G_EINVAL, "unknown source %d", source);
  if (nnz < 0 || nnz > 0x7fffffffLL)
    return v1g_fail(h, V1G_EINVAL, "nnz=%lld not representable", (long long)nnz);
  if (nnz > 0 && (!indices_host || !syn_ids_host))
    return v1g_fail(h, V1G_EINVAL, "null connectivity arrays");
  const int N = h->cfg.n_neurons;
  const int D = (source == V1G_SRC_REC) ? h->cfg.max_delay : 1;
  const int64_t n_src = (source == V1G_SRC_REC) ? N : (source == V1G_SRC_LGN ? h->cfg.n_lgn : h->cfg.n_bkg);
  // models.py:300-302
  if (n_source_cols <= 0)
    return v1g_fail(h, V1G_EINVAL, "`n_source_neurons` must be > 0, got %lld.", (long long)n_source_cols);
  if (n_source_cols != n_src * D)
    return v1g_fail(h, V1G_EINVAL, "source %d: n_source_cols=%lld but the handle expects %lld",
                    source, (long long)n_source_cols, (long long)(n_src * D));
  const int S = h->cfg.n_syn_types;
  for (int64_t i = 0; i < nnz; ++i) {
    const int64_t post = indices_host[2 * i], pre = indices_host[2 * i + 1];
    if (pre < 0 || pre >= n_source_cols)  // models.py:308-314
      return v1g_fail(h, V1G_EINVAL,
                      "Presynaptic index %lld is out of bounds for `n_source_neurons=%lld`.",
                      (long long)pre, (long long)n_source_cols);
    if (post < 0 || post >= N)
      return v1g_fail(h, V1G_EINVAL, "Postsynaptic index %lld is out of bounds for n_neurons=%d.",
                      (long long)post, N);
    if (syn_ids_host[i] >= S)
      return v1g_fail(h, V1G_EINVAL, "syn_id %d of synapse %lld is out of bounds for %d types.",
                      (int)syn_ids_host[i], (long long)i, S);
  }
  V1GSource& s = h->src[source];
  free_source(s);
  cudaFree(h->dw_csr[source]);
  h->dw_csr[source] = nullptr;
  s.nnz = nnz;
  s.n_cols = n_source_cols;
  s.n_src = (int)n_src;
  s.delays = D;

  // Stable counting sort by presynaptic column: the reference's table (models.py:317-341).
  s.row_splits_host.assign((size_t)n_source_cols + 1, 0);
  for (int64_t i = 0; i < nnz; ++i) s.row_splits_host[(size_t)indices_host[2 * i + 1] + 1]++;
  for (int64_t c = 0; c < n_source_cols; ++c) s.row_splits_host[c + 1] += s.row_splits_host[c];
  s.order_host.resize((size_t)nnz);
  {
    std::vector<int64_t> wp(s.row_splits_host.begin(), s.row_splits_host.end() - 1);
    for (int64_t i = 0; i < nnz; ++i) s.order_host[(size_t)wp[(size_t)indices_host[2 * i + 1]]++] = (int32_t)i;
  }
  // Device CSR with the delay buckets of a source neuron made contiguous.
  std::vector<int32_t> rowptr((size_t)n_source_cols + 1), post((size_t)nnz), perm((size_t)nnz);
  std::vector<uint8_t> sid((size_t)nnz);
  std::vector<uint2> syn8;
  const bool want_syn8 = source != V1G_SRC_BKG && S <= 128 && D <= 8 && N < (1 << 22);
  if (want_syn8) syn8.resize((size_t)nnz);
  int64_t pos = 0;
  for (int64_t src = 0; src < n_src; ++src) {
    for (int d = 0; d < D; ++d) {
      const int64_t c = src + n_src * d;
      rowptr[(size_t)(src * D + d)] = (int32_t)pos;
      for (int64_t q = s.row_splits_host[c]; q < s.row_splits_host[c + 1]; ++q) {
        const int32_t i = s.order_host[(size_t)q];
        post[(size_t)pos] = (int32_t)indices_host[2 * (int64_t)i];
        sid[(size_t)pos] = syn_ids_host[i];
        if (want_syn8)
          syn8[(size_t)pos] = make_uint2((uint32_t)indices_host[2 * (int64_t)i] |
                                             ((uint32_t)syn_ids_host[i] << 22) | ((uint32_t)d << 29), 0u);
        perm[(size_t)pos] = i;
        ++pos;
      }
    }
  }
  rowptr[(size_t)n_source_cols] = (int32_t)pos;
  // Post-major gather table.  The reference's arrays are already grouped by post; otherwise a
  // stable sort by post supplies the grouping and in_perm maps back.
  bool sorted = true;
  for (int64_t i = 1; i < nnz && sorted; ++i) sorted = indices_host[2 * i] >= indices_host[2 * (i - 1)];
  std::vector<int32_t> in_ptr((size_t)N + 1, 0), in_pre((size_t)nnz), in_perm;
  std::vector<uint8_t> in_sid((size_t)nnz);
  for (int64_t i = 0; i < nnz; ++i) in_ptr[(size_t)indices_host[2 * i] + 1]++;
  for (int n = 0; n < N; ++n) in_ptr[n + 1] += in_ptr[n];
  if (sorted) {
    for (int64_t i = 0; i < nnz; ++i) {
      in_pre[(size_t)i] = (int32_t)indices_host[2 * i + 1];
      in_sid[(size_t)i] = syn_ids_host[i];
    }
  } else {
    in_perm.resize((size_t)nnz);
    std::vector<int32_t> wp(in_ptr.begin(), in_ptr.end() - 1);
    for (int64_t i = 0; i < nnz; ++i) {
      const int32_t p = wp[(size_t)indices_host[2 * i]]++;
      in_perm[(size_t)p] = (int32_t)i;
      in_pre[(size_t)p] = (int32_t)indices_host[2 * i + 1];
      in_sid[(size_t)p] = syn_ids_host[i];
    }
  }
  s.post_sorted = sorted;
  s.in_ptr_host = in_ptr;
  if (source == V1G_SRC_REC && want_syn8) {
    s.rowptr_host = rowptr;
    s.syn8x_host.resize((size_t)nnz);
    for (int64_t i = 0; i < nnz; ++i) s.syn8x_host[(size_t)i] = syn8[(size_t)i].x;
  }
  int rc;
  if ((rc = upload(h, &s.rowptr, rowptr.data(), rowptr.size()))) return rc;
  if ((rc = upload(h, &s.post, post.data(), post.size()))) return rc;
  if ((rc = upload(h, &s.sid, sid.data(), sid.size()))) return rc;
  if ((rc = upload(h, &s.perm, perm.data(), perm.size()))) return rc;
  if (want_syn8 && (rc = upload(h, &s.syn8, syn8.data(), syn8.size()))) return rc;
  if ((rc = upload(h, &s.in_ptr, in_ptr.data(), in_ptr.size()))) return rc;
  if ((rc = upload(h, &s.in_pre, in_pre.data(), in_pre.size()))) return rc;
  if ((rc = upload(h, &s.in_sid, in_sid.data(), in_sid.size()))) return rc;
  if (!sorted) {
    if ((rc = upload(h, &s.in_perm, in_perm.data(), in_perm.size()))) return rc;
    V1G_CUDA(h, cudaMalloc((void**)&s.w_in, std::max<size_t>((size_t)nnz, 1) * sizeof(float)));
    V1G_CUDA(h, cudaMemset(s.w_in, 0, std::max<size_t>((size_t)nnz, 1) * sizeof(float)));
  }
  V1G_CUDA(h, cudaMalloc((void**)&s.w, std::max<size_t>((size_t)nnz, 1) * sizeof(float)));
  V1G_CUDA(h, cudaMalloc((void**)&s.w_ref, std::max<size_t>((size_t)nnz, 1) * sizeof(float)));
  V1G_CUDA(h, cudaMemset(s.w, 0, std::max<size_t>((size_t)nnz, 1) * sizeof(float)));
  V1G_CUDA(h, cudaMemset(s.w_ref, 0, std::max<size_t>((size_t)nnz, 1) * sizeof(float)));
  h->tape_valid = false;
  h->fwd_slice_host.clear();
  return V1G_OK;
}

extern "C" int v1g_build_pre_ind_table(int64_t nnz, const int64_t* indices_host,
                                       int64_t n_source_cols, int64_t* order_host,
                                       int64_t* row_splits_host) {
  if (n_source_cols <= 0 || nnz < 0 || (nnz > 0 && !indices_host) || !order_host || !row_splits_host)
    return V1G_EINVAL;
  for (int64_t i = 0; i < nnz; ++i) {
    const int64_t pre = indices_host[2 * i + 1];
    if (pre < 0 || pre >= n_source_cols) return V1G_EINVAL;
  }
  for (int64_t c = 0; c <= n_source_cols; ++c) row_splits_host[c] = 0;
  for (int64_t i = 0; i < nnz; ++i) row_splits_host[indices_host[2 * i + 1] + 1]++;
  for (int64_t c = 0; c < n_source_cols; ++c) row_splits_host[c + 1] += row_splits_host[c];
  std::vector<int64_t> wp(row_splits_host, row_splits_host + n_source_cols);
  for (int64_t i = 0; i < nnz; ++i) order_host[wp[(size_t)indices_host[2 * i + 1]]++] = i;
  return V1G_OK;
}

extern "C" int v1g_get_pre_ind_table(V1GHandle* h, int source, int64_t* order_host,
                                     int64_t* row_splits_host) {
  if (!h) return V1G_EINVAL;
  if (source < 0 || source >= V1G_NSRC) return v1g_fail(h, V1G_EINVAL, "unknown source %d", source);
  const V1GSource& s = h->src[source];
  if (s.row_splits_host.empty()) return v1g_fail(h, V1G_ESTATE, "connectivity of source %d not set", source);
  if (order_host)
    for (int64_t i = 0; i < s.nnz; ++i) order_host[i] = s.order_host[(size_t)i];
  if (row_splits_host)
    memcpy(row_splits_host, s.row_splits_host.data(), s.row_splits_host.size() * sizeof(int64_t));
  return V1G_OK;
}

extern "C" int v1g_set_neuron_params(V1GHandle* h, const float* decay, const float* current_factor,
                                     const float* asc_decay, const float* asc_amps,
                                     const int32_t* t_ref_steps, const float* syn_decay,
                                     const float* psc_initial, const float* basis) {
  if (!h) return V1G_EINVAL;
  if (!decay || !current_factor || !asc_decay || !asc_amps || !t_ref_steps || !syn_decay ||
      !psc_initial || !basis)
    return v1g_fail(h, V1G_EINVAL, "v1g_set_neuron_params: null argument");
  const int N = h->cfg.n_neurons, R = h->cfg.n_receptors, S = h->cfg.n_syn_types;
  for (int n = 0; n < N; ++n)
    if (t_ref_steps[n] < 1 || t_ref_steps[n] > 127)
      return v1g_fail(h, V1G_EINVAL,
                      "t_ref_steps[%d]=%d outside 1..127 (the int8 refractory state of "
                      "models.py:578-583)", n, t_ref_steps[n]);
  int rc;
  if ((rc = upload(h, &h->decay, decay, (size_t)N))) return rc;
  if ((rc = upload(h, &h->cf, current_factor, (size_t)N))) return rc;
  if ((rc = upload(h, &h->asc_decay, asc_decay, (size_t)N * 2))) return rc;
  if ((rc = upload(h, &h->asc_amps, asc_amps, (size_t)N * 2))) return rc;
  if ((rc = upload(h, &h->tref, t_ref_steps, (size_t)N))) return rc;
  if ((rc = upload(h, &h->basis, basis, (size_t)S * R))) return rc;
  for (int r = 0; r < R; ++r) {
    h->syn_decay[r] = syn_decay[r];
    h->psc_initial[r] = psc_initial[r];
  }
  h->params_set = true;
  return V1G_OK;
}

__global__ void sign_mask_kernel(const float* __restrict__ w, uint8_t* __restrict__ pos, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) pos[i] = w[i] >= 0.f ? 1 : 0;
}

// dst[perm[i]] = src[i]  (perm == nullptr: plain copy)
__global__ void unpermute_kernel(const float* __restrict__ src, const int32_t* __restrict__ perm,
                                 float* __restrict__ dst, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[perm ? perm[i] : i] = src[i];
}

__global__ void permute_weights_kernel(const float* __restrict__ w_ref,
                                       const int32_t* __restrict__ perm, float* __restrict__ w,
                                       int64_t nnz) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < nnz; i += stride) w[i] = w_ref[perm[i]];
}

// weights into the gather-ordered record copies of the paired backward ring
__global__ void pair_weights_kernel(const float* __restrict__ w, const int32_t* __restrict__ pos,
                                    uint2* __restrict__ rec, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) rec[i].y = __float_as_uint(w[pos[i]]);
}

static void refresh_pair_weights(V1GSource& s, cudaStream_t st) {
  if (!s.pair_built) return;
  for (int p = 0; p < 2; ++p) {
    if (s.pair_len[p] == 0) continue;
    const int blocks = (int)std::min<int64_t>((s.pair_len[p] + 255) / 256, 148 * 16);
    pair_weights_kernel<<<blocks, 256, 0, st>>>(s.w, s.pair_j[p], s.pair_rec[p], s.pair_len[p]);
    v1g_count_launches(1);
  }
}

int v1g_build_pair_tables(V1GHandle* h, cudaStream_t st) {
  V1GSource& s = h->src[V1G_SRC_REC];
  if (s.pair_built) return V1G_OK;
  if (s.rowptr_host.empty() || !s.syn8)
    return v1g_fail(h, V1G_ESTATE, "the paired backward ring needs the packed records of the recurrent source");
  const int D = s.delays;
  const int64_t n_src = s.n_src;
  for (int p = 0; p < 2; ++p) {
    std::vector<int32_t> ptr((size_t)n_src + 1), pos;
    std::vector<uint2> rec;
    pos.reserve((size_t)s.nnz);
    for (int64_t n = 0; n < n_src; ++n) {
      ptr[(size_t)n] = (int32_t)pos.size();
      const int32_t* rp = s.rowptr_host.data() + n * D;
      for (int j = rp[0]; j < rp[1]; ++j) pos.push_back(j);            // delay 1
      for (int d = 1 + p; d < D; d += 2)                                // delays 2 + p, 4 + p, ...
        for (int j = rp[d]; j < rp[d + 1]; ++j) pos.push_back(j);
    }
    ptr[(size_t)n_src] = (int32_t)pos.size();
    rec.resize(pos.size());
    for (size_t i = 0; i < pos.size(); ++i) rec[i] = make_uint2(s.syn8x_host[(size_t)pos[i]], 0u);
    s.pair_len[p] = (int64_t)pos.size();
    int rc;
    if ((rc = upload(h, &s.pair_ptr[p], ptr.data(), ptr.size()))) return rc;
    if ((rc = upload(h, &s.pair_rec[p], rec.data(), rec.size()))) return rc;
    if ((rc = upload(h, &s.pair_j[p], pos.data(), pos.size()))) return rc;
  }
  s.pair_built = true;
  refresh_pair_weights(s, st);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

// copy the weights into the packed synapse records of the backward gather
__global__ void syn8_weights_kernel(const float* __restrict__ w, uint2* __restrict__ syn8, int64_t nnz) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < nnz; i += stride) syn8[i].y = __float_as_uint(w[i]);
}

extern "C" int v1g_set_weights(V1GHandle* h, int source, const float* w, void* stream) {
  if (!h) return V1G_EINVAL;
  if (source < 0 || source >= V1G_NSRC) return v1g_fail(h, V1G_EINVAL, "unknown source %d", source);
  V1GSource& s = h->src[source];
  if (!s.rowptr) return v1g_fail(h, V1G_ESTATE, "connectivity of source %d not set", source);
  if (s.nnz == 0) return V1G_OK;
  if (!w) return v1g_fail(h, V1G_EINVAL, "v1g_set_weights: null weights");
  cudaStream_t st = (cudaStream_t)stream;
  V1G_CUDA(h, cudaMemcpyAsync(s.w_ref, w, (size_t)s.nnz * sizeof(float), cudaMemcpyDeviceToDevice, st));
  const int threads = 256;
  const int blocks = (int)std::min<int64_t>((s.nnz + threads - 1) / threads, 148 * 16);
  permute_weights_kernel<<<blocks, threads, 0, st>>>(s.w_ref, s.perm, s.w, s.nnz);
  v1g_count_launches(1);
  if (s.in_perm) {
    permute_weights_kernel<<<blocks, threads, 0, st>>>(s.w_ref, s.in_perm, s.w_in, s.nnz);
    v1g_count_launches(1);
  }
  if (s.syn8) {
    syn8_weights_kernel<<<blocks, threads, 0, st>>>(s.w, s.syn8, s.nnz);
    v1g_count_launches(1);
  }
  refresh_pair_weights(s, st);
  if (!s.pos_set) {
    // the sign of each weight at construction is what SignedConstraint preserves (models.py:647-666)
    if (!s.pos_int) V1G_CUDA(h, cudaMalloc((void**)&s.pos_int, (size_t)s.nnz));
    const float* w_int = (source == V1G_SRC_BKG) ? s.gather_w() : s.w;
    sign_mask_kernel<<<blocks, threads, 0, st>>>(w_int, s.pos_int, s.nnz);
    v1g_count_launches(1);
    s.pos_set = true;
  }
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

extern "C" int v1g_train_layout(V1GHandle* h, int64_t* sizes3) {
  if (!h || !sizes3) return V1G_EINVAL;
  for (int s = 0; s < V1G_NSRC; ++s) sizes3[s] = h->src[s].nnz;
  return V1G_OK;
}

extern "C" int v1g_get_weights(V1GHandle* h, int source, float* w_out, void* stream) {
  if (!h || !w_out) return V1G_EINVAL;
  if (source < 0 || source >= V1G_NSRC) return v1g_fail(h, V1G_EINVAL, "unknown source %d", source);
  V1GSource& s = h->src[source];
  if (!s.rowptr) return v1g_fail(h, V1G_ESTATE, "connectivity of source %d not set", source);
  if (s.nnz == 0) return V1G_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int blocks = (int)std::min<int64_t>((s.nnz + 255) / 256, 148 * 16);
  if (source == V1G_SRC_BKG)
    unpermute_kernel<<<blocks, 256, 0, st>>>(s.gather_w(), s.in_perm, w_out, s.nnz);
  else
    unpermute_kernel<<<blocks, 256, 0, st>>>(s.w, s.perm, w_out, s.nnz);
  v1g_count_launches(1);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

extern "C" int v1g_expadam_update_internal(V1GHandle* h, const float* grads_flat, float* m_flat,
                                           float* v_flat, int32_t train_mask, float lr, float beta1,
                                           float beta2, float eps, int64_t step, float grad_scale,
                                           void* stream) {
  if (!h || !grads_flat || !m_flat || !v_flat) return V1G_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  int64_t off = 0;
  for (int src = 0; src < V1G_NSRC; ++src) {
    V1GSource& s = h->src[src];
    if (((train_mask >> src) & 1) && s.nnz > 0) {
      if (!s.pos_set) return v1g_fail(h, V1G_ESTATE, "weights of source %d not set", src);
      float* w_int = (src == V1G_SRC_BKG) ? s.gather_w_mut() : s.w;
      int rc = v1g_expadam_update(w_int, grads_flat + off, m_flat + off, v_flat + off, s.pos_int, s.nnz,
                                  lr, beta1, beta2, eps, step, grad_scale, stream);
      if (rc) return v1g_fail(h, rc, "v1g_expadam_update failed for source %d", src);
      if (s.syn8) {
        const int blocks = (int)std::min<int64_t>((s.nnz + 255) / 256, 148 * 16);
        syn8_weights_kernel<<<blocks, 256, 0, st>>>(s.w, s.syn8, s.nnz);
        v1g_count_launches(1);
      }
      refresh_pair_weights(s, st);
      if (src == V1G_SRC_BKG) {
        // the background weights also exist in caller's and CSR order (operator-level entry points)
        const int blocks = (int)std::min<int64_t>((s.nnz + 255) / 256, 148 * 16);
        if (s.in_perm) {
          unpermute_kernel<<<blocks, 256, 0, st>>>(s.w_in, s.in_perm, s.w_ref, s.nnz);
          v1g_count_launches(1);
        }
        permute_weights_kernel<<<blocks, 256, 0, st>>>(s.w_ref, s.perm, s.w, s.nnz);
        v1g_count_launches(1);
      }
    }
    off += s.nnz;
  }
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

extern "C" int v1g_synchronize(V1GHandle* h, void* stream) {
  if (!h) return V1G_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  V1G_CUDA(h, cudaMemcpyAsync(h->h_count + 2, h->dev_status, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  V1G_CUDA(h, cudaStreamSynchronize(st));
  const int32_t status = h->h_count[2];
  if (status != V1G_DEV_OK) {
    V1G_CUDA(h, cudaMemsetAsync(h->dev_status, 0, sizeof(int32_t), st));
    h->tape_valid = false;
    return v1g_fail(h, V1G_ETIMEOUT,
                    "device status %d: a bounded grid-barrier wait gave up; results are invalid",
                    status);
  }
  return V1G_OK;
}

extern "C" int v1g_get_counters(V1GHandle* h, V1GCounters* out_host) {
  if (!h || !out_host) return V1G_EINVAL;
  V1G_CUDA(h, cudaMemcpy(out_host, h->counters, sizeof(V1GCounters), cudaMemcpyDeviceToHost));
  return V1G_OK;
}

extern "C" int v1g_last_kernel_ms(V1GHandle* h, int which, float* ms) {
  if (!h || !ms || which < 0 || which > 1) return V1G_EINVAL;
  if (!h->ev_valid[which]) return v1g_fail(h, V1G_ESTATE, "no rollout kernel of that kind has run");
  V1G_CUDA(h, cudaEventSynchronize(h->ev[2 * which + 1]));
  V1G_CUDA(h, cudaEventElapsedTime(ms, h->ev[2 * which], h->ev[2 * which + 1]));
  return V1G_OK;
}

extern "C" int v1g_get_phase_times(V1GHandle* h, unsigned long long* out_host, int32_t max_blocks,
                                   int32_t* n_blocks) {
  if (!h || !out_host || !n_blocks) return V1G_EINVAL;
  const int n = std::min<int>(h->phase_grid, max_blocks);
  *n_blocks = n;
  if (n > 0 && h->phase_ns)
    V1G_CUDA(h, cudaMemcpy(out_host, h->phase_ns, sizeof(unsigned long long) * 4 * n, cudaMemcpyDeviceToHost));
  return V1G_OK;
}

extern "C" int v1g_set_option(V1GHandle* h, const char* name, long long value) {
  if (!h || !name) return V1G_EINVAL;
  if (!strcmp(name, "rollout_chunk")) {
    if (value < 0 || (value % 32) != 0)
      return v1g_fail(h, V1G_EINVAL, "rollout_chunk must be 0 or a multiple of 32");
    h->opt_chunk = (int)value;
    h->fwd_slice_host.clear();  // balanced slices belong to one slicing of the neurons
  } else if (!strcmp(name, "state_in_global")) {
    h->opt_force_global = value != 0;
  } else if (!strcmp(name, "force_smem_kernel")) {
    h->opt_force_smem_kernel = value != 0;
  } else if (!strcmp(name, "no_meta")) {
    h->opt_no_meta = value != 0;
  } else if (!strcmp(name, "no_q_pack")) {
    h->opt_no_q_pack = value != 0;
  } else if (!strcmp(name, "pair_rows")) {
    h->opt_pair_rows = value != 0;
  } else if (!strcmp(name, "l2_window")) {
    h->opt_l2_window = value != 0;
  } else if (!strcmp(name, "csr_evict_first")) {
    h->opt_csr_evict_first = value != 0;
  } else if (!strcmp(name, "phase_timers")) {
    h->opt_phase_timers = value != 0;
  } else if (!strcmp(name, "spin_limit")) {
    if (value < 1) return v1g_fail(h, V1G_EINVAL, "spin_limit must be >= 1");
    h->opt_spin_limit = value;
  } else {
    return v1g_fail(h, V1G_EINVAL, "unknown option '%s'", name);
  }
  return V1G_OK;
}
