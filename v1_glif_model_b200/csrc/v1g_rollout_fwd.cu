// Fused forward rollout: T steps of V1Column.call (models.py:1059-1135) in ONE persistent
// cooperative kernel, one thread block per SM.
//
// Each block owns a contiguous slice of neurons for all batch rows and keeps their state
// (v, r, asc, psc_rise, psc, the last D spike bits) in shared memory for the whole rollout.
// Synaptic currents travel through a ring of K = D+1 future-step accumulators in global memory
// (L2-resident): a spike emitted at step t by neuron n adds w*basis[sid,:] of every outgoing
// synapse with delay d into slot (t+d) mod K, so the block that computed the spike scatters it
// immediately ("scatter on emit") and one grid barrier per step is enough.  LGN events of step
// t+1 (compacted ahead of time into a time-major list) are scattered during step t; background
// input is gathered per post-synaptic neuron from the step's Poisson counts (no atomics).
//
// Time step t of a block:
//   dense   : read+clear ring slot t%K, gather background, PSC/ASC/membrane/refractory/threshold
//             update, write v and z, push own spikes to a shared-memory list
//   scatter : one warp per listed spike walks the D contiguous delay buckets of the neuron's CSR
//             row; warps also share the LGN events of step t+1
//   barrier : bounded spin on a monotonically increasing counter
#include <algorithm>

#include "v1g_rollout_fwd.cuh"
#include "v1g_rng.cuh"

namespace {

constexpr int NT = 768;

// bit d-1 of hist0[b*N+n] = neuron n of batch row b spiked d steps before the rollout starts
// LGN event list with the bounds of each event's synapse row, so that the rollout kernels need no
// dependent row-pointer load per event
__global__ void lgn_resolve_kernel(const uint32_t* __restrict__ entries, int64_t n,
                                   const int32_t* __restrict__ rowptr, uint4* __restrict__ out) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const uint32_t ent = entries[i];
    const uint32_t u = ent & 0xffffffu;
    out[i] = make_uint4(ent, (uint32_t)rowptr[u], (uint32_t)rowptr[u + 1], 0u);
  }
}

__global__ void __launch_bounds__(256) hist0_kernel(const float* __restrict__ z_buf, int B, int D, int N,
                                                    uint8_t* __restrict__ hist0) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)B * N) return;
  const int b = (int)(i / N), n = (int)(i - (int64_t)b * N);
  unsigned hbits = 0;
  for (int d = 0; d < D; ++d)
    if (z_buf[((int64_t)b * D + d) * N + n] > 0.f) hbits |= 1u << d;
  hist0[i] = (uint8_t)hbits;
}

template <int R_>
__global__ void __launch_bounds__(NT, 1) rollout_fwd_kernel(const FwdArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int NW = NT / 32;
  const int B = a.B, D = a.D, K = a.K, N = a.N, Np = a.Np, chunkP = a.chunkP;
  const int n0 = blockIdx.x * a.chunk;
  const int cn = min(a.chunk, N - n0);
  const int items = B * cn;

  // ---- carve shared memory ----
  unsigned char* sp_ = smem_raw;
  auto take = [&](size_t bytes) {
    unsigned char* p = sp_;
    sp_ += (bytes + 15) & ~(size_t)15;
    return p;
  };
  float* c_decay = (float*)take(sizeof(float) * chunkP);
  float* c_cf = (float*)take(sizeof(float) * chunkP);
  float* c_ad0 = (float*)take(sizeof(float) * chunkP);
  float* c_ad1 = (float*)take(sizeof(float) * chunkP);
  float* c_am0 = (float*)take(sizeof(float) * chunkP);
  float* c_am1 = (float*)take(sizeof(float) * chunkP);
  int* c_tref = (int*)take(sizeof(int) * chunkP);
  int* c_bkptr = (int*)take(sizeof(int) * (chunkP + 1));
  float* basis_s = (float*)take(sizeof(float) * a.S * R_);
  uint32_t* spk_list = (uint32_t*)take(sizeof(uint32_t) * B * chunkP);
  int* s_cnt = (int*)take(sizeof(int) * 2 * B * a.n_bkg);
  int* s_misc = (int*)take(sizeof(int) * 4);  // [1] abort flag, [2],[3] spike counts (double buffer)
  int* bk_pre_s = nullptr;
  float* bk_w_s = nullptr;
  uint8_t* bk_sid_s = nullptr;
  if (a.bkg_in_smem) {
    bk_pre_s = (int*)take(sizeof(int) * a.bkg_cap);
    bk_w_s = (float*)take(sizeof(float) * a.bkg_cap);
    bk_sid_s = (uint8_t*)take(a.bkg_cap);
  }
  float *S_v, *S_a0, *S_a1, *S_p, *S_pr;
  uint8_t *S_r, *S_hist;
  {
    const size_t plane = (size_t)B * chunkP;
    float* base;
    if (a.state_in_smem) {
      base = (float*)take(sizeof(float) * plane * (3 + 2 * R_) + 2 * plane);
    } else {
      const size_t slab = plane * (3 + 2 * R_) + (2 * plane + 3) / 4;
      base = a.state_ws + (size_t)blockIdx.x * slab;
    }
    S_v = base;
    S_a0 = S_v + plane;
    S_a1 = S_a0 + plane;
    S_p = S_a1 + plane;
    S_pr = S_p + plane * R_;
    S_r = (uint8_t*)(S_pr + plane * R_);
    S_hist = S_r + plane;
  }

  // ---- load constants, background table, state ----
  for (int k = tid; k < cn; k += NT) {
    const int n = n0 + k;
    c_decay[k] = a.decay[n];
    c_cf[k] = a.cf[n];
    c_ad0[k] = a.asc_decay[2 * n];
    c_ad1[k] = a.asc_decay[2 * n + 1];
    c_am0[k] = a.asc_amps[2 * n];
    c_am1[k] = a.asc_amps[2 * n + 1];
    c_tref[k] = a.tref[n];
  }
  const int bk_base = a.bkg_inptr[n0];
  for (int k = tid; k <= cn; k += NT) c_bkptr[k] = a.bkg_inptr[n0 + k] - bk_base;
  for (int i = tid; i < a.S * R_; i += NT) basis_s[i] = a.basis[i];
  const int* bk_pre = a.bkg_inpre + bk_base;
  const float* bk_w = a.bkg_w + bk_base;
  const uint8_t* bk_sid = a.bkg_insid + bk_base;
  if (a.bkg_in_smem) {
    const int m = a.bkg_inptr[n0 + cn] - bk_base;
    for (int j = tid; j < m; j += NT) {
      bk_pre_s[j] = bk_pre[j];
      bk_w_s[j] = bk_w[j];
      bk_sid_s[j] = bk_sid[j];
    }
    bk_pre = bk_pre_s;
    bk_w = bk_w_s;
    bk_sid = bk_sid_s;
  }
  const bool have_state = a.st.v != nullptr;
  for (int i = tid; i < items; i += NT) {
    const int b = i / cn, k = i - b * cn, n = n0 + k;
    const int si = b * chunkP + k;
    const int64_t g = (int64_t)b * N + n;
    unsigned hist = 0;
    if (have_state) {
      S_v[si] = a.st.v[g];
      S_r[si] = (uint8_t)a.st.r[g];
      S_a0[si] = a.st.asc[2 * g];
      S_a1[si] = a.st.asc[2 * g + 1];
      for (int r = 0; r < R_; ++r) {
        S_p[(r * B + b) * chunkP + k] = a.st.psc[g * R_ + r];
        S_pr[(r * B + b) * chunkP + k] = a.st.psc_rise[g * R_ + r];
      }
      for (int d = 0; d < D; ++d)
        if (a.st.z_buf[((int64_t)b * D + d) * N + n] > 0.f) hist |= 1u << d;
    } else {
      S_v[si] = 0.f;
      S_r[si] = 0;
      S_a0[si] = 0.f;
      S_a1[si] = 0.f;
      for (int r = 0; r < R_; ++r) {
        S_p[(r * B + b) * chunkP + k] = 0.f;
        S_pr[(r * B + b) * chunkP + k] = 0.f;
      }
    }
    S_hist[si] = (uint8_t)hist;
  }
  if (tid == 0) {
    s_misc[0] = 0;
    s_misc[1] = 0;
    s_misc[2] = 0;
    s_misc[3] = 0;
  }
  __syncthreads();

  unsigned long long c_spikes = 0, c_rec_ev = 0, c_lgn_rows = 0, c_lgn_ev = 0, c_bkg_ev = 0,
                     c_bkg_rows = 0;

  auto walk_rec = [&](int b, int n, int te) {
    v1g_walk_rec<R_>(a, basis_s, lane, b, a.rec_rowptr + (int64_t)n * D, te, c_rec_ev);
  };
  auto scatter_lgn = [&](int tt) {
    v1g_scatter_lgn<R_>(a, basis_s, lane, (NW - 1 - warp) * gridDim.x + blockIdx.x, gridDim.x * NW, v1g_lgn_begin(a, tt),
                        v1g_lgn_begin(a, tt + 1), tt % a.K, c_lgn_rows, c_lgn_ev);
  };

  // ---- prologue: pending deliveries of the initial spike buffer, LGN events of step 0 ----
  if (have_state) {
    for (int i = warp; i < items; i += NW) {
      const int b = i / cn, k = i - b * cn;
      const unsigned hist = S_hist[b * chunkP + k];
      for (int d = 0; d < D; ++d)
        if (hist & (1u << d)) walk_rec(b, n0 + k, -(d + 1));
    }
  }
  if (a.T > 0) scatter_lgn(0);
  __syncthreads();
  if (tid == 0) v1g_arrive(v1g_phase_counter(a.barrier, 0));  // phase 0: prologue done

  const unsigned hist_mask = (1u << D) - 1u;
  const unsigned long long G = gridDim.x;
  const int nb = B * a.n_bkg;
  auto load_ring = [&](int b, int k, int slot, float (&I)[R_]) {
    const float* src = a.ring + ((int64_t)(slot * B + b) * R_) * Np + n0 + k;
#pragma unroll
    for (int r = 0; r < R_; ++r) I[r] = __ldcg(src + (int64_t)r * Np);
  };
  // total input of step s for item (b,k): ring slot (cleared on the way) + background gather
  auto finish_input = [&](int b, int k, int slot, const int* cnt_s, float (&I)[R_]) {
    float* dst = a.ring + ((int64_t)(slot * B + b) * R_) * Np + n0 + k;
#pragma unroll
    for (int r = 0; r < R_; ++r) __stcg(dst + (int64_t)r * Np, 0.f);
    float Gs[R_];
#pragma unroll
    for (int r = 0; r < R_; ++r) Gs[r] = 0.f;
    const int j1 = c_bkptr[k + 1];
    for (int j = c_bkptr[k]; j < j1; ++j) {
      const int cnt = cnt_s[b * a.n_bkg + bk_pre[j]];
      if (cnt > 0) {
        const float wc = bk_w[j] * (float)cnt;
        const float* bs = basis_s + (int)bk_sid[j] * R_;
#pragma unroll
        for (int r = 0; r < R_; ++r) Gs[r] += wc * bs[r];
        c_bkg_ev += 1;
      }
    }
#pragma unroll
    for (int r = 0; r < R_; ++r) I[r] = (I[r] + Gs[r]) * a.lr_scale;
  };

  unsigned long long ph_dense = 0, ph_scatter = 0, ph_barrier = 0;
  const bool prof = a.phase_ns != nullptr && tid == 0;
  const unsigned long long ph_start = prof ? gtime() : 0;
  unsigned long long seen = 0;  // thread 0: last value read from the barrier counter
  bool ok = true;

  // The currents delivered at step s enter psc_rise(s), reach psc(s+1) and the membrane only at
  // s+2, so iteration t (which produces v(t), z(t)) consumes ring slot t-2: it needs every block
  // to have finished iteration t-3, not t-1.  Blocks therefore synchronise through a LAGGED
  // counter and almost never wait.  On entry to iteration t the block holds psc(t-2) in S_p and
  // psc_rise(t-3) in S_pr (for t >= 2; the first two iterations start from the given state).
  for (int t = 0; t < a.T && ok; ++t) {
    const unsigned long long ph0 = prof ? gtime() : 0;
    if (tid == 0) {
      if (t >= 2) {
        // every block must have finished iteration t-3 (phase t-2)
        const unsigned long long target = v1g_phase_target(t - 2, G);
        if (seen < target)
          seen = v1g_wait(v1g_phase_counter(a.barrier, t - 2), target, a.spin_limit, a.status);
        if (seen < target) s_misc[1] = 1;
      }
    }
    __syncthreads();
    if (s_misc[1]) {
      ok = false;
      break;
    }
    // iteration t-1 of this block is complete: arrive at phase t
    if (tid == 0 && t >= 1) v1g_arrive(v1g_phase_counter(a.barrier, t));
    const unsigned long long ph1 = prof ? gtime() : 0;
    const bool consume = t >= 2;
    const int slot = consume ? (t - 2) % K : 0;
    const int* cnt_s = s_cnt + (t & 1) * nb;  // counts of step t-2
    // prefetch the counts of step t-1 (used by iteration t+1)
    int cnt_next[2] = {0, 0};
    if (t >= 1 && t + 1 < a.T + 2) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int i = tid + q * NT;
        if (i < nb) {
          const int b = i / a.n_bkg, j = i - b * a.n_bkg;
          cnt_next[q] = a.bkg_counts[((int64_t)b * a.T + (t - 1)) * a.n_bkg + j];
        }
      }
    }
    if (blockIdx.x == 0 && consume)
      for (int i = tid; i < nb; i += NT) c_bkg_rows += cnt_s[i] > 0 ? 1 : 0;
    int* nspk_p = &s_misc[2 + (t & 1)];

    // ---------------- dense phase ----------------
    float I[R_], In[R_];
    int b = 0, k = tid;
    while (k >= cn && b < B) { k -= cn; ++b; }
    if (consume && b < B) load_ring(b, k, slot, I);
    while (b < B) {
      int bn = b, kn = k + NT;
      while (kn >= cn && bn < B) { kn -= cn; ++bn; }
      if (consume && bn < B) load_ring(bn, kn, slot, In);
      const int n = n0 + k;
      const int si = b * chunkP + k;
      if (consume) finish_input(b, k, slot, cnt_s, I);
      // The whole state of the entry is read before any of it is written back: a load may not pass
      // an earlier store to the same array, and when the state lives in a global slab every read that
      // had to wait for the stores before it cost an L2 round trip of its own.
      const unsigned hist = S_hist[si];
      float pr_in[R_], p_in[R_];
#pragma unroll
      for (int r = 0; r < R_; ++r) {
        pr_in[r] = S_pr[(r * B + b) * chunkP + k];
        p_in[r] = S_p[(r * B + b) * chunkP + k];
      }
      const float a0 = S_a0[si], a1 = S_a1[si];
      const float v = S_v[si];
      const int r_in = (int)S_r[si];
      const float prev_z = (hist & 1u) ? 1.f : 0.f;
      float csum = 0.f;
#pragma unroll
      for (int r = 0; r < R_; ++r) {
        const int pi = (r * B + b) * chunkP + k;
        float pr = pr_in[r], p = p_in[r];
        if (consume) {
          pr = pr * a.sd[r] + I[r] * a.pinit[r];  // psc_rise(t-2)
          S_pr[pi] = pr;
        }
        if (t >= 1) {
          p = p * a.sd[r] + a.dtsd[r] * pr;  // psc(t-1)
          S_p[pi] = p;
        }
        csum = (r == 0) ? p : csum + p;
      }
      S_a0[si] = c_ad0[k] * a0 + prev_z * c_am0[k];
      S_a1[si] = c_ad1[k] * a1 + prev_z * c_am1[k];
      const float c1 = csum + (a0 + a1);
      const float dv = v * a.vd_keep + v * a.vd_drop;
      float nv = (c_decay[k] * dv + c_cf[k] * c1) - prev_z;
      int nr = r_in + ((hist & 1u) ? c_tref[k] : 0) - 1;
      nr = nr > 0 ? nr : 0;
      if (a.hard_reset && nr > 0) nv = 0.f;
      const bool z = ((nv - 1.f) > 0.f) && (nr == 0);
      S_v[si] = nv;
      S_r[si] = (uint8_t)nr;
      S_hist[si] = (uint8_t)(((hist << 1) | (z ? 1u : 0u)) & hist_mask);
      if (a.z_out) __stcs(a.z_out + ((int64_t)b * a.T + t) * N + n, (uint8_t)(z ? 1 : 0));
      if (a.v_out) __stcs(a.v_out + ((int64_t)b * a.T + t) * N + n, nv);
      if (a.tape_v) {
        const int64_t ti = ((int64_t)t * B + b) * N + n;
        // the voltage with its two lowest mantissa bits replaced by (spiked, refractory)
        __stcs(a.tape_v + ti, __uint_as_float((__float_as_uint(nv) & ~3u) | (z ? 1u : 0u) | (nr > 0 ? 2u : 0u)));
      }
      if (z) spk_list[atomicAdd(nspk_p, 1)] = ((uint32_t)b << 24) | (uint32_t)k;
#pragma unroll
      for (int r = 0; r < R_; ++r) I[r] = In[r];
      b = bn;
      k = kn;
    }
    {
      int* cnt_n = s_cnt + ((t + 1) & 1) * nb;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int ii = tid + q * NT;
        if (ii < nb) cnt_n[ii] = cnt_next[q];
      }
    }
    __syncthreads();
    const unsigned long long ph2 = prof ? gtime() : 0;
    // ---------------- scatter phase ----------------
    if (tid == 0) {
      // early poll of the phase the next iteration waits for
      seen = (t >= 1) ? v1g_ld_acquire(v1g_phase_counter(a.barrier, t - 1)) : 0;
      s_misc[2 + ((t + 1) & 1)] = 0;
    }
    const int nspk = *nspk_p;
    for (int e = warp; e < nspk; e += NW) {
      const uint32_t ent = spk_list[e];
      if (a.stat_neuron && lane == 0) {
        atomicAdd(a.stat_neuron + n0 + (int)(ent & 0xffffff), 1);
        atomicAdd(a.stat_pop + t * B + (int)(ent >> 24), 1);
      }
      walk_rec((int)(ent >> 24), n0 + (int)(ent & 0xffffff), t);
    }
    if (tid == 0) c_spikes += (unsigned long long)nspk;
    if (t + 1 < a.T) scatter_lgn(t + 1);
    if (prof) {
      const unsigned long long ph3 = gtime();
      ph_barrier += ph1 - ph0;
      ph_dense += ph2 - ph1;
      ph_scatter += ph3 - ph2;
    }
  }
  // ---- full barrier, then bring psc / psc_rise up to step T-1 ----
  __syncthreads();
  if (tid == 0) {
    if (ok && a.T >= 1) v1g_arrive(v1g_phase_counter(a.barrier, a.T));
    const unsigned long long target = v1g_phase_target(a.T, G);
    if (ok) {
      seen = v1g_wait(v1g_phase_counter(a.barrier, a.T), target, a.spin_limit, a.status);
      if (seen < target) s_misc[1] = 1;
    }
  }
  __syncthreads();
  ok = ok && !s_misc[1];
  if (ok && a.T >= 1) {
    // remaining input steps: T-2 (if any) and T-1
    for (int s = max(a.T - 2, 0); s < a.T; ++s) {
      __syncthreads();
      const int slot = s % K;
      for (int i = tid; i < nb; i += NT) {
        const int b = i / a.n_bkg, j = i - b * a.n_bkg;
        s_cnt[i] = a.bkg_counts[((int64_t)b * a.T + s) * a.n_bkg + j];
      }
      __syncthreads();
      if (blockIdx.x == 0)
        for (int i = tid; i < nb; i += NT) c_bkg_rows += s_cnt[i] > 0 ? 1 : 0;
      for (int i = tid; i < items; i += NT) {
        const int b = i / cn, k = i - b * cn;
        float I[R_];
        load_ring(b, k, slot, I);
        finish_input(b, k, slot, s_cnt, I);
#pragma unroll
        for (int r = 0; r < R_; ++r) {
          const int pi = (r * B + b) * chunkP + k;
          float pr = S_pr[pi];
          // psc(s) needs psc_rise(s-1): advance psc first unless it is already at step s
          if (s == a.T - 1 && a.T >= 1) S_p[pi] = S_p[pi] * a.sd[r] + a.dtsd[r] * pr;
          pr = pr * a.sd[r] + I[r] * a.pinit[r];
          S_pr[pi] = pr;
        }
      }
    }
    __syncthreads();
  }
  if (prof) {
    unsigned long long* o = a.phase_ns + 4 * blockIdx.x;
    o[0] = ph_dense;
    o[1] = ph_scatter;
    o[2] = ph_barrier;
    o[3] = gtime() - ph_start;
  }

  // ---- write the state back in the reference layouts ----
  if (have_state && ok) {
    for (int i = tid; i < items; i += NT) {
      const int b = i / cn, k = i - b * cn, n = n0 + k;
      const int si = b * chunkP + k;
      const int64_t g = (int64_t)b * N + n;
      a.st.v[g] = S_v[si];
      a.st.r[g] = (int8_t)S_r[si];
      a.st.asc[2 * g] = S_a0[si];
      a.st.asc[2 * g + 1] = S_a1[si];
      for (int r = 0; r < R_; ++r) {
        a.st.psc[g * R_ + r] = S_p[(r * B + b) * chunkP + k];
        a.st.psc_rise[g * R_ + r] = S_pr[(r * B + b) * chunkP + k];
      }
      const unsigned hist = S_hist[si];
      for (int d = 0; d < D; ++d) a.st.z_buf[((int64_t)b * D + d) * N + n] = (hist >> d) & 1u ? 1.f : 0.f;
    }
  }
  // ---- event counters ----
  c_rec_ev = v1g_warp_sum(c_rec_ev);
  c_lgn_rows = v1g_warp_sum(c_lgn_rows);
  c_lgn_ev = v1g_warp_sum(c_lgn_ev);
  c_bkg_ev = v1g_warp_sum(c_bkg_ev);
  c_bkg_rows = v1g_warp_sum(c_bkg_rows);
  if (lane == 0) {
    V1GCounters* c = (V1GCounters*)a.counters;
    if (c_rec_ev) atomicAdd(&c->rec_events, c_rec_ev);
    if (c_lgn_rows) atomicAdd(&c->lgn_rows, c_lgn_rows);
    if (c_lgn_ev) atomicAdd(&c->lgn_events, c_lgn_ev);
    if (c_bkg_ev) atomicAdd(&c->bkg_events, c_bkg_ev);
    if (c_bkg_rows) atomicAdd(&c->bkg_rows, c_bkg_rows);
    if (tid == 0 && c_spikes) {
      atomicAdd(&c->spikes, c_spikes);
      atomicAdd(&c->rec_rows, c_spikes * (unsigned long long)D);
    }
  }
}

template <int R_>
int launch_fwd(V1GHandle* h, const FwdArgs& a, int grid, size_t smem, cudaStream_t st) {
  auto kern = rollout_fwd_kernel<R_>;
  V1G_CUDA(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int per_sm = 0;
  V1G_CUDA(h, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NT, smem));
  if (per_sm < 1 || grid > per_sm * h->n_sms)
    return v1g_fail(h, V1G_ERANGE, "rollout grid of %d blocks cannot be co-resident (%d per SM)", grid, per_sm);
  void* args[] = {(void*)&a};
  V1G_CUDA(h, cudaEventRecord(h->ev[0], st));
  V1G_CUDA(h, cudaLaunchCooperativeKernel((void*)kern, dim3(grid), dim3(NT), args, smem, st));
  V1G_CUDA(h, cudaEventRecord(h->ev[1], st));
  h->ev_valid[0] = true;
  v1g_count_launches(1);
  return V1G_OK;
}

}  // namespace

// Sizes the per-block slice, decides where state and the background table live, and returns the
// dynamic shared-memory bytes.  Shared by the forward and backward rollouts.
size_t v1g_plan_rollout(const V1GHandle* h, int B, int per_item_floats, int per_item_bytes,
                        int fixed_per_neuron_bytes, V1GRolloutPlan* p) {
  const int N = h->cfg.n_neurons;
  int chunk = h->opt_chunk > 0 ? h->opt_chunk : (N + h->n_sms - 1) / h->n_sms;
  if (h->opt_chunk == 0 && chunk < 32) chunk = 32;
  if (chunk > N) chunk = N;
  p->chunk = chunk;
  p->grid = (N + chunk - 1) / chunk;
  p->chunkP = (chunk + 31) & ~31;
  const size_t plane = (size_t)B * p->chunkP;
  p->state_bytes = plane * per_item_floats * sizeof(float) + plane * per_item_bytes;
  p->fixed_bytes = (size_t)p->chunkP * fixed_per_neuron_bytes + 64 * 16;
  return p->fixed_bytes;
}

namespace {
// One thread waits, with the same bounded-wait helper the rollout kernels use, for a counter that
// nothing increments.
__global__ void bounded_wait_probe_kernel(unsigned long long* counter, long long polls, int32_t* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) v1g_wait(counter, 1ULL, polls, status);
}
}  // namespace

extern "C" int v1g_selftest_bounded_wait(V1GHandle* h, long long polls, void* stream) {
  if (!h || polls < 1 || polls > 100000000LL) return h ? v1g_fail(h, V1G_EINVAL, "polls outside 1..1e8") : V1G_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  V1G_CUDA(h, cudaMemsetAsync(h->barrier, 0, V1G_BARRIER_BYTES, st));
  bounded_wait_probe_kernel<<<1, 32, 0, st>>>(h->barrier, polls, h->dev_status);
  v1g_count_launches(1);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

// x: LGN spikes [B,T,n_lgn], or NULL with `rates` set (spikes drawn on the fly into the event list);
// bkg_counts NULL: drawn on the device for the steps that state->noise_step[0] names.
static int rollout_fwd_impl(V1GHandle* h, int32_t batch, int32_t n_steps, const uint8_t* x,
                            const V1GRateSource* rates, const int32_t* bkg_counts, V1GState* state,
                            uint8_t* z_out, float* v_out, int32_t save_for_bwd, void* stream) {
  if (!h) return V1G_EINVAL;
  if (!h->params_set) return v1g_fail(h, V1G_ESTATE, "neuron parameters not set");
  for (int s = 0; s < V1G_NSRC; ++s)
    if (!h->src[s].rowptr) return v1g_fail(h, V1G_ESTATE, "connectivity of source %d not set", s);
  if (batch <= 0 || batch > V1G_MAX_BATCH)
    return v1g_fail(h, V1G_ERANGE, "batch=%d outside 1..%d", batch, V1G_MAX_BATCH);
  if (n_steps < 0 || (!x && !rates)) return v1g_fail(h, V1G_EINVAL, "v1g_rollout_fwd: bad argument");
  if (state && !(state->z_buf && state->v && state->r && state->asc && state->psc_rise && state->psc))
    return v1g_fail(h, V1G_EINVAL, "v1g_rollout_fwd: state has null members");
  cudaStream_t st = (cudaStream_t)stream;
  const V1GConfig& c = h->cfg;
  const int N = c.n_neurons, R = c.n_receptors, D = c.max_delay, K = D + 6, B = batch, T = n_steps;
  h->tape_valid = false;
  if (T == 0) return V1G_OK;
  int rc;
  if (!bkg_counts) {
    // draw the counts into the handle's own buffer (kept for the backward pass when asked to save)
    const int64_t nc = (int64_t)B * T * c.n_bkg;
    if ((rc = v1g_reserve(h, &h->tape_counts_buf, &h->tape_counts_cap, nc))) return rc;
    if ((rc = v1g_sample_bkg_internal(h, B, T, state ? state->noise_step : nullptr, 0, h->tape_counts_buf, st)))
      return rc;
    bkg_counts = h->tape_counts_buf;
  }

  // ---- LGN events: ordered compaction of x[B,T,n_lgn] into a time-major list ----
  const int nseg = (c.n_lgn + V1G_SEG - 1) / V1G_SEG;
  const int64_t nsegs = (int64_t)B * T * nseg;
  if ((rc = v1g_reserve(h, &h->lgn_offsets, &h->lgn_offsets_cap, nsegs + 1))) return rc;
  const int lgn_kind = x ? V1G_COMPACT_U8_PACKED : V1G_COMPACT_LGN_RATES;
  const void* lgn_src = x ? (const void*)x : (const void*)rates;
  if ((rc = v1g_compact_count_scan(h, lgn_kind, lgn_src, B * T, c.n_lgn, T, h->lgn_offsets, nullptr, st)))
    return rc;
  V1G_CUDA(h, cudaMemcpyAsync(h->h_count, h->d_count, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  V1G_CUDA(h, cudaStreamSynchronize(st));
  const int64_t n_lgn_events = h->h_count[0];
  if ((rc = v1g_reserve(h, &h->lgn_entries, &h->lgn_entries_cap, n_lgn_events + 1))) return rc;
  if ((rc = v1g_compact_fill(h, lgn_kind, lgn_src, B * T, c.n_lgn, T, h->lgn_offsets, h->lgn_entries,
                             n_lgn_events, st)))
    return rc;
  if ((rc = v1g_reserve(h, &h->lgn_ent4, &h->lgn_ent4_cap, n_lgn_events + 1))) return rc;
  if (n_lgn_events > 0) {
    lgn_resolve_kernel<<<(unsigned)std::min<int64_t>((n_lgn_events + 255) / 256, 148 * 8), 256, 0, st>>>(
        h->lgn_entries, n_lgn_events, h->src[V1G_SRC_LGN].rowptr, h->lgn_ent4);
    v1g_count_launches(1);
    V1G_CUDA(h, cudaGetLastError());
  }
  h->lgn_nseg = nseg;

  // ---- plan ----
  V1GRolloutPlan plan;
  v1g_plan_rollout(h, B, 3 + 2 * R, 2, 0, &plan);
  const int Np = (N + 31) & ~31;
  const V1GSource& bk = h->src[V1G_SRC_BKG];
  // largest background in-synapse count of any block slice
  int bkg_cap = 0;
  for (int g = 0; g < plan.grid; ++g) {
    const int a0 = g * plan.chunk, a1 = std::min(N, a0 + plan.chunk);
    bkg_cap = std::max(bkg_cap, bk.in_ptr_host[a1] - bk.in_ptr_host[a0]);
  }
  // balanced slices (register-resident kernel only): valid for this grid, at most V1G_NT_REG neurons each
  const bool sliced = (int)h->fwd_slice_host.size() == plan.grid + 1 && h->fwd_slice != nullptr;
  int bkg_cap_sliced = 0;
  if (sliced)
    for (int g = 0; g < plan.grid; ++g)
      bkg_cap_sliced = std::max(bkg_cap_sliced, bk.in_ptr_host[h->fwd_slice_host[g + 1]] - bk.in_ptr_host[h->fwd_slice_host[g]]);
  auto al = [](size_t b) { return (b + 15) & ~(size_t)15; };
  size_t smem = 7 * al(sizeof(float) * plan.chunkP) + al(sizeof(int) * (plan.chunkP + 1)) +
                al(sizeof(float) * c.n_syn_types * R) + al(sizeof(uint32_t) * B * plan.chunkP) +
                al(sizeof(int) * 2 * B * c.n_bkg) + al(sizeof(int) * 4);
  const size_t bkg_bytes = al(sizeof(int) * bkg_cap) + al(sizeof(float) * bkg_cap) + al(bkg_cap);
  const size_t state_bytes = al(plan.state_bytes);
  const size_t limit = (size_t)h->smem_optin;
  int state_in_smem = 0, bkg_in_smem = 0;
  if (!h->opt_force_global && smem + state_bytes <= limit) {
    state_in_smem = 1;
    smem += state_bytes;
  }
  if (smem + bkg_bytes <= limit) {
    bkg_in_smem = 1;
    smem += bkg_bytes;
  }
  if (smem > limit) return v1g_fail(h, V1G_ERANGE, "rollout needs %zu B of shared memory per block", smem);
  if (!state_in_smem) {
    const size_t plane = (size_t)B * plan.chunkP;
    const size_t slab = plane * (3 + 2 * R) + (2 * plane + 3) / 4;
    if ((rc = v1g_reserve(h, &h->state_ws, &h->state_ws_cap, (int64_t)(slab * plan.grid)))) return rc;
  }
  const int64_t ring_elems = (int64_t)K * B * R * Np;
  if ((rc = v1g_reserve(h, &h->ring, &h->ring_cap, ring_elems))) return rc;
  if (save_for_bwd) {
    const int64_t need = (int64_t)T * B * N;
    if (need > h->tape_cap || !h->tape_v) {
      if (h->tape_v) cudaFree(h->tape_v);
      h->tape_v = nullptr;
      h->tape_cap = 0;
      V1G_CUDA(h, cudaMalloc((void**)&h->tape_v, (size_t)need * sizeof(float)));
      h->tape_cap = need;
    }
  }
  if (save_for_bwd) {
    const int64_t ns = (int64_t)N + (int64_t)T * B;
    if ((rc = v1g_reserve(h, &h->tape_stats, &h->tape_stats_cap, ns))) return rc;
    V1G_CUDA(h, cudaMemsetAsync(h->tape_stats, 0, (size_t)ns * sizeof(int32_t), st));
  }
  h->tape_has_hist0 = false;
  if (save_for_bwd && state) {
    if ((rc = v1g_reserve(h, &h->tape_hist0, &h->tape_hist0_cap, (int64_t)B * N))) return rc;
    hist0_kernel<<<(unsigned)(((int64_t)B * N + 255) / 256), 256, 0, st>>>(state->z_buf, B, D, N, h->tape_hist0);
    v1g_count_launches(1);
    h->tape_has_hist0 = true;
  }
  V1G_CUDA(h, cudaMemsetAsync(h->ring, 0, (size_t)ring_elems * sizeof(float), st));
  V1G_CUDA(h, cudaMemsetAsync(h->barrier, 0, V1G_BARRIER_BYTES, st));
  V1G_CUDA(h, cudaMemsetAsync(h->counters, 0, sizeof(V1GCounters), st));

  FwdArgs a;
  a.N = N; a.D = D; a.K = K; a.B = B; a.T = T; a.Np = Np;
  a.chunk = plan.chunk; a.chunkP = plan.chunkP; a.S = c.n_syn_types; a.n_bkg = c.n_bkg;
  a.state_in_smem = state_in_smem; a.bkg_in_smem = bkg_in_smem; a.bkg_cap = bkg_cap;
  const V1GSource& rs = h->src[V1G_SRC_REC];
  const V1GSource& ls = h->src[V1G_SRC_LGN];
  a.rec_rowptr = rs.rowptr; a.rec_post = rs.post; a.rec_w = rs.w; a.rec_sid = rs.sid;
  a.lgn_rowptr = ls.rowptr; a.lgn_post = ls.post; a.lgn_w = ls.w; a.lgn_sid = ls.sid;
  a.bkg_inptr = bk.in_ptr; a.bkg_inpre = bk.in_pre; a.bkg_w = bk.gather_w(); a.bkg_insid = bk.in_sid;
  a.decay = h->decay; a.cf = h->cf; a.asc_decay = h->asc_decay; a.asc_amps = h->asc_amps;
  a.basis = h->basis; a.tref = h->tref;
  for (int r = 0; r < V1G_MAX_RECEPTORS; ++r) {
    a.sd[r] = r < R ? h->syn_decay[r] : 0.f;
    a.pinit[r] = r < R ? h->psc_initial[r] : 0.f;
    a.dtsd[r] = c.dt * a.sd[r];
  }
  a.lr_scale = c.lr_scale; a.vd_keep = h->vd_keep; a.vd_drop = h->vd_drop;
  a.hard_reset = (c.flags & V1G_FLAG_HARD_RESET) ? 1 : 0;
  a.lgn_off = h->lgn_offsets; a.lgn_entries = h->lgn_entries; a.lgn_ent4 = h->lgn_ent4; a.lgn_nseg = nseg;
  a.rec_syn8 = h->opt_no_meta ? nullptr : h->src[V1G_SRC_REC].syn8;
  a.lgn_syn8 = h->opt_no_meta ? nullptr : h->src[V1G_SRC_LGN].syn8;
  a.bkg_counts = bkg_counts;
  a.stat_neuron = save_for_bwd ? h->tape_stats : nullptr;
  a.stat_pop = save_for_bwd ? h->tape_stats + N : nullptr;
  if (state) a.st = *state; else a.st = V1GState{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  a.state_ws = h->state_ws;
  a.z_out = z_out; a.v_out = v_out;
  a.tape_v = save_for_bwd ? h->tape_v : nullptr;
  a.ring = h->ring; a.barrier = h->barrier; a.status = h->dev_status; a.counters = h->counters;
  a.spin_limit = h->opt_spin_limit;
  a.phase_ns = nullptr;
  if (h->opt_phase_timers) {
    if ((rc = v1g_reserve(h, &h->phase_ns, &h->phase_ns_cap, (int64_t)4 * plan.grid))) return rc;
    V1G_CUDA(h, cudaMemsetAsync(h->phase_ns, 0, sizeof(unsigned long long) * 4 * plan.grid, st));
    a.phase_ns = h->phase_ns;
    h->phase_grid = plan.grid;
  }
  if (2 * NT < B * c.n_bkg)
    return v1g_fail(h, V1G_ERANGE, "batch*n_bkg=%d exceeds %d", B * c.n_bkg, 2 * NT);

  // Register-resident kernel when the slice fits one neuron per thread and the (R, B) pair is
  // instantiated; the shared-memory kernel otherwise.
  const bool reg_ok = !h->opt_force_smem_kernel && !h->opt_force_global && plan.chunk <= V1G_NT_REG &&
                      (R == 4 || R == 5) && B <= 6 &&
                      v1g_fwd_reg_smem(h, B, plan.chunkP, bkg_cap) <= limit;
  a.slice = nullptr;
  if (reg_ok && sliced && v1g_fwd_reg_smem(h, B, plan.chunkP, bkg_cap_sliced) <= limit) {
    a.slice = h->fwd_slice;
    a.bkg_cap = bkg_cap_sliced;
    rc = v1g_launch_fwd_reg(h, a, R, plan.grid, v1g_fwd_reg_smem(h, B, plan.chunkP, bkg_cap_sliced), st);
  } else if (reg_ok) {
    rc = v1g_launch_fwd_reg(h, a, R, plan.grid, v1g_fwd_reg_smem(h, B, plan.chunkP, bkg_cap), st);
  } else
  switch (R) {
    case 1: rc = launch_fwd<1>(h, a, plan.grid, smem, st); break;
    case 2: rc = launch_fwd<2>(h, a, plan.grid, smem, st); break;
    case 3: rc = launch_fwd<3>(h, a, plan.grid, smem, st); break;
    case 4: rc = launch_fwd<4>(h, a, plan.grid, smem, st); break;
    case 5: rc = launch_fwd<5>(h, a, plan.grid, smem, st); break;
    case 6: rc = launch_fwd<6>(h, a, plan.grid, smem, st); break;
    case 7: rc = launch_fwd<7>(h, a, plan.grid, smem, st); break;
    default: rc = launch_fwd<8>(h, a, plan.grid, smem, st); break;
  }
  if (rc) return rc;
  if (save_for_bwd) {
    // the backward pass needs the counts again; keep a copy so that the caller's buffer may be
    // reused as soon as this call has been queued
    const int64_t nc = (int64_t)B * T * c.n_bkg;
    if (bkg_counts != h->tape_counts_buf) {
      if ((rc = v1g_reserve(h, &h->tape_counts_buf, &h->tape_counts_cap, nc))) return rc;
      V1G_CUDA(h, cudaMemcpyAsync(h->tape_counts_buf, bkg_counts, (size_t)nc * sizeof(int32_t),
                                  cudaMemcpyDeviceToDevice, st));
    }
    h->tape_valid = true;
    h->tape_B = B;
    h->tape_T = T;
    h->tape_counts = h->tape_counts_buf;
  }
  if (state && state->noise_step) return v1g_advance_noise_step(h, state->noise_step, B, T, st);
  return V1G_OK;
}

// Slices of equal scatter work for the register-resident forward kernel.  The dense part costs the
// same whatever a block's slice holds (one neuron per thread, at most V1G_NT_REG), while the scatter
// costs one walk of a neuron's out-synapses per spike, and networks are ordered by cell type, so with
// equal slices the blocks that own the most active types set the pace of every step and the others
// wait.  cost[n] = spikes of neuron n x its out-degree (+ 2 % of the mean so that silent stretches are
// shared out too); boundaries by bisection on the largest slice cost, greedy from the left.
extern "C" int v1g_balance_slices(V1GHandle* h, const float* cost_host, void* stream) {
  if (!h) return V1G_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  const int N = h->cfg.n_neurons, D = h->cfg.max_delay;
  V1GRolloutPlan plan;
  v1g_plan_rollout(h, 1, 0, 0, 0, &plan);
  h->fwd_slice_host.clear();
  if (plan.chunk > V1G_NT_REG || plan.grid < 2) return V1G_OK;  // the general kernel keeps equal slices
  std::vector<double> cost((size_t)N);
  if (cost_host) {
    for (int n = 0; n < N; ++n) {
      if (!(cost_host[n] >= 0.f)) return v1g_fail(h, V1G_EINVAL, "v1g_balance_slices: cost[%d] is negative or not a number", n);
      cost[(size_t)n] = cost_host[n];
    }
  } else {
    const V1GSource& rs = h->src[V1G_SRC_REC];
    if (!h->tape_valid || !h->tape_stats || rs.rowptr_host.size() < (size_t)N * D + 1)
      return v1g_fail(h, V1G_EINVAL, "v1g_balance_slices without costs needs a rollout saved for the backward pass");
    std::vector<int32_t> spikes((size_t)N);
    V1G_CUDA(h, cudaMemcpyAsync(spikes.data(), h->tape_stats, sizeof(int32_t) * (size_t)N, cudaMemcpyDeviceToHost, st));
    V1G_CUDA(h, cudaStreamSynchronize(st));
    for (int n = 0; n < N; ++n)
      cost[(size_t)n] = (double)spikes[(size_t)n] * (double)(rs.rowptr_host[(size_t)(n + 1) * D] - rs.rowptr_host[(size_t)n * D]);
  }
  double total = 0.0, largest = 0.0;
  for (double c : cost) total += c;
  const double floor_cost = total > 0.0 ? 0.02 * total / N : 1.0;
  total = 0.0;
  for (double& c : cost) {
    c += floor_cost;
    total += c;
    largest = std::max(largest, c);
  }
  const int G = plan.grid, cap = V1G_NT_REG;
  auto cut = [&](double limit, std::vector<int32_t>* out) {  // greedy slices of cost <= limit and size <= cap
    int slices = 0, size = 0;
    double acc = 0.0;
    if (out) out->assign(1, 0);
    for (int n = 0; n < N; ++n) {
      if (size > 0 && (size == cap || acc + cost[(size_t)n] > limit)) {
        ++slices;
        if (out) out->push_back(n);
        size = 0;
        acc = 0.0;
      }
      ++size;
      acc += cost[(size_t)n];
    }
    if (out) out->push_back(N);
    return slices + 1;
  };
  if (cut(total, nullptr) > G) return V1G_OK;  // more than cap neurons per block on average: cannot happen with chunk <= cap
  double lo = largest, hi = total;
  for (int it = 0; it < 50; ++it) {
    const double mid = 0.5 * (lo + hi);
    if (cut(mid, nullptr) <= G) hi = mid; else lo = mid;
  }
  std::vector<int32_t> bounds;
  cut(hi, &bounds);
  while ((int)bounds.size() < G + 1) {  // fewer slices than blocks: halve the widest until every block has one
    size_t widest = 0;
    for (size_t g = 0; g + 1 < bounds.size(); ++g)
      if (bounds[g + 1] - bounds[g] > bounds[widest + 1] - bounds[widest]) widest = g;
    if (bounds[widest + 1] - bounds[widest] < 2) return V1G_OK;  // fewer neurons than blocks
    bounds.insert(bounds.begin() + (long)widest + 1, (bounds[widest] + bounds[widest + 1]) / 2);
  }
  if (!h->fwd_slice) V1G_CUDA(h, cudaMalloc((void**)&h->fwd_slice, sizeof(int32_t) * 1024));
  if (G + 1 > 1024) return V1G_OK;
  V1G_CUDA(h, cudaMemcpyAsync(h->fwd_slice, bounds.data(), sizeof(int32_t) * (size_t)(G + 1), cudaMemcpyHostToDevice, st));
  V1G_CUDA(h, cudaStreamSynchronize(st));
  h->fwd_slice_host = bounds;
  return V1G_OK;
}

extern "C" int v1g_rollout_fwd(V1GHandle* h, int32_t batch, int32_t n_steps, const uint8_t* x,
                               const int32_t* bkg_counts, V1GState* state, uint8_t* z_out,
                               float* v_out, int32_t save_for_bwd, void* stream) {
  if (h && !x) return v1g_fail(h, V1G_EINVAL, "v1g_rollout_fwd: x is NULL");
  return rollout_fwd_impl(h, batch, n_steps, x, nullptr, bkg_counts, state, z_out, v_out, save_for_bwd, stream);
}

extern "C" int v1g_rollout_fwd_rates(V1GHandle* h, int32_t batch, int32_t n_steps, const float* rates,
                                     int64_t rates_batch_stride, int64_t lgn_seed,
                                     const int32_t* bkg_counts, V1GState* state, uint8_t* z_out,
                                     float* v_out, int32_t save_for_bwd, void* stream) {
  if (!h) return V1G_EINVAL;
  if (!rates || rates_batch_stride < 0) return v1g_fail(h, V1G_EINVAL, "v1g_rollout_fwd_rates: bad argument");
  V1GRateSource src{rates, rates_batch_stride, (unsigned)lgn_seed, (unsigned)((uint64_t)lgn_seed >> 32)};
  return rollout_fwd_impl(h, batch, n_steps, nullptr, &src, bkg_counts, state, z_out, v_out, save_for_bwd, stream);
}

extern "C" int v1g_rollout_fwd_host(V1GHandle* h, int32_t batch, int32_t n_steps,
                                    const uint8_t* x_host, const int32_t* bkg_counts_host,
                                    uint8_t* z_out_host, float* v_out_host, int32_t save_for_bwd,
                                    void* stream) {
  if (!h) return V1G_EINVAL;
  if (batch <= 0 || n_steps < 0 || !x_host || !bkg_counts_host)
    return v1g_fail(h, V1G_EINVAL, "v1g_rollout_fwd_host: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  const V1GConfig& c = h->cfg;
  const int64_t nx = (int64_t)batch * n_steps * c.n_lgn, nc = (int64_t)batch * n_steps * c.n_bkg;
  const int64_t no = (int64_t)batch * n_steps * c.n_neurons;
  int rc;
  if ((rc = v1g_reserve(h, &h->stage_x, &h->stage_x_cap, nx))) return rc;
  if ((rc = v1g_reserve(h, &h->stage_counts, &h->stage_counts_cap, nc))) return rc;
  if (z_out_host && (rc = v1g_reserve(h, &h->stage_z, &h->stage_z_cap, no))) return rc;
  if (v_out_host && (rc = v1g_reserve(h, &h->stage_v, &h->stage_v_cap, no))) return rc;
  V1G_CUDA(h, cudaMemcpyAsync(h->stage_x, x_host, (size_t)nx, cudaMemcpyHostToDevice, st));
  V1G_CUDA(h, cudaMemcpyAsync(h->stage_counts, bkg_counts_host, (size_t)nc * sizeof(int32_t),
                              cudaMemcpyHostToDevice, st));
  if ((rc = v1g_rollout_fwd(h, batch, n_steps, h->stage_x, h->stage_counts, nullptr,
                            z_out_host ? h->stage_z : nullptr, v_out_host ? h->stage_v : nullptr,
                            save_for_bwd, st)))
    return rc;
  if (z_out_host)
    V1G_CUDA(h, cudaMemcpyAsync(z_out_host, h->stage_z, (size_t)no, cudaMemcpyDeviceToHost, st));
  if (v_out_host)
    V1G_CUDA(h, cudaMemcpyAsync(v_out_host, h->stage_v, (size_t)no * sizeof(float),
                                cudaMemcpyDeviceToHost, st));
  return v1g_synchronize(h, st);
}


// ------------------------------------------------------------------------------------------
// Forward-only evaluation through host buffers, pipelined
// ------------------------------------------------------------------------------------------
namespace {
// z[rows][N] uint8 -> bits[rows][nw] uint32 (bit n % 32 of word n / 32): one warp per 32 words,
// a ballot per word, one coalesced store of the 32 words
__global__ void __launch_bounds__(256) pack_bits_kernel(const uint8_t* __restrict__ z, int64_t rows, int N, int nw,
                                                        uint32_t* __restrict__ bits) {
  const int lane = threadIdx.x & 31;
  const int64_t groups_per_row = (nw + 31) / 32;
  const int64_t n_groups = rows * groups_per_row;
  for (int64_t g = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); g < n_groups;
       g += (int64_t)gridDim.x * (blockDim.x >> 5)) {
    const int64_t row = g / groups_per_row;
    const int w0 = (int)(g - row * groups_per_row) * 32;
    const uint8_t* zr = z + row * N;
    uint32_t mine = 0;
    for (int i = 0; i < 32; ++i) {
      const int n = (w0 + i) * 32 + lane;
      const unsigned bal = __ballot_sync(0xffffffffu, n < N && zr[n] != 0);
      if (i == lane) mine = bal;
    }
    if (w0 + lane < nw) bits[row * nw + w0 + lane] = mine;
  }
}
}  // namespace

extern "C" int v1g_rollout_fwd_host_pipelined(V1GHandle* h, int32_t batch, int32_t n_steps, const uint8_t* x_host,
                                              const int32_t* bkg_counts_host, void* z_out_host, int32_t z_format,
                                              int32_t chunk_steps, void* stream) {
  if (!h) return V1G_EINVAL;
  if (batch <= 0 || batch > V1G_MAX_BATCH || n_steps < 0 || !x_host || !bkg_counts_host || z_format < 0 ||
      z_format > 1 || chunk_steps < 0)
    return v1g_fail(h, V1G_EINVAL, "v1g_rollout_fwd_host_pipelined: bad argument");
  if (n_steps == 0) return V1G_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const V1GConfig& c = h->cfg;
  const int B = batch, T = n_steps, N = c.n_neurons, R = c.n_receptors, D = c.max_delay;
  const int nw = (N + 31) / 32;
  int ct = chunk_steps > 0 ? chunk_steps : std::min(std::max(T / 10, 50), 500);
  ct = std::min(ct, T);
  int rc;
  // streams and events of the pipeline
  if (!h->pipe_in) {
    V1G_CUDA(h, cudaStreamCreateWithFlags(&h->pipe_in, cudaStreamNonBlocking));
    V1G_CUDA(h, cudaStreamCreateWithFlags(&h->pipe_out, cudaStreamNonBlocking));
    for (int i = 0; i < 6; ++i) V1G_CUDA(h, cudaEventCreateWithFlags(&h->pipe_ev[i], cudaEventDisableTiming));
  }
  cudaEvent_t* in_ready = h->pipe_ev;      // [2] inputs of the buffer are on the device
  cudaEvent_t* done = h->pipe_ev + 2;      // [2] the rollout over the buffer has finished
  cudaEvent_t* out_done = h->pipe_ev + 4;  // [2] the results of the buffer are on the host
  // double buffers and the carried state
  const int64_t nx = (int64_t)B * ct * c.n_lgn, nc = (int64_t)B * ct * c.n_bkg, nz = (int64_t)B * ct * N;
  const int64_t nb = (int64_t)B * ct * nw;
  if ((rc = v1g_reserve(h, &h->stage_x, &h->stage_x_cap, 2 * nx))) return rc;
  if ((rc = v1g_reserve(h, &h->stage_counts, &h->stage_counts_cap, 2 * nc))) return rc;
  if (z_out_host && (rc = v1g_reserve(h, &h->stage_z, &h->stage_z_cap, 2 * nz))) return rc;
  if (z_out_host && z_format == 1 && (rc = v1g_reserve(h, &h->stage_bits, &h->stage_bits_cap, 2 * nb))) return rc;
  const int64_t sf = (int64_t)B * N * (D + 1 + 2 + 2 * R);  // z_buf, v, asc, psc_rise, psc
  if ((rc = v1g_reserve(h, &h->pipe_state, &h->pipe_state_cap, sf + ((int64_t)B * N + 3) / 4))) return rc;
  V1G_CUDA(h, cudaMemsetAsync(h->pipe_state, 0, (size_t)(sf + ((int64_t)B * N + 3) / 4) * sizeof(float), st));
  V1GState state;
  state.z_buf = h->pipe_state;
  state.v = state.z_buf + (int64_t)B * N * D;
  state.asc = state.v + (int64_t)B * N;
  state.psc_rise = state.asc + (int64_t)B * N * 2;
  state.psc = state.psc_rise + (int64_t)B * N * R;
  state.r = (int8_t*)(state.psc + (int64_t)B * N * R);
  state.noise_step = nullptr;
  // the side streams start after what is queued on the caller's stream
  V1G_CUDA(h, cudaEventRecord(done[0], st));
  V1G_CUDA(h, cudaEventRecord(done[1], st));
  V1G_CUDA(h, cudaEventRecord(out_done[0], st));
  V1G_CUDA(h, cudaEventRecord(out_done[1], st));
  const int n_chunks = (T + ct - 1) / ct;
  auto copy_in = [&](int k) -> int {
    const int s = k & 1, t0 = k * ct, len = std::min(ct, T - t0);
    V1G_CUDA(h, cudaStreamWaitEvent(h->pipe_in, done[s], 0));  // the rollout that read this buffer is through
    V1G_CUDA(h, cudaMemcpy2DAsync(h->stage_x + s * nx, (size_t)len * c.n_lgn, x_host + (int64_t)t0 * c.n_lgn,
                                  (size_t)T * c.n_lgn, (size_t)len * c.n_lgn, B, cudaMemcpyHostToDevice, h->pipe_in));
    V1G_CUDA(h, cudaMemcpy2DAsync(h->stage_counts + s * nc, (size_t)len * c.n_bkg * 4,
                                  bkg_counts_host + (int64_t)t0 * c.n_bkg, (size_t)T * c.n_bkg * 4,
                                  (size_t)len * c.n_bkg * 4, B, cudaMemcpyHostToDevice, h->pipe_in));
    V1G_CUDA(h, cudaEventRecord(in_ready[s], h->pipe_in));
    return V1G_OK;
  };
  if ((rc = copy_in(0))) return rc;
  for (int k = 0; k < n_chunks; ++k) {
    const int s = k & 1, t0 = k * ct, len = std::min(ct, T - t0);
    if (k + 1 < n_chunks && (rc = copy_in(k + 1))) return rc;
    V1G_CUDA(h, cudaStreamWaitEvent(st, in_ready[s], 0));
    V1G_CUDA(h, cudaStreamWaitEvent(st, out_done[s], 0));  // the previous results of this buffer have left
    uint8_t* zc = z_out_host ? h->stage_z + s * nz : nullptr;
    if ((rc = rollout_fwd_impl(h, B, len, h->stage_x + s * nx, nullptr, h->stage_counts + s * nc, &state, zc,
                               nullptr, 0, st)))
      return rc;
    if (z_out_host && z_format == 1) {
      const int64_t rows = (int64_t)B * len;
      pack_bits_kernel<<<(unsigned)std::min<int64_t>((rows * ((nw + 31) / 32) + 7) / 8, (int64_t)h->n_sms * 16), 256, 0,
                         st>>>(zc, rows, N, nw, h->stage_bits + s * nb);
      v1g_count_launches(1);
      V1G_CUDA(h, cudaGetLastError());
    }
    V1G_CUDA(h, cudaEventRecord(done[s], st));
    if (z_out_host) {
      V1G_CUDA(h, cudaStreamWaitEvent(h->pipe_out, done[s], 0));
      if (z_format == 1)
        V1G_CUDA(h, cudaMemcpy2DAsync((uint32_t*)z_out_host + (int64_t)t0 * nw, (size_t)T * nw * 4,
                                      h->stage_bits + s * nb, (size_t)len * nw * 4, (size_t)len * nw * 4, B,
                                      cudaMemcpyDeviceToHost, h->pipe_out));
      else
        V1G_CUDA(h, cudaMemcpy2DAsync((uint8_t*)z_out_host + (int64_t)t0 * N, (size_t)T * N, zc, (size_t)len * N,
                                      (size_t)len * N, B, cudaMemcpyDeviceToHost, h->pipe_out));
      V1G_CUDA(h, cudaEventRecord(out_done[s], h->pipe_out));
    }
  }
  V1G_CUDA(h, cudaStreamSynchronize(h->pipe_out));
  V1G_CUDA(h, cudaStreamSynchronize(h->pipe_in));
  return v1g_synchronize(h, st);
}
