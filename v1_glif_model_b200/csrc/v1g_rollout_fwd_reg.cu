// Forward rollout, register-resident variant: one thread per neuron, the batch unrolled at
// compile time, v / asc / psc / refractory counter / spike history of all batch rows of the
// neuron held in registers for the whole rollout (psc_rise, touched once per step, sits in a
// conflict-free shared-memory plane, one word per lane, to stay under 128 registers).  Per-neuron constants and the neuron's
// background in-synapses are read once per neuron and step instead of once per (batch, neuron).
// Used when the block slice has at most V1G_NT_REG neurons; otherwise the shared-memory kernel in
// v1g_rollout_fwd.cu runs.  Synchronisation, ring protocol and arithmetic (operation order
// included) are identical to that kernel.
#include "v1g_rollout_fwd.cuh"

namespace {

// asynchronous global -> shared copies of 4 and 16 bytes (both addresses aligned to the size)
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}

constexpr int NT = V1G_NT_REG;
constexpr int NW = NT / 32;

template <int R_, int B_>
__global__ void __launch_bounds__(NT, 1) rollout_fwd_reg_kernel(const FwdArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int D = a.D, K = a.K, N = a.N, Np = a.Np;
  // equal slices, or slices of equal scatter work (at most one neuron per thread either way)
  const int n0 = a.slice ? a.slice[blockIdx.x] : blockIdx.x * a.chunk;
  const int cn = a.slice ? a.slice[blockIdx.x + 1] - n0 : min(a.chunk, N - n0);
  const bool active = tid < cn;
  const int n = n0 + (active ? tid : 0);
  const int nb = B_ * a.n_bkg;

  unsigned char* sp_ = smem_raw;
  auto take = [&](size_t bytes) {
    unsigned char* p = sp_;
    sp_ += (bytes + 15) & ~(size_t)15;
    return p;
  };
  float* basis_s = (float*)take(sizeof(float) * a.S * R_);
  uint32_t* spk_list = (uint32_t*)take(sizeof(uint32_t) * B_ * NT);
  int* s_cnt = (int*)take(sizeof(int) * 2 * nb);
  // [1] abort, [2],[3] spike counts by parity, [8 + 2*(s&3)], [9 + 2*(s&3)] bounds of the LGN events of step s
  int* s_misc = (int*)take(sizeof(int) * 16);
  int2* rowb_s = (int2*)take(sizeof(int2) * NT);   // [first, end) of each neuron's out-synapses
  uint4* lgn_ent_s = (uint4*)take(sizeof(uint4) * 2 * NW);  // per warp: its first LGN event of the next two steps
  uint2* bk_s = (uint2*)take(sizeof(uint2) * a.bkg_cap);  // (pre | sid << 24, weight bits)
  float* pr_s = (float*)take(sizeof(float) * B_ * R_ * NT) + tid;  // [b][r][tid]
#define PR(b, r) pr_s[((b)*R_ + (r)) * NT]

  for (int i = tid; i < a.S * R_; i += NT) basis_s[i] = a.basis[i];
  const int bk_base = a.bkg_inptr[n0];
  {
    const int m = a.bkg_inptr[n0 + cn] - bk_base;
    for (int j = tid; j < m; j += NT)
      bk_s[j] = make_uint2((uint32_t)a.bkg_inpre[bk_base + j] | ((uint32_t)a.bkg_insid[bk_base + j] << 24),
                           __float_as_uint(a.bkg_w[bk_base + j]));
  }
  const int bj0 = active ? a.bkg_inptr[n] - bk_base : 0;
  const int bj1 = active ? a.bkg_inptr[n + 1] - bk_base : 0;
  const float k_decay = a.decay[n], k_cf = a.cf[n];
  const float k_ad0 = a.asc_decay[2 * n], k_ad1 = a.asc_decay[2 * n + 1];
  const float k_am0 = a.asc_amps[2 * n], k_am1 = a.asc_amps[2 * n + 1];
  const int k_tref = a.tref[n];

  // ---- state in registers ----
  float v[B_], a0[B_], a1[B_], p[B_][R_];
  unsigned rh[B_];  // bits 0..7 spike history (bit d-1 = spiked d steps ago), bits 8..15 refractory
  const bool have_state = a.st.v != nullptr;
#pragma unroll
  for (int b = 0; b < B_; ++b) {
    v[b] = a0[b] = a1[b] = 0.f;
    rh[b] = 0;
#pragma unroll
    for (int r = 0; r < R_; ++r) {
      p[b][r] = 0.f;
      PR(b, r) = 0.f;
    }
    if (have_state && active) {
      const int64_t g = (int64_t)b * N + n;
      v[b] = a.st.v[g];
      a0[b] = a.st.asc[2 * g];
      a1[b] = a.st.asc[2 * g + 1];
#pragma unroll
      for (int r = 0; r < R_; ++r) {
        p[b][r] = a.st.psc[g * R_ + r];
        PR(b, r) = a.st.psc_rise[g * R_ + r];
      }
      unsigned hist = 0;
      for (int d = 0; d < D; ++d)
        if (a.st.z_buf[((int64_t)b * D + d) * N + n] > 0.f) hist |= 1u << d;
      rh[b] = hist | ((unsigned)(uint8_t)a.st.r[g] << 8);
    }
  }
  if (tid < 16) s_misc[tid] = 0;
  rowb_s[tid] = active ? make_int2(a.rec_rowptr[(int64_t)n * D], a.rec_rowptr[(int64_t)n * D + D]) : make_int2(0, 0);
  __syncthreads();

  unsigned long long c_spikes = 0, c_rec_ev = 0, c_lgn_rows = 0, c_lgn_ev = 0, c_bkg_ev = 0,
                     c_bkg_rows = 0;
  // LGN events are dealt out over the grid's warps block by block (event i to block i mod grid), the
  // last warps of a block first: numbered block-major, the few hundred events of a step all fell on
  // the first third of the blocks, which then set the pace of every step
  const int gw = (NW - 1 - warp) * gridDim.x + blockIdx.x, gnw = gridDim.x * NW;

  // ---- prologue: pending deliveries of the initial spike buffer, LGN events of step 0 ----
  if (have_state) {
    // every warp walks the pending spikes of its own lanes, one lane at a time
#pragma unroll
    for (int b = 0; b < B_; ++b) {
      for (int d = 0; d < D; ++d) {
        unsigned m = __ballot_sync(0xffffffffu, active && (rh[b] & (1u << d)));
        while (m) {
          const int src = __ffs(m) - 1;
          m &= m - 1;
          v1g_walk_rec<R_>(a, basis_s, lane, b, a.rec_rowptr + (int64_t)(n0 + warp * 32 + src) * D,
                           -(d + 1), c_rec_ev);
        }
      }
    }
  }
  if (a.T > 0)
    v1g_scatter_lgn<R_>(a, basis_s, lane, gw, gnw, v1g_lgn_begin(a, 0), v1g_lgn_begin(a, 1), 0, c_lgn_rows, c_lgn_ev);
  // LGN hand-over: the bounds of the events of steps 1 and 2, and every warp's first event of step 1
  const bool lgn8 = a.lgn_syn8 != nullptr;
  if (tid == 0) {
    for (int s = 1; s <= 2; ++s) {
      s_misc[8 + 2 * (s & 3)] = s < a.T ? v1g_lgn_begin(a, s) : 0;
      s_misc[9 + 2 * (s & 3)] = s < a.T ? v1g_lgn_begin(a, s + 1) : 0;
    }
  }
  if (lane == 0) {
    uint4 ent = make_uint4(0u, 0u, 0u, 0u);
    if (a.T > 1) {
      const int e = v1g_lgn_begin(a, 1) + gw;
      if (e < v1g_lgn_begin(a, 2)) ent = a.lgn_ent4[e];
    }
    lgn_ent_s[(1 & 1) * NW + warp] = ent;
  }
  __syncthreads();
  if (tid == 0) v1g_arrive(v1g_phase_counter(a.barrier, 0));

  const unsigned hist_mask = (1u << D) - 1u;
  const unsigned long long G = gridDim.x;
  unsigned long long ph_dense = 0, ph_scatter = 0, ph_barrier = 0;
  const bool prof = a.phase_ns != nullptr && tid == 0;
  const unsigned long long ph_start = prof ? gtime() : 0;
  unsigned long long seen = 0;
  bool ok = true;

  // background input of one batch row of this neuron: sum over its in-synapses of
  // (w * count) * basis[sid, :] (models.py:890-934 in post-major form)
  unsigned c_bkg32 = 0;  // delivered background events of this thread (widened at the end)
  auto bkg_gather = [&](int b, const int* cnt_s, float (&Gs)[R_]) {
#pragma unroll
    for (int r = 0; r < R_; ++r) Gs[r] = 0.f;
    // branch-free: a zero count adds +0 to every channel, which leaves the sums unchanged
    for (int j = bj0; j < bj1; ++j) {
      const uint2 e = bk_s[j];
      const int cnt = cnt_s[b * a.n_bkg + (int)(e.x & 0xffffffu)];
      const float wc = __uint_as_float(e.y) * (float)cnt;
      const float* bs = basis_s + (e.x >> 24) * R_;
#pragma unroll
      for (int r = 0; r < R_; ++r) Gs[r] += wc * bs[r];
      c_bkg32 += cnt > 0 ? 1u : 0u;
    }
  };

  for (int t = 0; t < a.T && ok; ++t) {
    const unsigned long long ph0 = prof ? gtime() : 0;
    if (tid == 0 && t >= 2) {
      const unsigned long long target = v1g_phase_target(t - 2, G);
      if (seen < target)
        seen = v1g_wait(v1g_phase_counter(a.barrier, t - 2), target, a.spin_limit, a.status);
      if (seen < target) s_misc[1] = 1;
    }
    __syncthreads();
    if (s_misc[1]) {
      ok = false;
      break;
    }
    if (tid == 0 && t >= 1) v1g_arrive(v1g_phase_counter(a.barrier, t));
    const unsigned long long ph1 = prof ? gtime() : 0;
    const bool consume = t >= 2;
    const int slot = consume ? (t - 2) % K : 0;
    const int* cnt_s = s_cnt + (t & 1) * nb;
    if (t >= 1) {
      // counts of step t-1 for the next iteration, copied asynchronously into the other buffer
      int* cnt_n = s_cnt + ((t + 1) & 1) * nb;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int i = tid + q * NT;
        if (i < nb) {
          const int b = i / a.n_bkg, j = i - b * a.n_bkg;
          cp_async_4(cnt_n + i, a.bkg_counts + ((int64_t)b * a.T + (t - 1)) * a.n_bkg + j);
        }
      }
    }
    if (blockIdx.x == 0 && consume)
      for (int i = tid; i < nb; i += NT) c_bkg_rows += cnt_s[i] > 0 ? 1 : 0;
    int* nspk_p = &s_misc[2 + (t & 1)];

#ifndef V1G_FWD_NO_ROW_PREFETCH
    // the same for the LGN event this warp scatters after the dense phase (fetched an iteration ago)
    if (lane == 0 && lgn8 && t + 1 < a.T) {
      const uint4 ent = lgn_ent_s[((t + 1) & 1) * NW + warp];
      const char* p0 = (const char*)(a.lgn_syn8 + ent.y);
      const char* p1 = (const char*)(a.lgn_syn8 + ent.z);
      for (const char* p = p0; p < p1; p += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
    }
#endif
    // ---------------- dense phase ----------------
    if (active) {
      // ring values of batch row b+1 are requested while row b is processed
      float* rp = a.ring + ((int64_t)slot * B_ * R_) * Np + n;
      float Ic[R_], In_[R_];
      if (consume) {
#pragma unroll
        for (int r = 0; r < R_; ++r) Ic[r] = __ldcg(rp + (int64_t)r * Np);
      }
#pragma unroll
      for (int b = 0; b < B_; ++b) {
        float prv[R_];
#pragma unroll
        for (int r = 0; r < R_; ++r) prv[r] = PR(b, r);
        if (consume) {
          if (b + 1 < B_) {
#pragma unroll
            for (int r = 0; r < R_; ++r) In_[r] = __ldcg(rp + (int64_t)((b + 1) * R_ + r) * Np);
          }
          float Gs[R_];
          bkg_gather(b, cnt_s, Gs);
#pragma unroll
          for (int r = 0; r < R_; ++r) {
            __stcg(rp + (int64_t)(b * R_ + r) * Np, 0.f);
            prv[r] = prv[r] * a.sd[r] + ((Ic[r] + Gs[r]) * a.lr_scale) * a.pinit[r];
            PR(b, r) = prv[r];
            Ic[r] = In_[r];
          }
        }
        float csum = 0.f;
#pragma unroll
        for (int r = 0; r < R_; ++r) {
          if (t >= 1) p[b][r] = p[b][r] * a.sd[r] + a.dtsd[r] * prv[r];
          csum = (r == 0) ? p[b][r] : csum + p[b][r];
        }
        const unsigned hist = rh[b] & 0xffu;
        const float prev_z = (hist & 1u) ? 1.f : 0.f;
        const float c1 = csum + (a0[b] + a1[b]);
        a0[b] = k_ad0 * a0[b] + prev_z * k_am0;
        a1[b] = k_ad1 * a1[b] + prev_z * k_am1;
        const float dv = v[b] * a.vd_keep + v[b] * a.vd_drop;
        float nv = (k_decay * dv + k_cf * c1) - prev_z;
        int nr = (int)(rh[b] >> 8) + ((hist & 1u) ? k_tref : 0) - 1;
        nr = nr > 0 ? nr : 0;
        if (a.hard_reset && nr > 0) nv = 0.f;
        const bool z = ((nv - 1.f) > 0.f) && (nr == 0);
        v[b] = nv;
        rh[b] = (((hist << 1) | (z ? 1u : 0u)) & hist_mask) | ((unsigned)nr << 8);
        const int64_t oi = ((int64_t)b * a.T + t) * N + n;
        if (a.z_out) __stcs(a.z_out + oi, (uint8_t)(z ? 1 : 0));
        if (a.v_out) __stcs(a.v_out + oi, nv);
        if (a.tape_v) {
          const int64_t ti = ((int64_t)t * B_ + b) * N + n;
          // the voltage with its two lowest mantissa bits replaced by (spiked, refractory)
          __stcs(a.tape_v + ti, __uint_as_float((__float_as_uint(nv) & ~3u) | (z ? 1u : 0u) | (nr > 0 ? 2u : 0u)));
        }
        if (z) {
          spk_list[atomicAdd(nspk_p, 1)] = ((uint32_t)b << 24) | (uint32_t)tid;
#ifndef V1G_FWD_NO_ROW_PREFETCH
          // the scatter phase will walk this neuron's out-synapses: ask L2 for their records now, so that
          // they are on their way from HBM while the rest of the dense phase runs
          if (a.rec_syn8) {
            const int2 rb = rowb_s[tid];
            const char* p0 = (const char*)(a.rec_syn8 + rb.x);
            const char* p1 = (const char*)(a.rec_syn8 + rb.y);
            for (const char* p = p0; p < p1; p += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
          }
#endif
        }
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    const unsigned long long ph2 = prof ? gtime() : 0;
    // ---------------- scatter phase ----------------
    if (tid == 0) {
      seen = (t >= 1) ? v1g_ld_acquire(v1g_phase_counter(a.barrier, t - 1)) : 0;
      s_misc[2 + ((t + 1) & 1)] = 0;
    }
    const int nspk = *nspk_p;
    for (int e = warp; e < nspk; e += NW) {
      const uint32_t ent = spk_list[e];
      if (a.stat_neuron && lane == 0) {
        atomicAdd(a.stat_neuron + n0 + (int)(ent & 0xffffffu), 1);
        atomicAdd(a.stat_pop + t * B_ + (int)(ent >> 24), 1);
      }
      if (a.rec_syn8) {
        const int2 rb = rowb_s[ent & 0xffffffu];
        v1g_scatter_row8<R_>(a, a.rec_syn8, basis_s, lane, (int)(ent >> 24), rb.x, rb.y, t % K, true);
        if (lane == 0) c_rec_ev += (unsigned long long)(rb.y - rb.x);
      } else {
        v1g_walk_rec<R_>(a, basis_s, lane, (int)(ent >> 24),
                         a.rec_rowptr + (int64_t)(n0 + (int)(ent & 0xffffff)) * D, t, c_rec_ev);
      }
    }
    if (tid == 0) c_spikes += (unsigned long long)nspk;
    // LGN events of step t+1.  Dependent loads are spread over iterations and handed over in shared
    // memory: thread 0 fetches the bounds of the events of step t+3, every warp fetches its first
    // event of step t+2 (bounds known since the previous iteration), and what is left for now is
    // event (prefetched, with the bounds of its synapse row) -> synapse records -> atomics.
    // (asynchronous copies straight into shared memory: no register holds a value in flight)
    if (tid == 0) {
      int* bd = &s_misc[8 + 2 * ((t + 3) & 3)];
      if (t + 3 < a.T) {
        const int64_t spt = (int64_t)a.B * a.lgn_nseg;
        cp_async_4(bd, a.lgn_off + (int64_t)(t + 3) * spt);
        cp_async_4(bd + 1, a.lgn_off + (int64_t)(t + 4) * spt);
      } else {
        bd[0] = bd[1] = 0;
      }
    }
    if (lane == 0) {
      uint4* dst = &lgn_ent_s[(t & 1) * NW + warp];  // read in the next iteration (step t+2)
      const int e = s_misc[8 + 2 * ((t + 2) & 3)] + gw;
      if (t + 2 < a.T && e < s_misc[9 + 2 * ((t + 2) & 3)])
        cp_async_16(dst, a.lgn_ent4 + e);
      else
        *dst = make_uint4(0u, 0u, 0u, 0u);
    }
    if (t + 1 < a.T) {
      const int slot1 = (t + 1) % K;
      const int e0 = s_misc[8 + 2 * ((t + 1) & 3)], e1 = s_misc[9 + 2 * ((t + 1) & 3)];
      if (lgn8) {
        uint4 ent = lgn_ent_s[((t + 1) & 1) * NW + warp];
        ent.x = __shfl_sync(0xffffffffu, ent.x, 0);
        ent.y = __shfl_sync(0xffffffffu, ent.y, 0);
        ent.z = __shfl_sync(0xffffffffu, ent.z, 0);
        for (int e = e0 + gw; e < e1; e += gnw) {
          if (e != e0 + gw) ent = a.lgn_ent4[e];  // more events than warps in the grid
          v1g_scatter_row8<R_>(a, a.lgn_syn8, basis_s, lane, (int)(ent.x >> 24), (int)ent.y, (int)ent.z, slot1, false);
          if (lane == 0) {
            c_lgn_rows += 1;
            c_lgn_ev += (unsigned long long)(ent.z - ent.y);
          }
        }
      } else {
        v1g_scatter_lgn<R_>(a, basis_s, lane, gw, gnw, e0, e1, slot1, c_lgn_rows, c_lgn_ev);
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");  // own copies landed; the barrier at the top of the next iteration publishes them
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
    for (int s = max(a.T - 2, 0); s < a.T; ++s) {
      __syncthreads();
      for (int i = tid; i < nb; i += NT) {
        const int b = i / a.n_bkg, j = i - b * a.n_bkg;
        s_cnt[i] = a.bkg_counts[((int64_t)b * a.T + s) * a.n_bkg + j];
      }
      __syncthreads();
      if (blockIdx.x == 0)
        for (int i = tid; i < nb; i += NT) c_bkg_rows += s_cnt[i] > 0 ? 1 : 0;
      if (active) {
        float* rp = a.ring + ((int64_t)(s % K) * B_ * R_) * Np + n;
#pragma unroll
        for (int b = 0; b < B_; ++b) {
          float Gs[R_];
          bkg_gather(b, s_cnt, Gs);
#pragma unroll
          for (int r = 0; r < R_; ++r) {
            const float in = __ldcg(rp + (int64_t)(b * R_ + r) * Np);
            __stcg(rp + (int64_t)(b * R_ + r) * Np, 0.f);
            const float prv = PR(b, r);
            if (s == a.T - 1) p[b][r] = p[b][r] * a.sd[r] + a.dtsd[r] * prv;
            PR(b, r) = prv * a.sd[r] + ((in + Gs[r]) * a.lr_scale) * a.pinit[r];
          }
        }
      }
    }
  }
  if (prof) {
    unsigned long long* o = a.phase_ns + 4 * blockIdx.x;
    o[0] = ph_dense;
    o[1] = ph_scatter;
    o[2] = ph_barrier;
    o[3] = gtime() - ph_start;
  }
  if (have_state && ok && active) {
#pragma unroll
    for (int b = 0; b < B_; ++b) {
      const int64_t g = (int64_t)b * N + n;
      a.st.v[g] = v[b];
      a.st.r[g] = (int8_t)(rh[b] >> 8);
      a.st.asc[2 * g] = a0[b];
      a.st.asc[2 * g + 1] = a1[b];
#pragma unroll
      for (int r = 0; r < R_; ++r) {
        a.st.psc[g * R_ + r] = p[b][r];
        a.st.psc_rise[g * R_ + r] = PR(b, r);
      }
      for (int d = 0; d < D; ++d) a.st.z_buf[((int64_t)b * D + d) * N + n] = (rh[b] >> d) & 1u ? 1.f : 0.f;
    }
  }
  c_rec_ev = v1g_warp_sum(c_rec_ev);
  c_lgn_rows = v1g_warp_sum(c_lgn_rows);
  c_lgn_ev = v1g_warp_sum(c_lgn_ev);
  c_bkg_ev = v1g_warp_sum(c_bkg_ev + (unsigned long long)c_bkg32);
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

template <int R_, int B_>
int launch(V1GHandle* h, const FwdArgs& a, int grid, size_t smem, cudaStream_t st) {
  auto kern = rollout_fwd_reg_kernel<R_, B_>;
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

template <int R_>
int launch_b(V1GHandle* h, const FwdArgs& a, int grid, size_t smem, cudaStream_t st) {
  switch (a.B) {
    case 1: return launch<R_, 1>(h, a, grid, smem, st);
    case 2: return launch<R_, 2>(h, a, grid, smem, st);
    case 3: return launch<R_, 3>(h, a, grid, smem, st);
    case 4: return launch<R_, 4>(h, a, grid, smem, st);
    case 5: return launch<R_, 5>(h, a, grid, smem, st);
    case 6: return launch<R_, 6>(h, a, grid, smem, st);
    default: return V1G_ERANGE;
  }
}

}  // namespace

size_t v1g_fwd_reg_smem(const V1GHandle* h, int B, int chunkP, int bkg_cap) {
  auto al = [](size_t b) { return (b + 15) & ~(size_t)15; };
  const V1GConfig& c = h->cfg;
  return al(sizeof(float) * c.n_syn_types * c.n_receptors) + al(sizeof(uint32_t) * B * NT) +
         al(sizeof(int) * 2 * B * c.n_bkg) + al(sizeof(int) * 16) + al(sizeof(int2) * NT) + al(sizeof(uint4) * 2 * NW) +
         al(sizeof(uint2) * bkg_cap) +
         al(sizeof(float) * B * c.n_receptors * NT);
}

int v1g_launch_fwd_reg(V1GHandle* h, const FwdArgs& a, int R, int grid, size_t smem,
                       cudaStream_t st) {
  if (R == 4) return launch_b<4>(h, a, grid, smem, st);
  if (R == 5) return launch_b<5>(h, a, grid, smem, st);
  return V1G_ERANGE;
}
