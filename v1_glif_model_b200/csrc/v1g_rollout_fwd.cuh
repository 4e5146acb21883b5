// Argument block and device helpers shared by the two forward rollout kernels.
#pragma once

#include "v1g_rollout_common.cuh"

struct FwdArgs {
  int N, D, K, B, T, Np, chunk, chunkP, S, n_bkg;
  int state_in_smem, bkg_in_smem, bkg_cap;
  // connectivity
  const int32_t *rec_rowptr, *rec_post;
  const float* rec_w;
  const uint8_t* rec_sid;
  const int32_t *lgn_rowptr, *lgn_post;
  const float* lgn_w;
  const uint8_t* lgn_sid;
  const int32_t *bkg_inptr, *bkg_inpre;
  const float* bkg_w;
  const uint8_t* bkg_insid;
  // neuron constants
  const float *decay, *cf, *asc_decay, *asc_amps, *basis;
  const int32_t* tref;
  float sd[V1G_MAX_RECEPTORS], pinit[V1G_MAX_RECEPTORS], dtsd[V1G_MAX_RECEPTORS];
  float lr_scale, vd_keep, vd_drop;
  int hard_reset;
  // inputs
  const int32_t* lgn_off;  // exclusive offsets per (t, b, seg) segment
  const uint32_t* lgn_entries;
  int lgn_nseg;
  const int32_t* bkg_counts;  // [B][T][n_bkg]
  // state (reference layouts, all NULL = zero state / no write-back)
  V1GState st;
  float* state_ws;
  // outputs
  uint8_t* z_out;
  float* v_out;
  float* tape_v;
  uint8_t* tape_zr;
  // plumbing
  float* ring;
  unsigned long long* barrier;
  int32_t* status;
  unsigned long long* counters;
  long long spin_limit;
  unsigned long long* phase_ns;  // optional [grid][4]: dense, scatter, barrier, total (ns)
};


__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}


// Walk the D contiguous delay buckets of neuron n's CSR row for a spike of batch row b emitted
// at step te (te < 0: pending spike of the initial z_buf) and add w*basis[sid,:] of every synapse
// with delay d into ring slot (te+d) mod K; deliveries before step 0 are dropped.  One warp.
// `rowp` points at the D+1 row pointers of the neuron (global memory or a shared-memory copy).
template <int R_>
__device__ __forceinline__ void v1g_walk_rec(const FwdArgs& a, const float* basis_s, int lane,
                                             int b, const int32_t* rowp, int te,
                                             unsigned long long& events) {
  const int D = a.D, K = a.K;
  int rp = 0;
  if (lane <= D) rp = rowp[lane];
  int bound[V1G_MAX_DELAY + 1];
#pragma unroll
  for (int d = 0; d <= V1G_MAX_DELAY; ++d) bound[d] = __shfl_sync(0xffffffffu, rp, d <= D ? d : 0);
  const int j0 = bound[0], j1 = __shfl_sync(0xffffffffu, rp, D);
  const int tk = ((te % K) + K) % K;
  for (int j = j0 + lane; j < j1; j += 32) {
    int d = 1;
#pragma unroll
    for (int q = 1; q < V1G_MAX_DELAY; ++q) d += (q < D && j >= bound[q]) ? 1 : 0;
    if (te + d < 0) continue;
    int slot = tk + d;
    if (slot >= K) slot -= K;
    const float wv = a.rec_w[j];
    const float* bs = basis_s + (int)a.rec_sid[j] * R_;
    float* dst = a.ring + ((int64_t)(slot * a.B + b) * R_) * a.Np + a.rec_post[j];
#pragma unroll
    for (int r = 0; r < R_; ++r) {
      const float c = wv * bs[r];
      if (c != 0.f) atomicAdd(dst + (int64_t)r * a.Np, c);
    }
  }
  if (lane == 0) events += (unsigned long long)(j1 - j0);
}

// LGN events of step tt into ring slot tt mod K; the list is shared by all warps of the grid
// (gw = global warp index, gnw = warps in the grid).
template <int R_>
__device__ __forceinline__ void v1g_scatter_lgn(const FwdArgs& a, const float* basis_s, int lane,
                                                int gw, int gnw, int tt, unsigned long long& rows,
                                                unsigned long long& events) {
  const int seg_per_t = a.B * a.lgn_nseg;
  const int e0 = a.lgn_off[(int64_t)tt * seg_per_t], e1 = a.lgn_off[(int64_t)(tt + 1) * seg_per_t];
  const int slot = tt % a.K;
  for (int e = e0 + gw; e < e1; e += gnw) {
    const uint32_t ent = a.lgn_entries[e];
    const int b = ent >> 24, u = ent & 0xffffff;
    const int j0 = a.lgn_rowptr[u], j1 = a.lgn_rowptr[u + 1];
    for (int j = j0 + lane; j < j1; j += 32) {
      const float wv = a.lgn_w[j];
      const float* bs = basis_s + (int)a.lgn_sid[j] * R_;
      float* dst = a.ring + ((int64_t)(slot * a.B + b) * R_) * a.Np + a.lgn_post[j];
#pragma unroll
      for (int r = 0; r < R_; ++r) {
        const float c = wv * bs[r];
        if (c != 0.f) atomicAdd(dst + (int64_t)r * a.Np, c);
      }
    }
    if (lane == 0) {
      rows += 1;
      events += (unsigned long long)(j1 - j0);
    }
  }
}

// Register-resident variant (one thread per neuron, batch unrolled); V1G_ERANGE when the
// (receptors, batch) pair has no instantiation or the slice does not fit.
int v1g_launch_fwd_reg(V1GHandle* h, const FwdArgs& a, int R, int grid, size_t smem,
                       cudaStream_t st);
size_t v1g_fwd_reg_smem(const V1GHandle* h, int B, int chunkP, int bkg_cap);
constexpr int V1G_NT_REG = 512;
