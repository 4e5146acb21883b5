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
  const uint4* lgn_ent4;  // {batch row << 24 | unit, first synapse, end, 0} per event
  // packed synapse records {post | sid << 22 | (delay-1) << 29, weight bits}, or NULL
  const uint2 *rec_syn8, *lgn_syn8;
  int lgn_nseg;
  const int32_t* bkg_counts;  // [B][T][n_bkg]
  // spike statistics for the loss terms (with the tape, else NULL): spikes per neuron, population
  // spikes per (step, batch row)
  int32_t *stat_neuron, *stat_pop;
  // first neuron of every block's slice [grid + 1] (register-resident kernel), or NULL for equal slices
  const int32_t* slice;
  // state (reference layouts, all NULL = zero state / no write-back)
  V1GState st;
  float* state_ws;
  // outputs
  uint8_t* z_out;
  float* v_out;
  float* tape_v;
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

// first event of step tt in the time-major LGN list (tt = T gives the end of the list)
__device__ __forceinline__ int v1g_lgn_begin(const FwdArgs& a, int tt) {
  return a.lgn_off[(int64_t)tt * a.B * a.lgn_nseg];
}

// LGN events [e0, e1) of one step into ring slot `slot`; the list is shared by all warps of the grid
// (gw = global warp index, gnw = warps in the grid).  Each event carries the bounds of its row.
template <int R_>
__device__ __forceinline__ void v1g_scatter_lgn(const FwdArgs& a, const float* basis_s, int lane,
                                                int gw, int gnw, int e0, int e1, int slot,
                                                unsigned long long& rows, unsigned long long& events) {
  constexpr int UL = 3;  // 32-synapse groups whose loads are in flight together
  for (int e = e0 + gw; e < e1; e += gnw) {
    const uint4 ent = a.lgn_ent4[e];
    const int b = ent.x >> 24;
    const int j0 = (int)ent.y, j1 = (int)ent.z;
    float* const ring_b = a.ring + ((int64_t)(slot * a.B + b) * R_) * a.Np;
    for (int jb = j0; jb < j1; jb += 32 * UL) {
      float wv[UL];
      int sid[UL], post[UL];
#pragma unroll
      for (int q = 0; q < UL; ++q) {
        const int j = jb + q * 32 + lane;
        const bool in = j < j1;
        wv[q] = in ? a.lgn_w[j] : 0.f;
        sid[q] = in ? (int)a.lgn_sid[j] : 0;
        post[q] = in ? a.lgn_post[j] : 0;
      }
#pragma unroll
      for (int q = 0; q < UL; ++q) {
        const float* bs = basis_s + sid[q] * R_;
        float* dst = ring_b + post[q];
#pragma unroll
        for (int r = 0; r < R_; ++r) {
          const float c = wv[q] * bs[r];
          if (c != 0.f) atomicAdd(dst + (int64_t)r * a.Np, c);
        }
      }
    }
    if (lane == 0) {
      rows += 1;
      events += (unsigned long long)(j1 - j0);
    }
  }
}

// Packed-record form of the two walks above: one 8-byte load per synapse, the (up to 128) synapses
// of a pass requested together, so that a warp pays one memory latency per pass before its atomics.
// Synapses [j0, j1) of one source row; te = step of emission (delay from the record), slot0 = ring
// slot of step te.
template <int R_>
__device__ __forceinline__ void v1g_scatter_row8(const FwdArgs& a, const uint2* __restrict__ syn8,
                                                 const float* basis_s, int lane, int b, int j0, int j1,
                                                 int slot0, bool delayed) {
  constexpr int UL = 4;
  const int K = a.K;
  for (int jb = j0; jb < j1; jb += 32 * UL) {
    uint2 rec[UL];
#pragma unroll
    for (int q = 0; q < UL; ++q) {
      const int j = jb + q * 32 + lane;
      rec[q] = j < j1 ? __ldg(syn8 + j) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int q = 0; q < UL; ++q) {
      const unsigned x = rec[q].x;
      const float wv = __uint_as_float(rec[q].y);  // zero for the lanes past the end of the row
      int slot = slot0 + (delayed ? (int)(x >> 29) + 1 : 0);
      if (slot >= K) slot -= K;
      const float* bs = basis_s + ((x >> 22) & 127u) * R_;
      float* dst = a.ring + ((int64_t)(slot * a.B + b) * R_) * a.Np + (x & 0x3fffffu);
#pragma unroll
      for (int r = 0; r < R_; ++r) {
        const float c = wv * bs[r];
        if (c != 0.f) atomicAdd(dst + (int64_t)r * a.Np, c);
      }
    }
  }
}

// Register-resident variant (one thread per neuron, batch unrolled); V1G_ERANGE when the
// (receptors, batch) pair has no instantiation or the slice does not fit.
int v1g_launch_fwd_reg(V1GHandle* h, const FwdArgs& a, int R, int grid, size_t smem,
                       cudaStream_t st);
size_t v1g_fwd_reg_smem(const V1GHandle* h, int B, int chunkP, int bkg_cap);
constexpr int V1G_NT_REG = 512;
