// Fused backward rollout (BPTT): the reverse sweep over the T steps saved by v1g_rollout_fwd, in
// ONE persistent cooperative kernel with the same neuron slicing as the forward kernels.
//
// Adjoint recursion (g_* = dL/d(state after step t); reference: the custom gradients at
// models.py:58-64, 174-261 and the stop-gradients / straight-through factors at :994, 1010-1018,
// 1081), processed for t = T-1 .. 0:
//   g_z   = dl/dz(t) + rec_factor * sum over the out-synapses j of neuron n (delay d_j) of
//           w_j * sum_r basis[sid_j, r] * dy(t + d_j)[b, post_j, r]
//   g_v'  = dl/dv(t) + g_v + [r(t) == 0] * g_z * pseudo(v(t) - 1)        (hard reset: 0 if r(t) > 0)
//   g_v  <- decay * (1 - d_v) * g_v'              g_asc_k <- asc_decay_k * g_asc_k + cf * g_v'
//   g_p  <- sd * g_p + cf * g_v'                  g_pr   <- sd * g_pr + dt * sd * g_p(old)
//   dy(t)[b, n, r] = lr_scale * psc_initial_r * g_pr(t)
//   dW_rec[j] += sum_b z(t)[b, n] * sum_r basis[sid_j, r] * dy(t + d_j)[b, post_j, r]   (no dampening)
//   dW_lgn[j] += sum_b x(t)[b, pre_j] * (same with dy(t))      dW_bkg[j] += sum_b count(t)[b, pre_j] * (...)
//
// dy(t) only depends on g_pr(t+1) and g_p(t+1), which are final once step t+2 has been processed,
// so the block that owns neuron n publishes dy(t-2) while it processes step t.  A block at step t
// reads dy(t+1 .. t+D) of arbitrary neurons, i.e. values published at steps >= t+3: like the
// forward sweep, blocks synchronise through a lagged per-phase counter and rarely wait.
//
// What is published is Q, a ring over K = D+3 steps with a 16- or 32-byte row per (neuron, channel):
//   projected mode (S <= 8 synapse types): Q[slot][n][s][b] = sum_r basis[s, r] * dy[b, n, r]; a
//       synapse then needs ONE sector, Q[slot][post][sid][0..B)
//   raw mode: Q[slot][n][r][b] = dy[b, n, r]; the consumer contracts with basis[sid, :] (R sectors)
// The gather walks every neuron's CSR row (all synapses, every step: the pseudo-derivative is
// non-zero for non-spiking neurons), one warp per row, except rows whose B batch entries are all
// refractory / outside the pseudo-derivative's support and did not spike (exactly zero result).
//
// Paired mode (option "pair_rows"; 16-byte rows, projected, packed synapse records, at most one neuron
// per thread): the ring is laid out in PAIRS of steps, {Q(tau), Q(tau-1)} for even tau in one 32-byte
// row (one sector), and a synapse of delay d >= 2 reads one pair to serve the steps s and s-1 at once:
// Q(s+d) and Q(s-1+d), which costs the L2 one request instead of two.  The
// iteration whose dense part handles step t serves the steps (t-1, t-2) for the delays d >= 2 with
// t-1+d even - the other delay parity has its turn in the next iteration - and step t-1 alone for
// the synapses of delay 1, whose Q(t-1) for step t-2 is not complete yet (it is published by the
// slowest block during this very iteration; waiting for it would need a hard grid barrier).
// Everything read was published at least two iterations earlier, as in the unpaired loop, so the
// lagged counters are unchanged.  Requests per reverse step: 0.2 + 0.8 / 2 of the unpaired count for
// uniform delays 1..5.  Measured on B200 (66,634 neurons, batch 5, T=150, one launch each): L2 read
// requests 645 M -> 400 M, the L1-to-L2 request port 52 % -> 33 % busy and the L1 data pipe
// 55 % -> 47 %, but 2.65 G instead of 2.20 G warp instructions (two steps' values to unpack and
// accumulate per entry, a second warp reduction per row): 4.59 ms against 4.49 ms, and 40.3 against
// 39.3 us per reverse step at T=500 (gather 26.7 against 28.8 us, tape phase 5.0 against 3.3 us).
// The unpaired loop therefore stays the default: neither loop is bound by the request count; both
// spend most of a turn of the software pipeline waiting on its dependent chain (queue pop, row
// descriptor, records, Q rows, warp reduction), of which a warp runs one per row.
#include <algorithm>
#include <type_traits>

#include "v1g_rollout_common.cuh"

namespace {

struct BwdArgs {
  int N, D, K, B, T, Np, chunk, chunkP, S, C, n_bkg, state_in_smem, bkg_in_smem, bkg_cap;
  int KP;  // paired mode: ring slots, each holding the steps (2p, 2p-1)
  // paired mode: per delay parity p the synapse records of a neuron in gather order (delay-1 bucket,
  // then the buckets of delay d >= 2 with d - 1 == 1 + p mod 2), row starts, and CSR position of every entry
  const int32_t* pair_ptr[2];
  const uint2* pair_rec[2];
  const int32_t* pair_j[2];
  int pair_last[2];  // last valid index of each record array (clamp for lanes past a row's end)
  const int32_t *rec_rowptr, *rec_post;
  const float* rec_w;
  const uint8_t* rec_sid;
  int rec_nnz;
  const uint2* rec_syn8;  // packed records {post | sid << 22 | (delay-1) << 29, weight bits}, or NULL
  const int32_t *lgn_rowptr, *lgn_post;
  const uint8_t* lgn_sid;
  const int32_t *bkg_inptr, *bkg_inpre;
  const uint8_t* bkg_insid;
  const float *decay, *cf, *asc_decay, *basis;
  float sd[V1G_MAX_RECEPTORS], pinit[V1G_MAX_RECEPTORS], dtsd[V1G_MAX_RECEPTORS];
  float lr_scale, vd_keep, rec_factor, damp, inv_width, gauss_std;
  int gauss, hard_reset, csr_evict_first;
  // saved forward
  const float* tape_v;
  const uint8_t* hist0;  // initial spike-history bits [B][N], or NULL for a zero initial state
  const int32_t* lgn_off;
  const uint4* lgn_ent4;  // {batch row << 24 | unit, first synapse, end, 0} per event
  int lgn_nseg;
  const int32_t* bkg_counts;
  // loss
  const float* rate_coef;  // [N] dL/dz contribution of the rate term, or NULL
  int rate_t0, rate_t1;    // steps whose spikes enter the rate term
  V1GSyncTables sync;      // synchrony target over given samples (first == NULL: off)
  const float* osi_coef;   // [B][N] dL/dz of the OSI/DSI target inside [osi_t0, osi_t1), or NULL
  int osi_t0, osi_t1;
  const float* sgrad;      // [B][nbins] dL/d(bin count), or NULL
  int sync_bin, nbins;
  float volt_coef;  // voltage_cost * loss_scale / (B*T*N); gradient is 2*volt_coef*(...)
  int volt_threshold_mode;
  const float* v_lo;
  const float *g_z, *g_v;  // explicit [B,T,N] gradients, nullable
  // outputs (accumulated)
  float *dw_rec, *dw_lgn, *dw_bkg;  // CSR order, CSR order, gather-table order
  float* loss_acc;                  // [4]; [2] += voltage loss
  // plumbing
  float* Q;
  float* state_ws;
  unsigned long long* barrier;
  int32_t* status;
  unsigned long long* counters;
  long long spin_limit;
  unsigned long long* phase_ns;
};

#ifndef V1G_BWD_NT
#define V1G_BWD_NT 512
#endif
#ifndef V1G_BWD_GROUPS
#define V1G_BWD_GROUPS 4  // 32-synapse groups of a gather pass with 16-byte Q rows (3, 5, 6 measured slower)
#endif
#ifndef V1G_BWD_STAGES
#define V1G_BWD_STAGES 2  // Q-row buffers of the gather pipeline (registers: 20 per stage)
#endif
// Raw-mode gather (more than 8 synapse types, 4 channels in 16-byte rows): lanes that share a synapse
// and 32-lane groups per pass.  Measured on B200 (66,634 neurons, batch 5, the reference's 121 x 4
// basis, us per reverse step): 4 lanes x 4 groups 65.2, 2 lanes (two channels each, one 256-bit load)
// x 2 groups 61.0, x 3 groups 56.8, x 4 groups 65.9 (spills), 1 lane x 1 group 71.6; the gather over
// plain arrays that this path replaced 111.
#ifndef V1G_BWD_RAW_LANES
#define V1G_BWD_RAW_LANES 2
#endif
#ifndef V1G_BWD_RAW_GROUPS
#define V1G_BWD_RAW_GROUPS 3
#endif
#ifndef V1G_BWD_PAIR_GROUPS
#define V1G_BWD_PAIR_GROUPS 3  // 32-entry groups of a pass of the paired gather (32-byte rows)
#endif
constexpr int NT = V1G_BWD_NT;
constexpr int NW = NT / 32;
constexpr int BAR_TID = NT - 32;  // the thread that talks to the grid-wide phase counters

__device__ __forceinline__ unsigned long long gtime_b() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ float pseudo_h(float vs, const BwdArgs& a) {
  if (a.gauss) return expf(-(vs * vs) / (a.gauss_std * a.gauss_std)) * a.damp;
  float x = fabsf(vs);
  x = x * a.inv_width;
  return a.damp * fmaxf(1.f - x, 0.f);
}

// A Q row holds the values of all batch rows for one (neuron, channel): BP_ fp32 words, or - for a
// batch of exactly 5 - five 24-bit floats (sign, 8 exponent, 15 mantissa bits, round to nearest
// even: 7.6e-6 relative) packed into four words, which keeps the row at 16 bytes and the whole
// ring at half the size, inside L2.
__device__ __forceinline__ unsigned f24(float x) {
  unsigned u = __float_as_uint(x);
  u += 0x7fu + ((u >> 8) & 1u);
  return u >> 8;
}

__device__ __forceinline__ float4 pack_row5(const float (&v)[8]) {
  const unsigned r0 = f24(v[0]), r1 = f24(v[1]), r2 = f24(v[2]), r3 = f24(v[3]), r4 = f24(v[4]);
  uint4 w;
  w.x = r0 | (r1 << 24);
  w.y = (r1 >> 8) | (r2 << 16);
  w.z = (r2 >> 16) | (r3 << 8);
  w.w = r4;
  return make_float4(__uint_as_float(w.x), __uint_as_float(w.y), __uint_as_float(w.z), __uint_as_float(w.w));
}

// the 16-byte words of a Q row -> its BP_ batch values
template <int BP_, bool PACK>
__device__ __forceinline__ void unpack_row(const float4 (&raw)[PACK ? 1 : BP_ / 4], float (&q)[BP_]) {
  const float4 a = raw[0];
  if (PACK) {
    const unsigned w0 = __float_as_uint(a.x), w1 = __float_as_uint(a.y), w2 = __float_as_uint(a.z),
                   w3 = __float_as_uint(a.w);
    q[0] = __uint_as_float(w0 << 8);
    q[1] = __uint_as_float(__funnelshift_l(w0, w1, 16) & 0xffffff00u);
    q[2] = __uint_as_float(__funnelshift_l(w1, w2, 24) & 0xffffff00u);
    q[3] = __uint_as_float(w2 & 0xffffff00u);
    q[4 % BP_] = __uint_as_float(w3 << 8);
#pragma unroll
    for (int b = 5; b < BP_; ++b) q[b] = 0.f;
    return;
  }
  q[0] = a.x; q[1] = a.y; q[2] = a.z; q[3] = a.w;
  if (BP_ == 8) {
    const float4 b = raw[(BP_ / 4 - 1) % (PACK ? 1 : BP_ / 4)];
    q[4 % BP_] = b.x; q[5 % BP_] = b.y; q[6 % BP_] = b.z; q[7 % BP_] = b.w;
  }
}

template <int BP_, bool PACK>
__device__ __forceinline__ void load_row(const float* p, float (&q)[BP_]) {
  float4 raw[PACK ? 1 : BP_ / 4];
#pragma unroll
  for (int v = 0; v < (PACK ? 1 : BP_ / 4); ++v) raw[v] = __ldcg((const float4*)p + v);
  unpack_row<BP_, PACK>(raw, q);
}

// one 32-byte pair row {Q(tau), Q(tau-1)} with a single load instruction
__device__ __forceinline__ void load_pair(const float* p, float4& lo, float4& hi) {
  asm volatile("ld.global.cg.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(lo.x), "=f"(lo.y), "=f"(lo.z), "=f"(lo.w), "=f"(hi.x), "=f"(hi.y), "=f"(hi.z), "=f"(hi.w)
               : "l"(p));
}

// the NB batch values of one 16-byte row: five 24-bit floats (PACK) or four fp32 words
template <int NB, bool PACK>
__device__ __forceinline__ void unpack_half(const float4 a, float (&q)[NB]) {
  if (PACK) {
    const unsigned w0 = __float_as_uint(a.x), w1 = __float_as_uint(a.y), w2 = __float_as_uint(a.z),
                   w3 = __float_as_uint(a.w);
    q[0] = __uint_as_float(w0 << 8);
    q[1 % NB] = __uint_as_float(__funnelshift_l(w0, w1, 16) & 0xffffff00u);
    q[2 % NB] = __uint_as_float(__funnelshift_l(w1, w2, 24) & 0xffffff00u);
    q[3 % NB] = __uint_as_float(w2 & 0xffffff00u);
    q[4 % NB] = __uint_as_float(w3 << 8);
  } else {
    q[0] = a.x; q[1 % NB] = a.y; q[2 % NB] = a.z; q[3 % NB] = a.w;
  }
}

// Sum eight per-lane values over the warp with 9 shuffles (each exchange halves what a lane
// carries); lane l returns the total of value ((l >> 2) & 1) | ((l >> 3) & 1) << 1 | ((l >> 4) & 1) << 2.
__device__ __forceinline__ float warp_reduce8(const float (&v)[8], int lane) {
  float a4[4], a2[2], a1;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const bool hi = lane & 16;
    const float recv = __shfl_xor_sync(0xffffffffu, hi ? v[i] : v[i + 4], 16);
    a4[i] = (hi ? v[i + 4] : v[i]) + recv;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const bool hi = lane & 8;
    const float recv = __shfl_xor_sync(0xffffffffu, hi ? a4[i] : a4[i + 2], 8);
    a2[i] = (hi ? a4[i + 2] : a4[i]) + recv;
  }
  {
    const bool hi = lane & 4;
    const float recv = __shfl_xor_sync(0xffffffffu, hi ? a2[0] : a2[1], 4);
    a1 = (hi ? a2[1] : a2[0]) + recv;
  }
  a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
  a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
  return a1;
}

// Sum two per-lane values over the warp with 5 shuffles; lanes 0..15 return the total of v0,
// lanes 16..31 that of v1.
__device__ __forceinline__ float warp_reduce2(float v0, float v1, int lane) {
  const bool hi = lane & 16;
  float x = (hi ? v1 : v0) + __shfl_xor_sync(0xffffffffu, hi ? v0 : v1, 16);
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

template <int R_, int BP_, bool PROJ, int DT, bool PACK, bool PAIR>
__global__ void __launch_bounds__(NT, 1) rollout_bwd_kernel(const BwdArgs a) {
  constexpr int QW = PACK ? 4 : BP_;       // 32-bit words per Q row
  constexpr int RS = PAIR ? 2 * QW : QW;   // words between the rows of consecutive (neuron, channel) entries
  constexpr int NBX = PACK ? 5 : BP_;      // batch rows the tape and dense loops cover (packed rows: exactly 5)
  static_assert(!PAIR || (PROJ && QW == 4), "paired rows need the projected 16-byte form");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int B = a.B, K = a.K, N = a.N, Np = a.Np, chunkP = a.chunkP, T = a.T, C = a.C;
  const int D = DT > 0 ? DT : a.D;  // delay buckets; a compile-time constant in the common case
  constexpr int DMAX = DT > 0 ? DT : V1G_MAX_DELAY;
  const int n0 = blockIdx.x * a.chunk;
  const int cn = min(a.chunk, N - n0);
  const int nb = B * a.n_bkg;
  // first word of the rows of a step: row (n, c) of that step is at qbase(step) + (n * C + c) * RS
  auto qbase = [&](int step) -> int64_t {
    if (PAIR) return ((int64_t)(((step + 1) >> 1) % a.KP) * Np * C * 2 + (step & 1)) * QW;
    return (int64_t)(step % K) * Np * C * QW;
  };

  const bool fast_rows = a.rec_syn8 != nullptr;  // packed-record gather (in raw mode the host offers it only for R = 4 and 16-byte rows)
  unsigned char* sp_ = smem_raw;
  auto take = [&](size_t bytes) {
    unsigned char* p = sp_;
    sp_ += (bytes + 15) & ~(size_t)15;
    return p;
  };
  const size_t plane = (size_t)B * chunkP;
  float* basis_s = (float*)take(sizeof(float) * a.S * R_);
  // per-step planes [parity of the step][b][k]
  float* gz_s = (float*)take(sizeof(float) * 2 * plane);   // gathered spike gradient
  float* tv_s = (float*)take(sizeof(float) * 2 * plane);   // v(t) (paired mode: the saved word, flags in its low bits)
  uint8_t* tz_s = (uint8_t*)take(PAIR ? 0 : 2 * plane);    // spike / refractory bits
  uint8_t* zmask_s = (uint8_t*)take(PAIR ? 2 * chunkP : chunkP);  // batch rows that spiked at this step (paired mode: walk | mask << 1, by step parity)
  float* s_cnt = (float*)take(sizeof(float) * nb);  // background counts of step t-2, as floats
  int* s_misc = (int*)take(sizeof(int) * 8);  // [1] abort flag, [2+p] rows queued, [4+p] next queue slot (p = parity of the iteration)
  int* slot_s = (int*)take(sizeof(int) * 8);  // first Q row of step t+1+d, d = 0..7
  uint16_t* rowq_s = (uint16_t*)take(PAIR ? 0 : sizeof(uint16_t) * chunkP);  // rows to walk this step
  // the same rows as {first synapse, end, row | spike mask << 16, 0}; paired mode: {first entry, end,
  // row | spike mask(t-1) << 16 | spike mask(t-2) << 21, 0} over the gather-ordered records
  int4* rowd_s = (int4*)take(sizeof(int4) * chunkP);
  // row pointers of the slice: on chip for the gather that reads them per row pass, from global
  // memory (two loads per neuron and step) for the packed-record gathers
  const bool rp_on_chip = !fast_rows;
  int32_t* rp_s = (int32_t*)take(rp_on_chip ? sizeof(int32_t) * ((size_t)chunkP * D + 1) : 0);
  const int32_t* rpx = rp_on_chip ? rp_s : a.rec_rowptr + (int64_t)n0 * D;
  int* bkptr_s = (int*)take(sizeof(int) * (chunkP + 1));  // background in-synapse ranges, slice-relative
  // background in-synapses of the slice and their weight-gradient accumulators; on chip when they
  // fit, otherwise the global tables are used directly
  int* bk_pre_s = nullptr;
  uint8_t* bk_sid_s = nullptr;
  float* bk_dw_s = nullptr;
  if (a.bkg_in_smem) {
    bk_pre_s = (int*)take(sizeof(int) * a.bkg_cap);
    bk_dw_s = (float*)take(sizeof(float) * a.bkg_cap);
    bk_sid_s = (uint8_t*)take(a.bkg_cap);
  }
  float* base;
  if (a.state_in_smem)
    base = (float*)take(sizeof(float) * plane * (3 + 2 * R_));
  else
    base = a.state_ws + (size_t)blockIdx.x * plane * (3 + 2 * R_);
  float* G_v = base;
  float* G_a0 = G_v + plane;
  float* G_a1 = G_a0 + plane;
  float* G_p = G_a1 + plane;       // [r][b][k]
  float* G_pr = G_p + plane * R_;  // [r][b][k]

  for (int i = tid; i < a.S * R_; i += NT) basis_s[i] = a.basis[i];
  if (rp_on_chip)
    for (int i = tid; i <= cn * D; i += NT) rp_s[i] = a.rec_rowptr[(int64_t)n0 * D + i];
  if (PAIR)
    for (int i = tid; i < 2 * chunkP; i += NT) zmask_s[i] = 0;
  const int bk_base = a.bkg_inptr[n0];
  const int bk_m = a.bkg_inptr[n0 + cn] - bk_base;
  for (int k = tid; k <= cn; k += NT) bkptr_s[k] = a.bkg_inptr[n0 + k] - bk_base;
  const int* bk_pre = a.bkg_inpre + bk_base;
  const uint8_t* bk_sid = a.bkg_insid + bk_base;
  float* bk_dw = a.dw_bkg + bk_base;
  if (a.bkg_in_smem) {
    for (int j = tid; j < bk_m; j += NT) {
      bk_pre_s[j] = bk_pre[j];
      bk_sid_s[j] = bk_sid[j];
      bk_dw_s[j] = 0.f;
    }
    bk_pre = bk_pre_s;
    bk_sid = bk_sid_s;
    bk_dw = bk_dw_s;
  }
  for (int i = tid; i < (int)plane * (3 + 2 * R_); i += NT) base[i] = 0.f;
  if (tid < 8) s_misc[tid] = 0;
  __syncthreads();
  if (tid == 0) v1g_arrive(v1g_phase_counter(a.barrier, 0));

  const unsigned long long G = gridDim.x;
  unsigned long long seen = 0;
  bool ok = true;
  float volt_loss = 0.f;
  unsigned long long c_rows = 0, c_events = 0, c_dw = 0;
  unsigned long long ph_a = 0, ph_b = 0, ph_c = 0;
  const bool prof = a.phase_ns != nullptr && tid == 0;
  const unsigned long long ph_start = prof ? gtime_b() : 0;
  // LGN events are dealt out block by block (event i to block i mod grid), so that every block carries
  // its share of a step's few hundred events; first warps first: the last warp watches the barrier
  const int gw = warp * gridDim.x + blockIdx.x, gnw = gridDim.x * NW;

  // Weight gradient of the LGN events of step tt from Q(tt).  One warp per event; the (up to 128)
  // synapses of a pass are loaded together so that the three dependent accesses (record, Q row,
  // atomic) are each paid once per pass.
  auto lgn_dw = [&](int tt) {
    const int seg_per_t = B * a.lgn_nseg;
    const int e0 = a.lgn_off[(int64_t)tt * seg_per_t], e1 = a.lgn_off[(int64_t)(tt + 1) * seg_per_t];
    const float* Qs = a.Q + qbase(tt);
    constexpr int UL = 4;
    for (int e = e0 + gw; e < e1; e += gnw) {
      const uint4 ent = a.lgn_ent4[e];
      const int b = ent.x >> 24;
      const int j0 = (int)ent.y, j1 = (int)ent.z;
      for (int jb = j0; jb < j1; jb += 32 * UL) {
        int post[UL], sid[UL];
#pragma unroll
        for (int q = 0; q < UL; ++q) {
          const int j = jb + q * 32 + lane;
          post[q] = j < j1 ? a.lgn_post[j] : 0;
          sid[q] = j < j1 ? (int)a.lgn_sid[j] : 0;
        }
        float val[UL];
        if (PROJ) {
          float qv[UL][BP_];
#pragma unroll
          for (int q = 0; q < UL; ++q) load_row<BP_, PACK>(Qs + ((int64_t)post[q] * C + sid[q]) * RS, qv[q]);
#pragma unroll
          for (int q = 0; q < UL; ++q) {
            val[q] = 0.f;
#pragma unroll
            for (int bb = 0; bb < BP_; ++bb) val[q] = (bb == b) ? qv[q][bb] : val[q];
          }
        } else {
#pragma unroll
          for (int q = 0; q < UL; ++q) {
            val[q] = 0.f;
#pragma unroll
            for (int r = 0; r < R_; ++r) {
              float qr[BP_];
              load_row<BP_, PACK>(Qs + ((int64_t)post[q] * C + r) * RS, qr);
              float qb = 0.f;
#pragma unroll
              for (int bb = 0; bb < BP_; ++bb) qb = (bb == b) ? qr[bb] : qb;
              val[q] += qb * basis_s[sid[q] * R_ + r];
            }
          }
        }
#pragma unroll
        for (int q = 0; q < UL; ++q) {
          const int j = jb + q * 32 + lane;
          if (j < j1) atomicAdd(a.dw_lgn + j, val[q]);
        }
      }
      if (lane == 0) c_dw += (unsigned long long)(j1 - j0);
    }
  };

  // Tape of step ts into the planes of its parity: v, spike / refractory bits, the rows that must be
  // walked (queue and descriptors) and zeros in the spike-gradient plane for those that need not.
  int* q_cnt_cur = s_misc + 2;  // queue counter of the current iteration
  auto load_step = [&](int ts, float* tvp, uint8_t* tzp, float* gzp, bool queue) {
    for (int k0 = 0; k0 < cn; k0 += NT) {
      const int k = k0 + tid;
      const bool act = k < cn;
      const int n = n0 + (act ? k : 0);
      // the row's bounds do not depend on the tape: requested first, they arrive together with it
      int rj0 = 0, rj1 = 0;
      if (queue && fast_rows && act) {
        rj0 = rpx[k * D];
        rj1 = rpx[k * D + D];
      }
      // all tape loads of the neuron are issued before any of them is used
      float vv[NBX];
      unsigned zz[NBX];
#pragma unroll
      for (int b = 0; b < NBX; ++b) {
        vv[b] = 0.f;
        zz[b] = 2u;
        if (b < B && act) {
          const int64_t ti = ((int64_t)ts * B + b) * N + n;
          const float w = __ldcs(a.tape_v + ti);  // voltage, low two mantissa bits = (spiked, refractory)
          vv[b] = __uint_as_float(__float_as_uint(w) & ~3u);
          zz[b] = __float_as_uint(w) & 3u;
        }
      }
      unsigned zm = 0, need = 0;
#pragma unroll
      for (int b = 0; b < NBX; ++b) {
        if (b < B && act) {
          tvp[b * chunkP + k] = vv[b];
          tzp[b * chunkP + k] = (uint8_t)zz[b];
          zm |= (zz[b] & 1u) << b;
          if (!(zz[b] & 2u) && pseudo_h(vv[b] - 1.f, a) != 0.f) need = 1;
        }
      }
      if (!queue) continue;
      const bool walk = act && (need | zm);
      if (act) {
        zmask_s[k] = (uint8_t)zm;
        if (!walk)
          for (int b = 0; b < B; ++b) gzp[b * chunkP + k] = 0.f;  // row is not walked
      }
      // queue the rows to walk: one shared-memory atomic per warp (order is irrelevant)
      const unsigned wm = __ballot_sync(0xffffffffu, walk);
      if (wm) {
        int base = 0;
        if (lane == 0) base = atomicAdd(q_cnt_cur, __popc(wm));
        base = __shfl_sync(0xffffffffu, base, 0);
        if (walk) {
          const int qpos = base + __popc(wm & ((1u << lane) - 1u));
          rowq_s[qpos] = (uint16_t)k;
          if (fast_rows) {
            const int j0 = rj0, j1 = rj1;
            rowd_s[qpos] = make_int4(j0, j1, k | (int)(zm << 16), 0);
            c_rows += (unsigned long long)D;
            c_events += (unsigned long long)(j1 - j0);
            if (zm) c_dw += (unsigned long long)(j1 - j0) * __popc(zm);
          }
        }
      }
    }
  };

  // Paired mode: the saved words of step ts for this thread's neuron into `pl` (the thread is the
  // only reader and writer of its entries); returns walk | spike mask << 1.
  auto load_tape_own = [&](int ts, float* pl) -> unsigned {
    if (tid >= cn || ts < 0) return 0u;
    unsigned ww[NBX];
#pragma unroll
    for (int b = 0; b < NBX; ++b)
      ww[b] = b < B ? __float_as_uint(__ldcs(a.tape_v + ((int64_t)ts * B + b) * N + n0 + tid)) : 2u;
    unsigned zm = 0, need = 0;
#pragma unroll
    for (int b = 0; b < NBX; ++b) {
      if (b < B) {
        pl[b * chunkP + tid] = __uint_as_float(ww[b]);
        zm |= (ww[b] & 1u) << b;
        if (!(ww[b] & 2u) && pseudo_h(__uint_as_float(ww[b] & ~3u) - 1.f, a) != 0.f) need = 1;
      }
    }
    return ((need | zm) ? 1u : 0u) | (zm << 1);
  };

  // The loop runs one iteration per step t, newest first.  An iteration loads the tape of step t-1,
  // then every warp does its share of the dense adjoint of step t and goes straight on to the gather
  // of step t-1 (spike gradients of step t-1, needed by the next iteration): the two have no
  // dependence on each other, the dense part is bound by instruction issue and the gather by L2
  // requests, so running them without a barrier in between lets them overlap.  Per-step planes
  // (v, bits, spike gradient) are double-buffered by step parity.
  // Gather(t-1) reads Q(t .. t-1+D); Q(t) was published by the dense part of step t+2, so every block
  // must have finished iteration it-2 (phase it-1).  A block is then at most one iteration ahead of
  // the slowest one and writes Q(t-3) at the earliest: D+3 ring slots suffice.
  if (PAIR) {
    // prologue: the saved words of the last two steps (and the row flags of step T-2); the spike
    // gradient that later steps send to them is zero
    if (T >= 1) {
      load_tape_own(T - 1, tv_s + ((T - 1) & 1) * plane);
      const unsigned f = load_tape_own(T - 2, tv_s + ((T - 2) & 1) * plane);
      if (tid < cn) zmask_s[((T - 2) & 1) * chunkP + tid] = (uint8_t)f;
    }
    for (int i = tid; i < 2 * (int)plane; i += NT) gz_s[i] = 0.f;
    __syncthreads();
  } else if (T >= 1) {
    // prologue: tape of the last step; its spike gradient from later steps is zero
    load_step(T - 1, tv_s + ((T - 1) & 1) * plane, tz_s + ((T - 1) & 1) * plane, gz_s + ((T - 1) & 1) * plane, false);
    __syncthreads();
    for (int i = tid; i < (int)plane; i += NT) gz_s[((T - 1) & 1) * plane + i] = 0.f;
    __syncthreads();
  }
  for (int it = 0; it < T && ok; ++it) {
    const int t = T - 1 - it;   // step of the dense adjoint
    const int tg = t - 1;       // step of the gather (none in the last iteration)
    float* const tvC = tv_s + (t & 1) * plane;
    uint8_t* const tzC = tz_s + (t & 1) * plane;
    float* const gzC = gz_s + (t & 1) * plane;
    float* const gzB = gz_s + ((t & 1) ^ 1) * plane;
    const unsigned long long ph0 = prof ? gtime_b() : 0;
    int* const q_cnt = s_misc + 2 + (it & 1);  // rows queued / next queue slot of this iteration
    int* const q_pop = s_misc + 4 + (it & 1);
    if (tid == 0) {
      s_misc[2 + ((it + 1) & 1)] = 0;  // the counters of the next iteration
      s_misc[4 + ((it + 1) & 1)] = 0;
    }
    if (PAIR) {
      // first 32-byte row of the pair that a synapse of delay tid+1 reads in this iteration: delay 1
      // the pair holding Q(t), the delays of this iteration's parity the pair {Q(t-1+d), Q(t-2+d)}
      if (tid < 8) slot_s[tid] = (((tid == 0 ? t + 1 : t + tid + 1) >> 1) % a.KP) * Np * C;
    } else if (tid < 8) slot_s[tid] = ((tg + 1 + tid) % K) * Np * C;
    // Lagged barrier, by a thread of the last warp (which owns no neuron when the slice has fewer
    // neurons than the block has threads) while the others load the tape: this block has finished
    // iteration it-1; every block must have finished iteration it-2 before the gather below.
    if (tid == BAR_TID && it >= 1) {
      v1g_arrive(v1g_phase_counter(a.barrier, it));
      const unsigned long long target = v1g_phase_target(it - 1, G);
      if (seen < target)
        seen = v1g_wait(v1g_phase_counter(a.barrier, it - 1), target, a.spin_limit, a.status);
      if (seen < target) s_misc[1] = 1;
    }

    // ---------------- phase A: tape of step t-1, row flags, counts of step t-2 ----------------
    q_cnt_cur = q_cnt;
    float gzr[NBX];    // paired mode: gathered spike gradient and saved word of step t for the dense part
    unsigned twr[NBX];
    if (PAIR) {
      // Planes are shared by the steps t and t-2; every entry belongs to one thread, which takes its
      // values of step t into registers before it overwrites them with those of step t-2.
#pragma unroll
      for (int b = 0; b < NBX; ++b) {
        const bool own = b < B && tid < cn;
        gzr[b] = own ? gzC[b * chunkP + tid] : 0.f;
        twr[b] = own ? __float_as_uint(tvC[b * chunkP + tid]) : 2u;
      }
      const unsigned f2 = load_tape_own(t - 2, tvC);
      unsigned f1 = 0;
      if (tid < cn) {
        if (tg >= 0) f1 = zmask_s[((t & 1) ^ 1) * chunkP + tid];
        zmask_s[(t & 1) * chunkP + tid] = (uint8_t)f2;
      }
      // the row is walked for the delays >= 2 when either step needs it, for delay 1 when step t-1 does
      const bool walk = ((f1 | f2) & 1u) != 0;
      if (tid < cn && !walk)
        for (int b = 0; b < B; ++b) gzC[b * chunkP + tid] = 0.f;  // spike gradient of step t-2 so far
      const unsigned wm = __ballot_sync(0xffffffffu, walk);
      if (wm) {
        int base = 0;
        if (lane == 0) base = atomicAdd(q_cnt_cur, __popc(wm));
        base = __shfl_sync(0xffffffffu, base, 0);
        if (walk) {
          const unsigned zm1 = f1 >> 1, zm2 = f2 >> 1;
          const int32_t* pp = a.pair_ptr[(t - 1) & 1] + n0 + tid;
          const int len1 = rpx[tid * D + 1] - rpx[tid * D];   // delay-1 entries: they lead the row and serve step t-1 only
          const int skip = (f1 & 1u) ? 0 : len1;              // not needed when only step t-2 asks for the row
          const int j0 = pp[0] + skip, j1 = pp[1];
          rowd_s[base + __popc(wm & ((1u << lane) - 1u))] = make_int4(j0, j1, tid | (int)(zm1 << 16) | (int)(zm2 << 21), 0);
          c_rows += 1ull + (unsigned long long)((D - ((t - 1) & 1)) / 2);
          c_events += (unsigned long long)(j1 - j0);
          c_dw += (unsigned long long)(j1 - j0) * __popc(zm1) + (unsigned long long)(j1 - pp[0] - len1) * __popc(zm2);
        }
      }
    } else
    if (tg >= 0) load_step(tg, tv_s + ((t & 1) ^ 1) * plane, tz_s + ((t & 1) ^ 1) * plane, gzB, true);
    if (t >= 2)
      for (int i = tid; i < nb; i += NT) {
        const int b = i / a.n_bkg, j = i - b * a.n_bkg;
        s_cnt[i] = (float)a.bkg_counts[((int64_t)b * T + (t - 2)) * a.n_bkg + j];
      }
    __syncthreads();
    if (s_misc[1]) {
      ok = false;
      break;
    }
    const unsigned long long ph1 = prof ? gtime_b() : 0;

    // ---------------- dense adjoint of step t, publish Q(t-2), background weight gradient ----------------
    const int bin = (a.sgrad && a.sync_bin > 0 && t / a.sync_bin < a.nbins) ? t / a.sync_bin : -1;
    float* Qw = a.Q + (t >= 2 ? qbase(t - 2) : 0);
    const bool sync_on = a.sync.first != nullptr && t >= a.sync.t0 && t < a.sync.t0 + a.sync.W;
    const bool osi_on = a.osi_coef != nullptr && t >= a.osi_t0 && t < a.osi_t1;
    for (int k = tid; k < cn; k += NT) {
      const int n = n0 + k;
      const float k_decay = a.decay[n], k_cf = a.cf[n], k_ad0 = a.asc_decay[2 * n], k_ad1 = a.asc_decay[2 * n + 1];
      const float rc = (a.rate_coef && t >= a.rate_t0 && t < a.rate_t1) ? a.rate_coef[n] : 0.f;
      const float vlo = a.v_lo ? a.v_lo[n] : 0.f;
      float sadd[NBX];  // synchrony target over given samples and OSI/DSI target: dL/dz[b, t, n]
#pragma unroll
      for (int b = 0; b < NBX; ++b) sadd[b] = 0.f;
      if (sync_on) {
        for (int sp = a.sync.first[n]; sp >= 0; sp = a.sync.next[sp]) {
          const int smp = a.sync.pos_sample[sp];
          const int tb = a.sync.trial[smp];
          const float gs = a.sync.g[(int64_t)smp * a.sync.W + (t - a.sync.t0)];
#pragma unroll
          for (int b = 0; b < NBX; ++b) sadd[b] += (b == tb) ? gs : 0.f;
        }
      }
      if (osi_on) {
#pragma unroll
        for (int b = 0; b < NBX; ++b)
          if (b < B) sadd[b] += a.osi_coef[(int64_t)b * N + n];
      }
      float dyv[NBX][R_];  // dy(t-2) of every batch row of this neuron
      // The state of a batch row is read before any of it is written back.  A load may not pass an
      // earlier store to the same array; when the state lives in a global slab (slices that do not fit
      // in shared memory) each of the 13 reads of a row would otherwise wait a full L2 round trip on its
      // own (230,924-neuron column: dense part 99 -> 46 us per step), and on chip the loop is 0.8 %
      // faster this way as well.
      {
#pragma unroll
        for (int b = 0; b < NBX; ++b) {
#pragma unroll
          for (int r = 0; r < R_; ++r) dyv[b][r] = 0.f;
          if (b < B) {
            const int si = b * chunkP + k;
            const float sv = G_v[si], s0 = G_a0[si], s1 = G_a1[si];
            float sp[R_], spr[R_];
#pragma unroll
            for (int r = 0; r < R_; ++r) {
              sp[r] = G_p[(r * B + b) * chunkP + k];
              spr[r] = G_pr[(r * B + b) * chunkP + k];
            }
            const float v = PAIR ? __uint_as_float(twr[b] & ~3u) : tvC[si];
            const unsigned zr = PAIR ? (twr[b] & 3u) : (unsigned)tzC[si];
            const bool free_ = !(zr & 2u);
            const int64_t oi = ((int64_t)b * T + t) * N + n;
            float gz = rc + (bin >= 0 ? a.sgrad[b * a.nbins + bin] : 0.f) + (a.g_z ? a.g_z[oi] : 0.f);
            gz += sadd[b];
            gz += a.rec_factor * (PAIR ? gzr[b] : gzC[si]);
            float gv = sv + (a.g_v ? a.g_v[oi] : 0.f);
            if (a.volt_coef != 0.f) {
              // range mode: outside [vlo, 1]; threshold mode: distance from the threshold
              const float hi = a.volt_threshold_mode ? v - 1.f : fmaxf(v - 1.f, 0.f);
              const float lo = a.volt_threshold_mode ? 0.f : fmaxf(vlo - v, 0.f);
              gv += 2.f * a.volt_coef * (hi - lo);
              volt_loss += hi * hi + lo * lo;
            }
            if (free_) gv += gz * pseudo_h(v - 1.f, a);
            if (a.hard_reset && !free_) gv = 0.f;
            G_v[si] = k_decay * a.vd_keep * gv;
            const float gc1 = k_cf * gv;
            G_a0[si] = k_ad0 * s0 + gc1;
            G_a1[si] = k_ad1 * s1 + gc1;
#pragma unroll
            for (int r = 0; r < R_; ++r) {
              const int pi = (r * B + b) * chunkP + k;
              const float gp = sp[r], gpr = spr[r];
              const float gp1 = a.sd[r] * gp + gc1;                // g_p(t-1)
              const float gpr1 = a.sd[r] * gpr + a.dtsd[r] * gp;   // g_pr(t-1)
              G_p[pi] = gp1;
              G_pr[pi] = gpr1;
              const float gpr2 = a.sd[r] * gpr1 + a.dtsd[r] * gp1;  // g_pr(t-2)
              dyv[b][r] = (gpr2 * a.pinit[r]) * a.lr_scale;
            }
          }
        }
      }
      if (t >= 2) {
        // one 16/32-byte row per channel, all batch rows of the neuron at once
        float4* qd = (float4*)(Qw + (int64_t)n * C * RS);
        for (int c = 0; c < C; ++c) {
          float row[NBX];
#pragma unroll
          for (int b = 0; b < NBX; ++b) {
            if (PROJ) {
              float s2 = 0.f;
#pragma unroll
              for (int r = 0; r < R_; ++r) s2 += basis_s[c * R_ + r] * dyv[b][r];
              row[b] = s2;
            } else {
              float s2 = 0.f;
#pragma unroll
              for (int r = 0; r < R_; ++r) s2 = (r == c) ? dyv[b][r] : s2;
              row[b] = s2;
            }
          }
          if (PACK) {
            float r8[8];
#pragma unroll
            for (int b = 0; b < 8; ++b) r8[b] = b < NBX ? row[b % NBX] : 0.f;
            __stcg(qd + c * (RS / 4), pack_row5(r8));
          } else {
            __stcg(qd + c * (RS / 4), make_float4(row[0], row[1], row[2], row[3]));
            if (BP_ == 8)
              __stcg(qd + c * (RS / 4) + 1, make_float4(row[4 % NBX], row[5 % NBX], row[6 % NBX], row[7 % NBX]));
          }
        }
        // background weight gradient of step t-2 for the synapses this thread owns (branch-free:
        // a zero count contributes zero)
        auto bkg_grad = [&](int pre, int sid) {
          const float* bs = basis_s + sid * R_;
          float bsr[R_];
#pragma unroll
          for (int r = 0; r < R_; ++r) bsr[r] = bs[r];
          float accw = 0.f;
#pragma unroll
          for (int b = 0; b < NBX; ++b) {
            if (b < B) {
              float s2 = 0.f;
#pragma unroll
              for (int r = 0; r < R_; ++r) s2 += dyv[b][r] * bsr[r];
              accw += s2 * s_cnt[b * a.n_bkg + pre];
            }
          }
          return accw;
        };
        if (a.bkg_in_smem) {
          for (int j = bkptr_s[k]; j < bkptr_s[k + 1]; ++j) bk_dw[j] += bkg_grad(bk_pre[j], (int)bk_sid[j]);
        } else {
          // tables and accumulators in global memory: four synapses' entries are requested together
          for (int j0 = bkptr_s[k], j1 = bkptr_s[k + 1]; j0 < j1; j0 += 4) {
            int pre[4], sid[4];
            float old[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int j = min(j0 + u, j1 - 1);
              pre[u] = bk_pre[j];
              sid[u] = (int)bk_sid[j];
              old[u] = bk_dw[j];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float accw = bkg_grad(pre[u], sid[u]);
              if (j0 + u < j1 && accw != 0.f) bk_dw[j0 + u] = old[u] + accw;
            }
          }
        }
      }
    }
    const unsigned long long ph2 = prof ? gtime_b() : 0;
    // ---------------- gather of step t-1 over the out-synapses of every needed neuron ----------------
    if (tid == BAR_TID) seen = v1g_ld_acquire(v1g_phase_counter(a.barrier, it));
    const int tk = (tg + K) % K;
    constexpr int U = PROJ ? 4 : 1;  // row iterations (32 synapses each) kept in flight per warp
    // one pass = U*32 consecutive synapses of a row, lane l holding synapses jb + u*32 + l
    auto load_pass = [&](int jb, int j1, int (&post)[U], int (&sid)[U], float (&w)[U]) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int j = jb + u * 32 + lane;
        const bool v = j < j1;
        if (a.csr_evict_first) {
          post[u] = v ? __ldcs(a.rec_post + j) : 0;
          sid[u] = v ? (int)__ldcs(a.rec_sid + j) : 0;
          w[u] = v ? __ldcs(a.rec_w + j) : 0.f;
        } else {
          post[u] = v ? a.rec_post[j] : 0;
          sid[u] = v ? (int)a.rec_sid[j] : 0;
          w[u] = v ? a.rec_w[j] : 0.f;
        }
      }
    };
    // sum the BP_ accumulators over the warp: each exchange halves the values a lane carries
    // (9 shuffles for 8 accumulators instead of 40); lane l ends with the total of batch row
    // ((l >> 2) & 1) | ((l >> 3) & 1) << 1 | ((l >> 4) & 1) << 2
    auto reduce_store = [&](const float (&acc)[BP_], int k) {
      float a4[4];
      if (BP_ == 8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const bool hi = lane & 16;
          const float recv = __shfl_xor_sync(0xffffffffu, hi ? acc[i] : acc[(i + 4) % BP_], 16);
          a4[i] = (hi ? acc[(i + 4) % BP_] : acc[i]) + recv;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) a4[i] = acc[i] + __shfl_xor_sync(0xffffffffu, acc[i], 16);
      }
      float a2[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const bool hi = lane & 8;
        const float recv = __shfl_xor_sync(0xffffffffu, hi ? a4[i] : a4[i + 2], 8);
        a2[i] = (hi ? a4[i + 2] : a4[i]) + recv;
      }
      float a1;
      {
        const bool hi = lane & 4;
        const float recv = __shfl_xor_sync(0xffffffffu, hi ? a2[0] : a2[1], 4);
        a1 = (hi ? a2[1] : a2[0]) + recv;
      }
      a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
      a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
      int bsel = ((lane >> 2) & 1) | (((lane >> 3) & 1) << 1);
      if (BP_ == 8) bsel |= ((lane >> 4) & 1) << 2;
      if ((lane & 3) == 0 && (BP_ == 8 || lane < 16) && bsel < B) gzB[bsel * chunkP + k] = a1;
    };
    // The LGN events of step t first (Q(t) is complete, and all zero in the first two iterations):
    // the few warps that hold one start on the row queue a little later and simply take fewer rows.
    if (it >= 2) lgn_dw(t);
    // warps take rows from the queue one at a time, so a warp that drew long rows takes fewer
    const int nq = tg >= 0 ? *q_cnt : 0;
    auto pop_row = [&]() {
      int q = 0;
      if (lane == 0) q = atomicAdd(q_pop, 1);
      return __shfl_sync(0xffffffffu, q, 0);
    };
    if (PAIR) {
      // Paired gather.  The records of a neuron are stored a second time in gather order, once per
      // delay parity: its delay-1 bucket (serves step t-1 only) followed by the buckets of delay d >= 2
      // with t-1+d even (one 32-byte pair row {Q(t-1+d), Q(t-2+d)} serves the steps t-1 and t-2).  A
      // row is therefore one contiguous range, walked exactly like the unpaired packed-record path:
      // passes of UF*32 entries, records of the pass after next and pair rows of the next pass in
      // flight while the current one is accumulated.
      constexpr int NB = PACK ? 5 : BP_;  // batch values a row carries
      constexpr int UF = V1G_BWD_PAIR_GROUPS, NS = 2;
      const int cpar = (t - 1) & 1;
      const bool todd = t & 1;            // Q(t) is the second half of its pair when t is odd
      const uint2* const prec = a.pair_rec[cpar];
      const int plast = a.pair_last[cpar];
      float* const gz1 = gzB;             // spike gradient of step t-1: add
      float* const gz2 = gzC;             // spike gradient of step t-2: first contribution
      struct Pass { int jb, j1, kz, fl; };  // kz = row | spike mask(t-1) << 16 | spike mask(t-2) << 21; fl: 1 first pass of its row, 4 valid
      Pass pr{0, 0, 0, 0};
      Pass ps_[NS];
      uint2 rec[UF];
      float4 qLo[NS][UF], qHi[NS][UF];
      float wS[NS][UF];
      int cS[NS];           // bit u: entry u of the pass is a delay-1 entry
      float acc1[NB], acc2[NB];
#pragma unroll
      for (int i = 0; i < NS; ++i) {
        ps_[i] = Pass{0, 0, 0, 0};
        cS[i] = 0;
      }
#pragma unroll
      for (int b = 0; b < NB; ++b) acc1[b] = acc2[b] = 0.f;
      auto issue_rec = [&]() {  // advance pr to the following pass and request its records
        if (pr.fl && pr.jb + 32 * UF < pr.j1) {
          pr.jb += 32 * UF;
          pr.fl = 4;
        } else {
          const int q = pop_row();
          if (q < nq) {
            const int4 d = rowd_s[q];
            pr = Pass{d.x, d.y, d.z, 5};
          } else {
            pr = Pass{0, 0, 0, 0};
          }
        }
#pragma unroll
        for (int u = 0; u < UF; ++u) rec[u] = __ldcs(prec + min(pr.jb + u * 32 + lane, plast));
      };
      auto issue_q = [&](const Pass& ps, float4 (&lo)[UF], float4 (&hi)[UF], float (&w)[UF], int& c) {
        c = 0;
#pragma unroll
        for (int u = 0; u < UF; ++u) {
          const bool in_row = ps.jb + u * 32 + lane < ps.j1;
          const unsigned w0 = rec[u].x;
          unsigned row = (unsigned)slot_s[w0 >> 29] + (w0 & 0x3fffffu) * (unsigned)C + ((w0 >> 22) & 127u);
          row = in_row ? row : 0u;  // lanes past the end of the row share one request
          load_pair(a.Q + (size_t)row * 8u, lo[u], hi[u]);
          w[u] = in_row ? __uint_as_float(rec[u].y) : 0.f;
          c |= ((w0 >> 29) == 0u) ? (1 << u) : 0;
        }
      };
      auto compute = [&](const Pass& ps, const float4 (&lo)[UF], const float4 (&hi)[UF], const float (&w)[UF],
                         const int c) {
        if (ps.fl & 1) {
#pragma unroll
          for (int b = 0; b < NB; ++b) acc1[b] = acc2[b] = 0.f;
        }
        const unsigned zm1 = ((unsigned)ps.kz >> 16) & 31u, zm2 = ((unsigned)ps.kz >> 21) & 31u;
#pragma unroll
        for (int u = 0; u < UF; ++u) {
          float pl[NB], ph[NB];
          unpack_half<NB, PACK>(lo[u], pl);
          unpack_half<NB, PACK>(hi[u], ph);
          const bool d1 = (c >> u) & 1;
          const bool sw = d1 && todd;      // delay 1 with Q(t) in the second half
          const float w2 = d1 ? 0.f : w[u];
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            acc1[b] += w[u] * (sw ? ph[b] : pl[b]);
            acc2[b] += w2 * ph[b];
          }
          if (zm1 | zm2) {
            // the source neuron spiked at step t-1 (zm1) or t-2 (zm2): recurrent weight gradient
            const int js = ps.jb + u * 32 + lane;
            if (js < ps.j1) {
              float dwv = 0.f;
#pragma unroll
              for (int b = 0; b < NB; ++b) {
                if (zm1 & (1u << b)) dwv += sw ? ph[b] : pl[b];
                if (!d1 && (zm2 & (1u << b))) dwv += ph[b];
              }
              a.dw_rec[a.pair_j[cpar][js]] += dwv;  // this lane is the only writer of the synapse
            }
          }
        }
        if (ps.jb + 32 * UF >= ps.j1) {
          const int k = ps.kz & 0xffff;
          float v8[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            v8[i] = acc1[i % NB];
            v8[i + 4] = acc2[i % NB];
          }
          const float tot = warp_reduce8(v8, lane);
          const int idx = (lane >> 2) & 7, b = idx & 3;
          if ((lane & 3) == 0 && b < B) {
            if (idx < 4) gz1[b * chunkP + k] += tot;
            else gz2[b * chunkP + k] = tot;
          }
          if (NB == 5) {
            const float t5 = warp_reduce2(acc1[4 % NB], acc2[4 % NB], lane);
            if (lane == 0) gz1[4 * chunkP + k] += t5;
            if (lane == 16) gz2[4 * chunkP + k] = t5;
          }
        }
      };
      auto turn = [&](auto I) -> bool {
        constexpr int i = decltype(I)::value;
        if (!pr.fl) {
#pragma unroll
          for (int o = 1; o < NS; ++o)
            if (ps_[(i + o) % NS].fl)
              compute(ps_[(i + o) % NS], qLo[(i + o) % NS], qHi[(i + o) % NS], wS[(i + o) % NS], cS[(i + o) % NS]);
          return false;
        }
        ps_[i] = pr;
        issue_q(ps_[i], qLo[i], qHi[i], wS[i], cS[i]);
        issue_rec();
        constexpr int x = (i + 1) % NS;  // the oldest pass
        if (ps_[x].fl) {
          compute(ps_[x], qLo[x], qHi[x], wS[x], cS[x]);
          ps_[x].fl = 0;
        }
        return true;
      };
      if (nq > 0) {
        issue_rec();
        for (;;) {
          if (!turn(std::integral_constant<int, 0>{})) break;
          if (!turn(std::integral_constant<int, 1>{})) break;
        }
      }
    } else if (fast_rows) {
      // Two forms of the same pipeline, chosen at compile time.  The projected one (one lane per
      // synapse, one 16/32-byte row) is kept apart from the raw one (lanes sharing a synapse):
      // written as one generic body the projected kernel ran 0.3 % slower.
      if (PROJ) {
        // Packed-record path.  The unit of work is a pass: up to UF*32 consecutive synapses of one
        // row, one 8-byte record per synapse.  Warps draw rows from the queue of row descriptors
        // written in phase A.  Each warp keeps the records of the pass after next
        // and the Q rows of the next pass in flight while it accumulates the current one.  Registers
        // that receive a load are never copied while the load is in flight (a copy would wait for
        // it): the loop body is written out once per Q buffer, NS buffers in rotation.
        // The Q row index comes from a per-step table of the D slot bases.  Steps past the end of
        // the rollout need no test: their ring slots still hold the zeros of the initial clear.
        // Lanes past the end of a row read a neighbouring record (always inside the array) and get
        // weight zero.
        constexpr int NB = PACK ? 5 : BP_;     // batch values a row really carries
        constexpr int QV = QW / 4;             // 16-byte words per Q row
        constexpr int UF = QV == 1 ? V1G_BWD_GROUPS : 2;  // 32-synapse groups per pass
        constexpr int NS = V1G_BWD_STAGES;
        struct Pass { int jb, j1, kz, fl; };   // kz = row | spike mask << 16; fl: 1 first pass of its row, 4 valid
        const int jmax = a.rec_nnz - 1;
        Pass pr{0, 0, 0, 0};
        Pass ps_[NS];
        uint2 rec[UF];
        float4 qS[NS][UF][QV];
        float wS[NS][UF];
        float acc[BP_];
#pragma unroll
        for (int i = 0; i < NS; ++i) ps_[i] = Pass{0, 0, 0, 0};
#pragma unroll
        for (int b = 0; b < BP_; ++b) acc[b] = 0.f;
        auto issue_rec = [&]() {  // advance pr to the following pass and request its records
          if (pr.fl && pr.jb + 32 * UF < pr.j1) {
            pr.jb += 32 * UF;
            pr.fl = 4;
          } else {
            const int q = pop_row();  // warps that drew long rows, or rows with spikes, take fewer
            if (q < nq) {
              const int4 d = rowd_s[q];
              pr = Pass{d.x, d.y, d.z, 5};
            } else {
              pr = Pass{0, 0, 0, 0};
            }
          }
#pragma unroll
          for (int u = 0; u < UF; ++u) rec[u] = __ldcs(a.rec_syn8 + min(pr.jb + u * 32 + lane, jmax));
        };
        auto issue_q = [&](const Pass& ps, float4 (&q)[UF][QV], float (&w)[UF]) {  // Q rows of the pass in rec
#pragma unroll
          for (int u = 0; u < UF; ++u) {
            const bool in_row = ps.jb + u * 32 + lane < ps.j1;
            const unsigned w0 = rec[u].x;
            unsigned row = (unsigned)slot_s[w0 >> 29] + (w0 & 0x3fffffu) * (unsigned)C + ((w0 >> 22) & 127u);
            row = in_row ? row : 0u;  // lanes past the end of the row share one request
            const float4* qp = (const float4*)(a.Q + row * (unsigned)QW);  // < 2^31 words, checked by the host
#pragma unroll
            for (int v = 0; v < QV; ++v) q[u][v] = __ldcg(qp + v);
            w[u] = in_row ? __uint_as_float(rec[u].y) : 0.f;
          }
        };
        auto compute = [&](const Pass& ps, const float4 (&q)[UF][QV], const float (&w)[UF]) {
          if (ps.fl & 1) {
#pragma unroll
            for (int b = 0; b < BP_; ++b) acc[b] = 0.f;
          }
          const unsigned zm = (unsigned)ps.kz >> 16;
          if (!zm) {
#pragma unroll
            for (int u = 0; u < UF; ++u) {
              float pj[BP_];
              unpack_row<BP_, PACK>(q[u], pj);
#pragma unroll
              for (int b = 0; b < NB; ++b) acc[b] += w[u] * pj[b];
            }
          } else {
            // the source neuron spiked at this step in the batch rows of zm: weight gradient.  The
            // pass's old gradient values are requested together (a load after a store to the same array
            // would wait for its own round trip); this lane is the only writer of its synapses
            float dw_old[UF];
#pragma unroll
            for (int u = 0; u < UF; ++u) dw_old[u] = a.dw_rec[min(ps.jb + u * 32 + lane, jmax)];
#pragma unroll
            for (int u = 0; u < UF; ++u) {
              float pj[BP_];
              unpack_row<BP_, PACK>(q[u], pj);
#pragma unroll
              for (int b = 0; b < NB; ++b) acc[b] += w[u] * pj[b];
              const int j = ps.jb + u * 32 + lane;
              if (j < ps.j1) {
                float dwv = 0.f;
#pragma unroll
                for (int b = 0; b < NB; ++b)
                  if (zm & (1u << b)) dwv += pj[b];
                a.dw_rec[j] = dw_old[u] + dwv;
              }
            }
          }
          if (ps.jb + 32 * UF >= ps.j1) reduce_store(acc, ps.kz & 0xffff);
        };
        // one turn of the pipeline with buffer I: false when the warp has no further pass
        auto turn = [&](auto I) -> bool {
          constexpr int i = decltype(I)::value;
          if (!pr.fl) {
            // accumulate what is still in flight, oldest first
#pragma unroll
            for (int o = 1; o < NS; ++o)
              if (ps_[(i + o) % NS].fl) compute(ps_[(i + o) % NS], qS[(i + o) % NS], wS[(i + o) % NS]);
            return false;
          }
          ps_[i] = pr;
          issue_q(ps_[i], qS[i], wS[i]);
          issue_rec();
          constexpr int x = (i + 1) % NS;  // the oldest pass
          if (ps_[x].fl) {
            compute(ps_[x], qS[x], wS[x]);
            ps_[x].fl = 0;
          }
          return true;
        };
        issue_rec();
        for (;;) {
          if (!turn(std::integral_constant<int, 0>{})) break;
          if (!turn(std::integral_constant<int, 1 % NS>{})) break;
          if (NS > 2 && !turn(std::integral_constant<int, 2 % NS>{})) break;
          if (NS > 3 && !turn(std::integral_constant<int, 3 % NS>{})) break;
        }
      } else {
        // Packed-record path.  The unit of work is a pass: up to UF*32 consecutive synapses of one
        // row, one 8-byte record per synapse.  Warps draw rows from the queue of row descriptors
        // written in phase A.  Each warp keeps the records of the pass after next
        // and the Q rows of the next pass in flight while it accumulates the current one.  Registers
        // that receive a load are never copied while the load is in flight (a copy would wait for
        // it): the loop body is written out once per Q buffer, NS buffers in rotation.
        // The Q row index comes from a per-step table of the D slot bases.  Steps past the end of
        // the rollout need no test: their ring slots still hold the zeros of the initial clear.
        // Lanes past the end of a row read a neighbouring record (always inside the array) and get
        // weight zero.
        // Raw mode (more than 8 synapse types: the ring holds the R = 4 channels of a neuron as four
        // consecutive 16-byte rows, one 64-byte half line): LPS lanes share a synapse, each taking
        // CPL = 4 / LPS channels, so that one load instruction touches one line per synapse instead of
        // four; a lane accumulates w * basis[sid][c] * Q[post][c][b] over its channels, and the reduction
        // over the warp at the end of the row sums channels and synapses alike.
        constexpr bool QUAD = !PROJ;
        constexpr int LPS = QUAD ? V1G_BWD_RAW_LANES : 1;  // lanes per synapse
        constexpr int CPL = QUAD ? 4 / LPS : 1;            // channels (16-byte rows) a lane loads
        constexpr int SPG = 32 / LPS;          // synapses per 32-lane group
        constexpr int NB = PACK ? 5 : BP_;     // batch values a row really carries
        constexpr int QV = QW / 4;             // 16-byte words per Q row
        constexpr int QVL = QV * CPL;          // 16-byte words per lane and synapse
        constexpr int UF = QUAD ? V1G_BWD_RAW_GROUPS : QV == 1 ? V1G_BWD_GROUPS : 2;  // 32-lane groups per pass
        static_assert(!QUAD || UF <= 4, "the synapse types of a pass are kept as four 8-bit fields of one word");
        constexpr int SPP = SPG * UF;          // synapses per pass
        const int lsyn = lane / LPS, lch = lane % LPS;
        constexpr int NS = V1G_BWD_STAGES;
        struct Pass { int jb, j1, kz, fl; };   // kz = row | spike mask << 16; fl: 1 first pass of its row, 4 valid
        const int jmax = a.rec_nnz - 1;
        Pass pr{0, 0, 0, 0};
        Pass ps_[NS];
        uint2 rec[UF];
        float4 qS[NS][UF][QVL];
        float wS[NS][UF][CPL];
        unsigned sidS[QUAD ? NS : 1];  // raw mode: the synapse types of the pass, 8 bits per group (for the weight gradient)
        float acc[BP_];
#pragma unroll
        for (int i = 0; i < NS; ++i) ps_[i] = Pass{0, 0, 0, 0};
#pragma unroll
        for (int b = 0; b < BP_; ++b) acc[b] = 0.f;
        auto issue_rec = [&]() {  // advance pr to the following pass and request its records
          if (pr.fl && pr.jb + SPP < pr.j1) {
            pr.jb += SPP;
            pr.fl = 4;
          } else {
            const int q = pop_row();  // warps that drew long rows, or rows with spikes, take fewer
            if (q < nq) {
              const int4 d = rowd_s[q];
              pr = Pass{d.x, d.y, d.z, 5};
            } else {
              pr = Pass{0, 0, 0, 0};
            }
          }
#pragma unroll
          for (int u = 0; u < UF; ++u) rec[u] = __ldcs(a.rec_syn8 + min(pr.jb + u * SPG + lsyn, jmax));
        };
        auto issue_q = [&](const Pass& ps, float4 (&q)[UF][QVL], float (&w)[UF][CPL], unsigned& sids) {  // Q rows of the pass in rec
          if (QUAD) sids = 0u;
#pragma unroll
          for (int u = 0; u < UF; ++u) {
            const bool in_row = ps.jb + u * SPG + lsyn < ps.j1;
            const unsigned w0 = rec[u].x;
            const unsigned sid = (w0 >> 22) & 127u;
            unsigned row = (unsigned)slot_s[w0 >> 29] + (w0 & 0x3fffffu) * (unsigned)C + (QUAD ? (unsigned)(lch * CPL) : sid);
            row = in_row ? row : 0u;  // lanes past the end of the row share one request
            const float4* qp = (const float4*)(a.Q + row * (unsigned)QW);  // < 2^31 words, checked by the host
            if (QVL == 2 && CPL == 2) {
              load_pair((const float*)qp, q[u][0], q[u][QVL - 1]);  // two channels with one 256-bit load
            } else if (QVL == 4 && CPL == 4) {
              load_pair((const float*)qp, q[u][0], q[u][1 % QVL]);
              load_pair((const float*)(qp + 2), q[u][2 % QVL], q[u][3 % QVL]);
            } else {
#pragma unroll
              for (int v = 0; v < QVL; ++v) q[u][v] = __ldcg(qp + v);
            }
            const float wt = in_row ? __uint_as_float(rec[u].y) : 0.f;
#pragma unroll
            for (int c = 0; c < CPL; ++c) w[u][c] = QUAD ? wt * basis_s[sid * R_ + lch * CPL + c] : wt;
            if (QUAD) sids |= sid << (8 * u);
          }
        };
        auto compute = [&](const Pass& ps, const float4 (&q)[UF][QVL], const float (&w)[UF][CPL], unsigned sids) {
          if (ps.fl & 1) {
#pragma unroll
            for (int b = 0; b < BP_; ++b) acc[b] = 0.f;
          }
          const unsigned zm = (unsigned)ps.kz >> 16;
          if (!zm) {
#pragma unroll
            for (int u = 0; u < UF; ++u) {
#pragma unroll
              for (int c = 0; c < CPL; ++c) {
                float4 one[QV];
#pragma unroll
                for (int v = 0; v < QV; ++v) one[v] = q[u][c * QV + v];
                float pj[BP_];
                unpack_row<BP_, PACK>(one, pj);
#pragma unroll
                for (int b = 0; b < NB; ++b) acc[b] += w[u][c] * pj[b];
              }
            }
          } else {
            // the source neuron spiked at this step in the batch rows of zm: weight gradient
#pragma unroll
            for (int u = 0; u < UF; ++u) {
              float pj[BP_];
              float dwq = 0.f;  // raw mode: this lane's share of the synapse's weight gradient
#pragma unroll
              for (int c = 0; c < CPL; ++c) {
                float4 one[QV];
#pragma unroll
                for (int v = 0; v < QV; ++v) one[v] = q[u][c * QV + v];
                unpack_row<BP_, PACK>(one, pj);
#pragma unroll
                for (int b = 0; b < NB; ++b) acc[b] += w[u][c] * pj[b];
                if (QUAD) {
                  float dws = 0.f;
#pragma unroll
                  for (int b = 0; b < NB; ++b)
                    if (zm & (1u << b)) dws += pj[b];
                  dwq += dws * basis_s[((sids >> (8 * u)) & 127u) * R_ + lch * CPL + c];
                }
              }
              const int j = ps.jb + u * SPG + lsyn;
              if (QUAD) {
                // contract with the synapse's basis row over the lanes that share the synapse
                if (LPS >= 2) dwq += __shfl_xor_sync(0xffffffffu, dwq, 1);
                if (LPS == 4) dwq += __shfl_xor_sync(0xffffffffu, dwq, 2);
                if (j < ps.j1 && lch == 0) a.dw_rec[j] += dwq;  // this lane is the only writer of the synapse
              } else if (j < ps.j1) {
                float dwv = 0.f;
#pragma unroll
                for (int b = 0; b < NB; ++b)
                  if (zm & (1u << b)) dwv += pj[b];
                a.dw_rec[j] += dwv;  // this lane is the only writer of the synapse
              }
            }
          }
          if (ps.jb + SPP >= ps.j1) reduce_store(acc, ps.kz & 0xffff);
        };
        // one turn of the pipeline with buffer I: false when the warp has no further pass
        auto turn = [&](auto I) -> bool {
          constexpr int i = decltype(I)::value;
          if (!pr.fl) {
            // accumulate what is still in flight, oldest first
#pragma unroll
            for (int o = 1; o < NS; ++o)
              if (ps_[(i + o) % NS].fl) compute(ps_[(i + o) % NS], qS[(i + o) % NS], wS[(i + o) % NS], sidS[QUAD ? (i + o) % NS : 0]);
            return false;
          }
          ps_[i] = pr;
          issue_q(ps_[i], qS[i], wS[i], sidS[QUAD ? i : 0]);
          issue_rec();
          constexpr int x = (i + 1) % NS;  // the oldest pass
          if (ps_[x].fl) {
            compute(ps_[x], qS[x], wS[x], sidS[QUAD ? x : 0]);
            ps_[x].fl = 0;
          }
          return true;
        };
        issue_rec();
        for (;;) {
          if (!turn(std::integral_constant<int, 0>{})) break;
          if (!turn(std::integral_constant<int, 1 % NS>{})) break;
          if (NS > 2 && !turn(std::integral_constant<int, 2 % NS>{})) break;
          if (NS > 3 && !turn(std::integral_constant<int, 3 % NS>{})) break;
        }
      }
    } else
    for (;;) {
      const int qi = pop_row();
      if (qi >= nq) break;
      const int k = rowq_s[qi];
      int cpost[U], csid[U];
      float cw[U];
      load_pass(rpx[k * D], rpx[k * D + D], cpost, csid, cw);
      const unsigned zm = zmask_s[k];
      const int32_t* rp = rpx + k * D;
      int bound[DMAX + 1];
#pragma unroll
      for (int d = 0; d <= DMAX; ++d) bound[d] = rp[d <= D ? d : D];
      const int j0 = bound[0], j1 = rp[D];
      float acc[BP_];
#pragma unroll
      for (int b = 0; b < BP_; ++b) acc[b] = 0.f;
      for (int jb = j0; jb < j1; jb += 32 * U) {
        if (jb != j0) load_pass(jb, j1, cpost, csid, cw);  // rows longer than one pass
        int slot[U];
        bool valid[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = jb + u * 32 + lane;
          valid[u] = j < j1;
          int d = 1;
#pragma unroll
          for (int q = 1; q < DMAX; ++q) d += (q < D && j >= bound[q]) ? 1 : 0;
          if (tg + d >= T) valid[u] = false;  // no step after the rollout's end
          slot[u] = tk + d;
          if (slot[u] >= K) slot[u] -= K;
          if (!valid[u]) {
            slot[u] = tk;
            cw[u] = 0.f;
            cpost[u] = 0;
            csid[u] = 0;
          }
        }
        float pj[U][BP_];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float* Qp = a.Q + (unsigned)((slot[u] * Np + cpost[u]) * C) * QW;  // < 2^31, checked by the host
          if (PROJ) {
            load_row<BP_, PACK>(Qp + csid[u] * QW, pj[u]);
          } else {
#pragma unroll
            for (int b = 0; b < BP_; ++b) pj[u][b] = 0.f;
#pragma unroll
            for (int r = 0; r < R_; ++r) {
              float q[BP_];
              load_row<BP_, PACK>(Qp + r * QW, q);
              const float bs = basis_s[csid[u] * R_ + r];
#pragma unroll
              for (int b = 0; b < BP_; ++b) pj[u][b] += q[b] * bs;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int b = 0; b < BP_; ++b) acc[b] += cw[u] * pj[u][b];
          if (zm && valid[u]) {
            float dwv = 0.f;
#pragma unroll
            for (int b = 0; b < BP_; ++b)
              if (zm & (1u << b)) dwv += pj[u][b];
            a.dw_rec[jb + u * 32 + lane] += dwv;  // this lane is the only writer of the synapse
          }
        }
      }
      reduce_store(acc, k);
      if (lane == 0) {
        c_rows += (unsigned long long)D;
        c_events += (unsigned long long)(j1 - j0);
        if (zm) c_dw += (unsigned long long)(j1 - j0) * __popc(zm);
      }
    }
        __syncthreads();
    if (prof) {
      const unsigned long long ph3 = gtime_b();
      ph_a += ph1 - ph0;
      ph_c += ph2 - ph1;
      ph_b += ph3 - ph2;
    }
  }
  // ---- full barrier: Q(0..D-1) of every block is in the ring ----
  __syncthreads();
  if (tid == 0) {
    if (ok && T >= 1) v1g_arrive(v1g_phase_counter(a.barrier, T));
    const unsigned long long target = v1g_phase_target(T, G);
    if (ok) {
      seen = v1g_wait(v1g_phase_counter(a.barrier, T), target, a.spin_limit, a.status);
      if (seen < target) s_misc[1] = 1;
    }
  }
  __syncthreads();
  ok = ok && !s_misc[1];
  // Spikes that were pending in the initial z_buf (emitted at step -(kb+1), bit kb) are delivered
  // at steps 0..D-1 and contribute to the recurrent weight gradient; Q(0..D-1) is still in the ring.
  if (ok && a.hist0) {
    for (int k = warp; k < cn; k += NW) {
      const int32_t* rp = rpx + k * D;
      const int j0 = rp[0], j1 = rp[D];
      for (int b = 0; b < B; ++b) {
        const unsigned hbits = a.hist0[(int64_t)b * N + n0 + k];
        if (!hbits) continue;
        for (int j = j0 + lane; j < j1; j += 32) {
          int d = 1;
          for (int q = 1; q < D; ++q) d += (j >= rp[q]) ? 1 : 0;
          const int post = a.rec_post[j], sid = a.rec_sid[j];
          float dwv = 0.f;
          for (int kb = 0; kb < D; ++kb) {
            const int sstep = d - (kb + 1);
            if (!(hbits & (1u << kb)) || sstep < 0 || sstep >= T) continue;
            const float* Qp = a.Q + qbase(sstep) + (int64_t)post * C * RS;
            float pj[BP_];
            if (PROJ) {
              load_row<BP_, PACK>(Qp + sid * RS, pj);
            } else {
#pragma unroll
              for (int bb = 0; bb < BP_; ++bb) pj[bb] = 0.f;
#pragma unroll
              for (int r = 0; r < R_; ++r) {
                float q[BP_];
                load_row<BP_, PACK>(Qp + r * RS, q);
#pragma unroll
                for (int bb = 0; bb < BP_; ++bb) pj[bb] += q[bb] * basis_s[sid * R_ + r];
              }
            }
#pragma unroll
            for (int bb = 0; bb < BP_; ++bb) dwv += (bb == b) ? pj[bb] : 0.f;
          }
          if (dwv != 0.f) a.dw_rec[j] += dwv;
        }
      }
    }
  }
  if (a.bkg_in_smem)
    for (int j = tid; j < bk_m; j += NT) a.dw_bkg[bk_base + j] += bk_dw_s[j];

  if (prof) {
    unsigned long long* o = a.phase_ns + 4 * blockIdx.x;
    o[0] = ph_c;  // dense adjoint
    o[1] = ph_b;  // gather
    o[2] = ph_a;  // wait + tape
    o[3] = gtime_b() - ph_start;
  }
  // voltage loss and counters
  for (int o = 16; o > 0; o >>= 1) volt_loss += __shfl_down_sync(0xffffffffu, volt_loss, o);
  c_rows = v1g_warp_sum(c_rows);
  c_events = v1g_warp_sum(c_events);
  c_dw = v1g_warp_sum(c_dw);
  if (lane == 0) {
    if (volt_loss != 0.f) atomicAdd(a.loss_acc + 2, volt_loss * a.volt_coef);
    V1GCounters* c = (V1GCounters*)a.counters;
    if (c_rows) atomicAdd(&c->bwd_rows, c_rows);
    if (c_events) atomicAdd(&c->bwd_events, c_events);
    if (c_dw) atomicAdd(&c->dw_events, c_dw);
  }
}

// ---- loss preparation over the saved spikes ------------------------------------------------

// rate_coef[n] = rate_cost*ls*2*(m_n - target_n)/(N*B*T); loss[1] = rate loss
__global__ void __launch_bounds__(256) rate_loss_kernel(const int* __restrict__ spike_count,
                                                        const float* __restrict__ target, int N,
                                                        float inv_bt, float cost, float* rate_coef,
                                                        float* loss) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  float l = 0.f;
  if (n < N) {
    const float m = (float)spike_count[n] * inv_bt;
    const float dlt = m - target[n];
    rate_coef[n] = cost * 2.f * dlt / (float)N * inv_bt;
    l = dlt * dlt;
  }
  __shared__ float ws[8];
  for (int o = 16; o > 0; o >>= 1) l += __shfl_down_sync(0xffffffffu, l, o);
  if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = l;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += ws[w];
    atomicAdd(loss + 1, cost * s / (float)N);
  }
}

// Fano-factor loss of the population spike count in bins of `bin` steps (one block).
// sgrad[b*nbins + k] = dL/d(count of bin k, row b); loss[3] = synchrony loss.
__global__ void __launch_bounds__(256) sync_loss_kernel(const int* __restrict__ popcount, int T, int B,
                                                        int bin, int nbins, float cost, float target,
                                                        float* __restrict__ sgrad, float* loss) {
  extern __shared__ float sh[];  // counts [B*nbins], then mean[B], var[B], fano[B]
  float* cnt = sh;
  float* mean = sh + B * nbins;
  float* var = mean + B;
  float* fano = var + B;
  for (int i = threadIdx.x; i < B * nbins; i += blockDim.x) {
    const int b = i / nbins, k = i - b * nbins;
    int s = 0;
    for (int q = 0; q < bin; ++q) s += popcount[(k * bin + q) * B + b];
    cnt[i] = (float)s;
  }
  __syncthreads();
  if (threadIdx.x < B) {
    const int b = threadIdx.x;
    float m = 0.f;
    for (int k = 0; k < nbins; ++k) m += cnt[b * nbins + k];
    m /= (float)nbins;
    float v = 0.f;
    for (int k = 0; k < nbins; ++k) {
      const float d = cnt[b * nbins + k] - m;
      v += d * d;
    }
    v /= (float)nbins;
    mean[b] = m;
    var[b] = v;
    fano[b] = v / fmaxf(m, 1e-7f);
  }
  __syncthreads();
  float fbar = 0.f;
  for (int b = 0; b < B; ++b) fbar += fano[b];
  fbar /= (float)B;
  const float dl_df = cost * 2.f * (fbar - target) / (float)B;
  for (int i = threadIdx.x; i < B * nbins; i += blockDim.x) {
    const int b = i / nbins;
    const float m = mean[b], v = var[b];
    const float dv = 2.f * (cnt[i] - m) / (float)nbins;
    float df;
    if (m > 1e-7f)
      df = dv / m - v / (m * m) / (float)nbins;
    else
      df = dv / 1e-7f;
    sgrad[i] = dl_df * df;
  }
  if (threadIdx.x == 0) atomicAdd(loss + 3, cost * (fbar - target) * (fbar - target));
}

__global__ void __launch_bounds__(256) permute_add_kernel(const float* __restrict__ src,
                                                          const int32_t* __restrict__ perm,
                                                          float* __restrict__ dst, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[perm ? perm[i] : i] += src[i];
}

__global__ void finish_loss_kernel(float* acc, float* out) {
  if (threadIdx.x == 0) {
    acc[0] = acc[1] + acc[2] + acc[3];
    if (out)
      for (int i = 0; i < 4; ++i) out[i] = acc[i];
  }
}

template <int R_, int BP_, bool PROJ, int DT, bool PACK, bool PAIR = false>
int launch_bwd_d(V1GHandle* h, const BwdArgs& a, int grid, size_t smem, cudaStream_t st) {
  auto kern = rollout_bwd_kernel<R_, BP_, PROJ, DT, PACK, PAIR>;
  V1G_CUDA(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int per_sm = 0;
  V1G_CUDA(h, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NT, smem));
  if (per_sm < 1 || grid > per_sm * h->n_sms)
    return v1g_fail(h, V1G_ERANGE, "rollout grid of %d blocks cannot be co-resident (%d per SM)", grid, per_sm);
  void* args[] = {(void*)&a};
  V1G_CUDA(h, cudaEventRecord(h->ev[2], st));
  V1G_CUDA(h, cudaLaunchCooperativeKernel((void*)kern, dim3(grid), dim3(NT), args, smem, st));
  V1G_CUDA(h, cudaEventRecord(h->ev[3], st));
  h->ev_valid[1] = true;
  v1g_count_launches(1);
  return V1G_OK;
}

template <int R_, int BP_, bool PROJ, bool PACK>
int launch_bwd(V1GHandle* h, const BwdArgs& a, int grid, size_t smem, cudaStream_t st) {
  if (a.D == 5) return launch_bwd_d<R_, BP_, PROJ, 5, PACK>(h, a, grid, smem, st);
  return launch_bwd_d<R_, BP_, PROJ, 0, PACK>(h, a, grid, smem, st);
}

// paired rows: projected mode with 16-byte rows (batch <= 4 in fp32, batch 5 as 24-bit floats)
template <int R_, int BP_, bool PACK>
int launch_bwd_pair(V1GHandle* h, const BwdArgs& a, int grid, size_t smem, cudaStream_t st) {
  if (a.D == 5) return launch_bwd_d<R_, BP_, true, 5, PACK, true>(h, a, grid, smem, st);
  return launch_bwd_d<R_, BP_, true, 0, PACK, true>(h, a, grid, smem, st);
}

template <int R_>
int launch_bwd_r(V1GHandle* h, const BwdArgs& a, int BP, bool proj, bool pack, bool pair, int grid, size_t smem,
                 cudaStream_t st) {
  if (pair)
    return BP == 4 ? launch_bwd_pair<R_, 4, false>(h, a, grid, smem, st)
                   : launch_bwd_pair<R_, 8, true>(h, a, grid, smem, st);
  if (BP == 4)
    return proj ? launch_bwd<R_, 4, true, false>(h, a, grid, smem, st)
                : launch_bwd<R_, 4, false, false>(h, a, grid, smem, st);
  if (pack)
    return proj ? launch_bwd<R_, 8, true, true>(h, a, grid, smem, st)
                : launch_bwd<R_, 8, false, true>(h, a, grid, smem, st);
  return proj ? launch_bwd<R_, 8, true, false>(h, a, grid, smem, st)
              : launch_bwd<R_, 8, false, false>(h, a, grid, smem, st);
}

}  // namespace

// internal_order: d_w_* are buffers in the library's own synapse order (presynaptic CSR for the
// recurrent and LGN sources, gather-table order for the background) that the kernel accumulates
// into directly; otherwise they are in the caller's order and filled through a permutation.
static int rollout_bwd_impl(V1GHandle* h, const V1GLossSpec* loss, const float* g_z, const float* g_v,
                            float* d_w_rec, float* d_w_lgn, float* d_w_bkg, float* loss_out,
                            bool internal_order, void* stream) {
  if (!h) return V1G_EINVAL;
  if (!h->tape_valid)
    return v1g_fail(h, V1G_ESTATE, "v1g_rollout_bwd needs a preceding v1g_rollout_fwd with save_for_bwd");
  cudaStream_t st = (cudaStream_t)stream;
  const V1GConfig& c = h->cfg;
  const int N = c.n_neurons, R = c.n_receptors, D = c.max_delay, K = D + 3, S = c.n_syn_types;
  const int B = h->tape_B, T = h->tape_T;
  if (R != 4 && R != 5)
    return v1g_fail(h, V1G_ERANGE, "backward rollout is built for 4 or 5 receptor channels, got %d", R);
  V1GLossSpec ls;
  if (loss) ls = *loss; else ls = V1GLossSpec{nullptr, nullptr, 0.f, 0.f, 0.f, 1.f, 50, 1.f};
  const bool rate_groups = ls.n_rate_groups > 0;
  if (ls.rate_cost != 0.f && !ls.rate_target && !rate_groups)
    return v1g_fail(h, V1G_EINVAL, "rate_cost without rate_target or rate populations");
  const bool proj = S <= 8;
  const int C = proj ? S : R;
  const int BP = B <= 4 ? 4 : 8;
  const bool pack = (B == 5) && !h->opt_no_q_pack;  // five 24-bit floats per 16-byte row
  const int QW = pack ? 4 : BP;
  const int Np = (N + 31) & ~31;
  int rc;

  V1GRolloutPlan plan;
  v1g_plan_rollout(h, B, 3 + 2 * R, 0, 0, &plan);
  plan.chunkP = (plan.chunk + 3) & ~3;  // planes only need 16-byte alignment here
  if (plan.chunkP > 65535) return v1g_fail(h, V1G_ERANGE, "slice of %d neurons per block exceeds 65535", plan.chunkP);
  auto al = [](size_t b) { return (b + 15) & ~(size_t)15; };
  const size_t plane = (size_t)B * plan.chunkP;
  // packed-record gather: projected rows, or raw rows of four channels in 16 bytes each (lane quads)
  const bool fast = (proj || (R == 4 && QW == 4)) && !h->opt_no_meta && h->src[V1G_SRC_REC].syn8 != nullptr &&
                    h->src[V1G_SRC_REC].nnz > 0;
  // paired rows (two steps per 32-byte row): 16-byte rows, packed records, one neuron per thread
  bool pair = fast && proj && QW == 4 && plan.chunk <= NT && h->opt_pair_rows;
  const int KP = ((D + 3) >> 1) + 1;  // pair slots covering D+3 consecutive steps at either alignment
  if (pair && (rc = v1g_build_pair_tables(h, st))) return rc;
  // a delay parity without any entry leaves nothing to clamp the lanes past a row's end to
  if (pair && std::min(h->src[V1G_SRC_REC].pair_len[0], h->src[V1G_SRC_REC].pair_len[1]) < 1) pair = false;
  size_t smem = al(sizeof(float) * S * R) + 2 * al(sizeof(float) * 2 * plane) + al(pair ? 0 : 2 * plane) +
                al(pair ? 2 * plan.chunkP : plan.chunkP) + al(sizeof(int) * B * c.n_bkg) + al(sizeof(int) * 8) +
                al(sizeof(int) * 8) + al(pair ? 0 : sizeof(uint16_t) * plan.chunkP) +
                al(sizeof(int4) * plan.chunkP) +
                (fast ? 0 : al(sizeof(int32_t) * ((size_t)plan.chunkP * D + 1))) +
                al(sizeof(int) * (plan.chunkP + 1));
  const size_t state_bytes = al(sizeof(float) * plane * (3 + 2 * R));
  int state_in_smem = 0;
  if (!h->opt_force_global && smem + state_bytes <= std::min<size_t>((size_t)h->smem_optin, 195 * 1024)) {
    state_in_smem = 1;
    smem += state_bytes;
  }
  int bkg_cap = 0;
  {
    const V1GSource& bk0 = h->src[V1G_SRC_BKG];
    for (int g = 0; g < plan.grid; ++g) {
      const int a0 = g * plan.chunk, a1 = std::min(N, a0 + plan.chunk);
      bkg_cap = std::max(bkg_cap, bk0.in_ptr_host[a1] - bk0.in_ptr_host[a0]);
    }
  }
  const size_t bkg_bytes = al(sizeof(int) * bkg_cap) + al(sizeof(float) * bkg_cap) + al(bkg_cap);
  // The L1 cache is what is left of the SM's 256 KB after the shared-memory carve-out, and it holds
  // the sectors of the gather's loads in flight: with less than ~60 KB of it the gather runs at half
  // speed.  The background tables therefore go on chip only while the block stays below 195 KB.
  int bkg_in_smem = 0;
  if (smem + bkg_bytes <= std::min<size_t>((size_t)h->smem_optin, 195 * 1024)) {
    bkg_in_smem = 1;
    smem += bkg_bytes;
  }
  if (smem > (size_t)h->smem_optin)
    return v1g_fail(h, V1G_ERANGE, "backward rollout needs %zu B of shared memory per block", smem);
  if (!state_in_smem)
    if ((rc = v1g_reserve(h, &h->state_ws, &h->state_ws_cap, (int64_t)(plane * (3 + 2 * R) * plan.grid)))) return rc;

  // scratch: Q ring, CSR-order weight gradients, loss tables
  const int64_t q_elems = pair ? (int64_t)KP * Np * C * 2 * QW : (int64_t)K * Np * C * QW;
  if (q_elems >= 0x7fffffffLL) return v1g_fail(h, V1G_ERANGE, "backward Q ring of %lld elements exceeds 32-bit indexing", (long long)q_elems);
  if ((rc = v1g_reserve(h, &h->dy_ring, &h->dy_ring_cap, q_elems))) return rc;
  const bool sync_samples = ls.sync_cost != 0.f && ls.n_sync_samples > 0;
  const int nbins = (ls.sync_cost != 0.f && !sync_samples && ls.sync_bin > 0) ? T / ls.sync_bin : 0;
  // loss scratch layout (floats): acc[4] | rate_coef[N] | sgrad[B*nbins] | spike_count[N] (int) | popcount[T*B] (int)
  const int64_t ls_elems = 4 + (int64_t)N + (int64_t)B * std::max(nbins, 1) + N + (int64_t)T * B;
  if ((rc = v1g_reserve(h, &h->loss_scratch, &h->loss_scratch_cap, ls_elems))) return rc;
  float* acc = h->loss_scratch;
  float* rate_coef = acc + 4;
  float* sgrad = rate_coef + N;
  int* spike_count = (int*)(sgrad + (int64_t)B * std::max(nbins, 1));
  int* popcount = spike_count + N;
  float* dw_int[V1G_NSRC] = {d_w_rec, d_w_lgn, d_w_bkg};
  for (int s = 0; s < V1G_NSRC; ++s) {
    if (internal_order && dw_int[s]) continue;  // the caller's buffer is accumulated into directly
    const int64_t nnz = std::max<int64_t>(h->src[s].nnz, 1);
    if (!h->dw_csr[s]) V1G_CUDA(h, cudaMalloc((void**)&h->dw_csr[s], (size_t)nnz * sizeof(float)));
    V1G_CUDA(h, cudaMemsetAsync(h->dw_csr[s], 0, (size_t)nnz * sizeof(float), st));
    dw_int[s] = h->dw_csr[s];
  }
  V1G_CUDA(h, cudaMemsetAsync(h->loss_scratch, 0, (size_t)ls_elems * sizeof(float), st));
  V1G_CUDA(h, cudaMemsetAsync(h->dy_ring, 0, (size_t)q_elems * sizeof(float), st));
  V1G_CUDA(h, cudaMemsetAsync(h->barrier, 0, V1G_BARRIER_BYTES, st));

  const bool want_rate = ls.rate_cost != 0.f, want_sync = nbins >= 1;
  if (want_rate || want_sync) {
    // spike counts per neuron and per (step, batch row) come from the forward kernel
    spike_count = h->tape_stats;
    popcount = h->tape_stats + N;
    v1g_count_launches(((want_rate && !rate_groups) ? 1 : 0) + (want_sync ? 1 : 0));
    if (want_rate && rate_groups) {
      if ((rc = v1g_rate_distribution_loss(h, &ls, spike_count, B, T, rate_coef, acc + 1, st))) return rc;
    } else if (want_rate) {
      rate_loss_kernel<<<(N + 255) / 256, 256, 0, st>>>(spike_count, ls.rate_target, N,
                                                       1.f / ((float)B * (float)T),
                                                       ls.rate_cost * ls.loss_scale, rate_coef, acc);
    }
    if (want_sync)
      sync_loss_kernel<<<1, 256, sizeof(float) * (B * nbins + 3 * B), st>>>(
          popcount, T, B, ls.sync_bin, nbins, ls.sync_cost * ls.loss_scale, ls.fano_target, sgrad, acc);
    V1G_CUDA(h, cudaGetLastError());
  }

  V1GSyncTables sync_tables;
  sync_tables.first = nullptr;
  if (sync_samples)
    if ((rc = v1g_sync_samples_loss(h, &ls, B, T, acc + 3, &sync_tables, st))) return rc;

  const float* osi_coef = nullptr;
  int osi_t0 = 0, osi_t1 = 0;
  if ((rc = v1g_osi_dsi_loss(h, &ls, B, T, acc + 3, &osi_coef, &osi_t0, &osi_t1, st))) return rc;

  BwdArgs a;
  a.sync = sync_tables;
  a.osi_coef = osi_coef; a.osi_t0 = osi_t0; a.osi_t1 = osi_t1;
  a.N = N; a.D = D; a.K = K; a.KP = KP; a.B = B; a.T = T; a.Np = Np;
  a.chunk = plan.chunk; a.chunkP = plan.chunkP; a.S = S; a.C = C; a.n_bkg = c.n_bkg;
  a.state_in_smem = state_in_smem;
  a.bkg_in_smem = bkg_in_smem;
  a.bkg_cap = bkg_cap;
  const V1GSource& rs = h->src[V1G_SRC_REC];
  const V1GSource& lsrc = h->src[V1G_SRC_LGN];
  const V1GSource& bk = h->src[V1G_SRC_BKG];
  a.rec_rowptr = rs.rowptr; a.rec_post = rs.post; a.rec_w = rs.w; a.rec_sid = rs.sid;
  a.rec_syn8 = fast ? rs.syn8 : nullptr;
  for (int p2 = 0; p2 < 2; ++p2) {
    a.pair_ptr[p2] = rs.pair_ptr[p2];
    a.pair_rec[p2] = rs.pair_rec[p2];
    a.pair_j[p2] = rs.pair_j[p2];
  }
  a.pair_last[0] = (int)rs.pair_len[0] - 1;
  a.pair_last[1] = (int)rs.pair_len[1] - 1;
  a.rec_nnz = (int)rs.nnz;
  a.lgn_rowptr = lsrc.rowptr; a.lgn_post = lsrc.post; a.lgn_sid = lsrc.sid;
  a.bkg_inptr = bk.in_ptr; a.bkg_inpre = bk.in_pre; a.bkg_insid = bk.in_sid;
  a.decay = h->decay; a.cf = h->cf; a.asc_decay = h->asc_decay; a.basis = h->basis;
  for (int r = 0; r < V1G_MAX_RECEPTORS; ++r) {
    a.sd[r] = r < R ? h->syn_decay[r] : 0.f;
    a.pinit[r] = r < R ? h->psc_initial[r] : 0.f;
    a.dtsd[r] = c.dt * a.sd[r];
  }
  a.lr_scale = c.lr_scale; a.vd_keep = h->vd_keep; a.rec_factor = h->rec_grad_factor;
  a.damp = c.dampening_factor; a.inv_width = 1.f / c.pseudo_width; a.gauss_std = c.gauss_std;
  a.gauss = (c.flags & V1G_FLAG_PSEUDO_GAUSS) ? 1 : 0;
  a.hard_reset = (c.flags & V1G_FLAG_HARD_RESET) ? 1 : 0;
  a.csr_evict_first = h->opt_csr_evict_first;
  a.tape_v = h->tape_v;
  a.hist0 = h->tape_has_hist0 ? h->tape_hist0 : nullptr;
  a.lgn_off = h->lgn_offsets; a.lgn_ent4 = h->lgn_ent4; a.lgn_nseg = h->lgn_nseg;
  a.bkg_counts = h->tape_counts;
  a.rate_coef = want_rate ? rate_coef : nullptr;
  a.rate_t0 = rate_groups ? std::max(ls.rate_pre_delay, 0) : 0;
  a.rate_t1 = rate_groups ? T - std::max(ls.rate_post_delay, 0) : T;
  a.sgrad = want_sync ? sgrad : nullptr;
  a.sync_bin = ls.sync_bin; a.nbins = nbins;
  a.volt_coef = ls.voltage_cost * ls.loss_scale / ((float)B * (float)T * (float)N);
  a.volt_threshold_mode = ls.voltage_mode == 1 ? 1 : 0;
  a.v_lo = ls.v_lo;
  a.g_z = g_z; a.g_v = g_v;
  a.dw_rec = dw_int[V1G_SRC_REC]; a.dw_lgn = dw_int[V1G_SRC_LGN]; a.dw_bkg = dw_int[V1G_SRC_BKG];
  a.loss_acc = acc;
  a.Q = h->dy_ring; a.state_ws = h->state_ws;
  a.barrier = h->barrier; a.status = h->dev_status; a.counters = h->counters;
  a.spin_limit = h->opt_spin_limit;
  a.phase_ns = nullptr;
  if (h->opt_phase_timers) {
    if ((rc = v1g_reserve(h, &h->phase_ns, &h->phase_ns_cap, (int64_t)4 * plan.grid))) return rc;
    V1G_CUDA(h, cudaMemsetAsync(h->phase_ns, 0, sizeof(unsigned long long) * 4 * plan.grid, st));
    a.phase_ns = h->phase_ns;
    h->phase_grid = plan.grid;
  }
  // keep the Q ring resident in L2 (it is gathered at random, one sector per synapse and step)
  if (h->opt_l2_window) {
    cudaDeviceProp prop;
    V1G_CUDA(h, cudaGetDeviceProperties(&prop, h->device));
    const size_t q_bytes = (size_t)q_elems * sizeof(float);
    if (prop.persistingL2CacheMaxSize > 0 && prop.accessPolicyMaxWindowSize > 0) {
      const size_t carve = std::min<size_t>((size_t)prop.persistingL2CacheMaxSize, q_bytes);
      V1G_CUDA(h, cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, carve));
      cudaStreamAttrValue attr;
      attr.accessPolicyWindow.base_ptr = h->dy_ring;
      attr.accessPolicyWindow.num_bytes = std::min<size_t>(q_bytes, (size_t)prop.accessPolicyMaxWindowSize);
      attr.accessPolicyWindow.hitRatio = (float)std::min(1.0, (double)carve / (double)attr.accessPolicyWindow.num_bytes);
      attr.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
      attr.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
      V1G_CUDA(h, cudaStreamSetAttribute(st, cudaStreamAttributeAccessPolicyWindow, &attr));
    }
  }
  rc = (R == 4) ? launch_bwd_r<4>(h, a, BP, proj, pack, pair, plan.grid, smem, st)
                : launch_bwd_r<5>(h, a, BP, proj, pack, pair, plan.grid, smem, st);
  if (h->opt_l2_window) {
    cudaStreamAttrValue attr;
    attr.accessPolicyWindow.base_ptr = nullptr;
    attr.accessPolicyWindow.num_bytes = 0;
    attr.accessPolicyWindow.hitRatio = 0.f;
    attr.accessPolicyWindow.hitProp = cudaAccessPropertyNormal;
    attr.accessPolicyWindow.missProp = cudaAccessPropertyNormal;
    cudaStreamSetAttribute(st, cudaStreamAttributeAccessPolicyWindow, &attr);
  }
  if (rc) return rc;

  // weight gradients back to the caller's synapse order, accumulated
  const int blocks = h->n_sms * 8;
  if (internal_order) {
    finish_loss_kernel<<<1, 32, 0, st>>>(acc, loss_out);
    v1g_count_launches(1);
    V1G_CUDA(h, cudaGetLastError());
    return V1G_OK;
  }
  if (d_w_rec && rs.nnz) permute_add_kernel<<<blocks, 256, 0, st>>>(h->dw_csr[V1G_SRC_REC], rs.perm, d_w_rec, rs.nnz);
  if (d_w_lgn && lsrc.nnz) permute_add_kernel<<<blocks, 256, 0, st>>>(h->dw_csr[V1G_SRC_LGN], lsrc.perm, d_w_lgn, lsrc.nnz);
  if (d_w_bkg && bk.nnz) permute_add_kernel<<<blocks, 256, 0, st>>>(h->dw_csr[V1G_SRC_BKG], bk.in_perm, d_w_bkg, bk.nnz);
  finish_loss_kernel<<<1, 32, 0, st>>>(acc, loss_out);
  v1g_count_launches(1 + ((d_w_rec && rs.nnz) ? 1 : 0) + ((d_w_lgn && lsrc.nnz) ? 1 : 0) + ((d_w_bkg && bk.nnz) ? 1 : 0));
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

extern "C" int v1g_rollout_bwd(V1GHandle* h, const V1GLossSpec* loss, const float* g_z,
                               const float* g_v, float* d_w_rec, float* d_w_lgn, float* d_w_bkg,
                               float* loss_out, void* stream) {
  return rollout_bwd_impl(h, loss, g_z, g_v, d_w_rec, d_w_lgn, d_w_bkg, loss_out, false, stream);
}

extern "C" int v1g_rollout_bwd_internal(V1GHandle* h, const V1GLossSpec* loss, const float* g_z,
                                        const float* g_v, float* grads_flat, float* loss_out,
                                        void* stream) {
  if (!h) return V1G_EINVAL;
  if (!grads_flat) return v1g_fail(h, V1G_EINVAL, "v1g_rollout_bwd_internal: null gradient buffer");
  float* g0 = grads_flat;
  float* g1 = g0 + h->src[V1G_SRC_REC].nnz;
  float* g2 = g1 + h->src[V1G_SRC_LGN].nnz;
  return rollout_bwd_impl(h, loss, g_z, g_v, g0, g1, g2, loss_out, true, stream);
}
