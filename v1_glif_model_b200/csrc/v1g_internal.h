// Internal definitions shared by the translation units of libv1g.so (not part of the C ABI).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include <vector>

#include "v1g.h"

#define V1G_NSRC 3

// Device-side status word values (written by kernels, read by v1g_synchronize).
#define V1G_DEV_OK 0
#define V1G_DEV_BARRIER_TIMEOUT 1

// One synaptic source: presynaptic CSR (scatter / transposed gather) + post-major gather table.
struct V1GSource {
  int64_t nnz = 0;
  int64_t n_cols = 0;  // columns of the reference's dense_shape[1] (D*N for REC)
  int n_src = 0;       // source neurons (N for REC, n_lgn, n_bkg)
  int delays = 1;      // delay buckets per source neuron (D for REC, else 1)
  // presynaptic CSR, rows numbered src*delays + (d-1): the `delays` buckets of one source neuron
  // are contiguous, each bucket holding the same entries in the same order as row
  // src + n_src*(d-1) of the reference's pre_ind_table
  int32_t* rowptr = nullptr;  // [n_cols + 1]
  int32_t* post = nullptr;    // [nnz]
  float* w = nullptr;         // [nnz] weights in CSR order
  uint8_t* sid = nullptr;     // [nnz]
  int32_t* perm = nullptr;    // [nnz] CSR position -> position in the caller's arrays
  uint8_t* pos_int = nullptr; // [nnz] sign mask (w >= 0 at the first v1g_set_weights), internal order
  bool pos_set = false;
  // [nnz] packed synapse records for the rollout kernels (recurrent and LGN sources, when N < 2^22
  // and S <= 128): x = post | sid << 22 | (delay-1) << 29, y = bits of the weight (kept equal to w)
  uint2* syn8 = nullptr;
  // post-major table in the caller's order (the reference sorts synapses by post, so this is a
  // plain row pointer over the caller's arrays)
  int32_t* in_ptr = nullptr;  // [N + 1]
  int32_t* in_pre = nullptr;  // [nnz] source column of each synapse, caller's order
  uint8_t* in_sid = nullptr;  // [nnz]
  float* w_ref = nullptr;     // [nnz] weights, caller's order
  // only when the caller's arrays are not grouped by post: the gather table is a stable sort by
  // post, in_perm maps its positions to the caller's, w_in holds the weights in table order
  int32_t* in_perm = nullptr;
  float* w_in = nullptr;
  bool post_sorted = false;
  const float* gather_w() const { return in_perm ? w_in : w_ref; }
  float* gather_w_mut() { return in_perm ? w_in : w_ref; }
  // host copy of the reference-numbered table for v1g_get_pre_ind_table
  std::vector<int32_t> order_host;
  std::vector<int64_t> row_splits_host;
  std::vector<int32_t> in_ptr_host;  // host copy of in_ptr
  // Recurrent source, built on first use of the paired backward ring: per delay parity p the records
  // of every source neuron in gather order (its delay-1 bucket, then its buckets of delay d >= 2 with
  // d - 1 = 1 + p, 3 + p, ...), the row starts and the CSR position of every entry.
  std::vector<int32_t> rowptr_host;   // host copy of rowptr
  std::vector<uint32_t> syn8x_host;   // host copy of the first word of syn8
  int32_t* pair_ptr[2] = {nullptr, nullptr};  // [n_src + 1]
  uint2* pair_rec[2] = {nullptr, nullptr};
  int32_t* pair_j[2] = {nullptr, nullptr};
  int64_t pair_len[2] = {0, 0};
  bool pair_built = false;
};

struct V1GHandle {
  V1GConfig cfg;
  int device = 0;
  int n_sms = 0;
  int smem_optin = 0;
  mutable std::string err;
  V1GSource src[V1G_NSRC];
  bool params_set = false;
  // keys of the device-side background sampler (models.py:506, 869-877)
  int64_t noise_seed = 0;
  int32_t noise_replica = 0;
  // per-neuron constants (device)
  float *decay = nullptr, *cf = nullptr, *asc_decay = nullptr, *asc_amps = nullptr;
  int32_t* tref = nullptr;
  float* basis = nullptr;  // [S*R]
  float syn_decay[V1G_MAX_RECEPTORS], psc_initial[V1G_MAX_RECEPTORS];
  // straight-through factors computed in fp32 exactly as the reference does
  float vd_keep = 1.f, vd_drop = 0.f;  // (1-d), d of the voltage self-loop
  float rec_grad_factor = 1.f;         // 1 - clip(1 - recurrent_dampening)

  // ---- scratch (grown on demand, freed in v1g_destroy) ----
  int32_t* seg_counts = nullptr;  // compaction: per-segment counts / offsets
  int64_t seg_cap = 0;
  int64_t* coords = nullptr;  // op-level active list (row, col)
  int64_t coords_cap = 0;
  int32_t* d_count = nullptr;  // device int for counts
  int32_t* h_count = nullptr;  // pinned host mirror
  uint32_t* lgn_entries = nullptr;
  uint4* lgn_ent4 = nullptr;  // the same events resolved: {batch row << 24 | unit, first synapse, end, 0}
  int64_t lgn_ent4_cap = 0;
  int64_t lgn_entries_cap = 0;
  int32_t* lgn_offsets = nullptr;  // [T*B*nseg + 1]
  int64_t lgn_offsets_cap = 0;
  int lgn_nseg = 0;
  float* ring = nullptr;  // current ring [K][B][R][Np]
  int64_t ring_cap = 0;
  float* state_ws = nullptr;  // rollout state when it does not fit in shared memory
  int64_t state_ws_cap = 0;
  unsigned long long* barrier = nullptr;  // [0] = barrier counter
  int32_t* dev_status = nullptr;          // device status word
  unsigned long long* counters = nullptr;  // V1GCounters on the device
  // saved forward for BPTT
  float* tape_v = nullptr;    // [T][B][N]
  int64_t tape_cap = 0;
  uint8_t* tape_hist0 = nullptr;  // [B][N] spike-history bits of the initial z_buf of the saved rollout
  int64_t tape_hist0_cap = 0;
  bool tape_has_hist0 = false;
  int tape_B = 0, tape_T = 0;
  bool tape_valid = false;
  // spike statistics of the saved rollout, counted by the forward kernel: [N] spikes per neuron
  // (all batch rows and steps) followed by [T*B] population spikes per (step, batch row)
  int32_t* tape_stats = nullptr;
  int64_t tape_stats_cap = 0;
  // forward slices balanced by scatter work (v1g_balance_slices): first neuron of every block's slice,
  // [grid + 1], on the device and on the host; empty = equal slices
  int32_t* fwd_slice = nullptr;
  std::vector<int32_t> fwd_slice_host;
  const int32_t* tape_counts = nullptr;  // background counts of the saved rollout (= tape_counts_buf)
  int32_t* tape_counts_buf = nullptr;    // handle-owned copy [B][T][n_bkg]
  int64_t tape_counts_cap = 0;
  // backward scratch
  float* dy_ring = nullptr;
  int64_t dy_ring_cap = 0;
  float* dw_csr[V1G_NSRC] = {nullptr, nullptr, nullptr};
  float* osi_scratch = nullptr;  // spike counts, segment sums and the [B][N] gradient table of the OSI/DSI target
  int64_t osi_scratch_cap = 0;
  int32_t* sync_scratch = nullptr;  // membership lists, population counts and gradients of the synchrony samples
  int64_t sync_scratch_cap = 0;
  int32_t* rate_scratch = nullptr;  // sort buffers of the rate-distribution target
  int64_t rate_scratch_cap = 0;
  int32_t* reg_scratch = nullptr;  // group sums / sort buffers of the weight regularisers
  int64_t reg_scratch_cap = 0;
  float* loss_scratch = nullptr;  // rate sums [N], pop counts [B][T], bin grads, partial losses
  int64_t loss_scratch_cap = 0;
  // staging for the host-buffer entry point
  uint8_t* stage_x = nullptr;
  int32_t* stage_counts = nullptr;
  uint8_t* stage_z = nullptr;
  float* stage_v = nullptr;
  int64_t stage_x_cap = 0, stage_counts_cap = 0, stage_z_cap = 0, stage_v_cap = 0;
  // pipelined host-buffer entry point: copy streams, events, bit-packed spikes, carried state
  cudaStream_t pipe_in = nullptr, pipe_out = nullptr;
  cudaEvent_t pipe_ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  uint32_t* stage_bits = nullptr;
  int64_t stage_bits_cap = 0;
  float* pipe_state = nullptr;
  int64_t pipe_state_cap = 0;
  // tuning (tests shrink these to exercise multi-block paths on tiny nets)
  int opt_chunk = 0;          // neurons per block in the rollout kernels (0 = auto)
  int opt_force_global = 0;   // keep rollout state in global memory even if it fits on chip
  long long opt_spin_limit = 4000000LL;
  int opt_force_smem_kernel = 0;  // never pick the register-resident forward kernel
  int opt_no_meta = 0;            // backward gather reads post / sid / w arrays instead of the packed records
  int opt_no_q_pack = 0;          // keep the backward Q rows in fp32 even for a batch of 5
  int opt_pair_rows = 0;          // two steps per 32-byte row in the backward ring where the layout allows it
  int opt_l2_window = 0;          // pin the backward Q ring in L2 with an access-policy window
  int opt_csr_evict_first = 1;    // read the backward synapse stream with evict-first loads
  int opt_phase_timers = 0;   // record per-block phase times of the rollout kernels
  unsigned long long* phase_ns = nullptr;
  int64_t phase_ns_cap = 0;
  int phase_grid = 0;
  // CUDA events bracketing the last forward [0,1] and backward [2,3] rollout kernel
  cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
  bool ev_valid[2] = {false, false};
};

int v1g_fail(const V1GHandle* h, int code, const char* fmt, ...);

// process-wide count of kernel launches made by this library (for the bench's gpu_launches)
void v1g_count_launches(int n);

// message returned by v1g_last_error(NULL), for entry points that take no handle
void v1g_set_global_error(const char* msg);

// gather-ordered record tables of the recurrent source for the paired backward ring (built once)
int v1g_build_pair_tables(V1GHandle* h, cudaStream_t st);

#define V1G_CUDA(h, call)                                                              \
  do {                                                                                 \
    cudaError_t e_ = (call);                                                           \
    if (e_ != cudaSuccess)                                                             \
      return v1g_fail(h, e_ == cudaErrorMemoryAllocation ? V1G_ENOMEM : V1G_ECUDA,     \
                      "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, \
                      __LINE__);                                                       \
  } while (0)

// Grow-only device buffer helper: keeps contents undefined after growth.
template <typename T>
int v1g_reserve(V1GHandle* h, T** p, int64_t* cap, int64_t need) {
  if (need <= *cap && *p) return V1G_OK;
  if (*p) {
    V1G_CUDA(h, cudaFree(*p));
    *p = nullptr;
    *cap = 0;
  }
  if (need < 1) need = 1;
  V1G_CUDA(h, cudaMalloc((void**)p, (size_t)need * sizeof(T)));
  *cap = need;
  return V1G_OK;
}

// ---- synchrony target over given samples (v1g_losses.cu) ----
struct V1GSyncTables {
  const int32_t* first;       // [N] first membership position of a neuron, -1 = in no sample (NULL: term off)
  const int32_t* next;        // [P] next membership position of the same neuron, -1 = end
  const int32_t* pos_sample;  // [P] sample of a membership position
  const int32_t* trial;       // [S] batch row of a sample
  const float* g;             // [S][W] d loss / d population count
  int t0, W;
};
int v1g_sync_samples_loss(V1GHandle* h, const V1GLossSpec* ls, int B, int T, float* loss_acc,
                          V1GSyncTables* out, cudaStream_t st);

// ---- population OSI/DSI target (v1g_losses.cu) ----
int v1g_osi_dsi_loss(V1GHandle* h, const V1GLossSpec* ls, int B, int T, float* loss_acc, const float** coef_out,
                     int* t0_out, int* t1_out, cudaStream_t st);

// ---- rate-distribution target (v1g_losses.cu) ----
int v1g_rate_distribution_loss(V1GHandle* h, const V1GLossSpec* ls, const int32_t* count, int B, int T,
                               float* rate_coef, float* loss_acc, cudaStream_t st);

// ---- ordered compaction (v1g_compact.cu) ----
// Input viewed as [n_rows][n_cols]; positives are listed in output order.  time_major_T > 0:
// rows are (b, t) = (row / T, row % T) and the output is ordered (t, b, col); otherwise (row, col).
// offsets[] gets the exclusive scan per (ordered) segment, offsets[n_segments] the total.
enum V1GCompactKind { V1G_COMPACT_F32_COORDS = 0, V1G_COMPACT_U8_PACKED = 1, V1G_COMPACT_LGN_RATES = 2 };
// input of kind V1G_COMPACT_LGN_RATES: spikes are drawn on the fly from firing rates
struct V1GRateSource {
  const float* rates;    // [T, n_cols] or [B, T, n_cols]
  int64_t batch_stride;  // elements between the tables of consecutive trials, 0 = one table
  unsigned key0, key1;
};
#define V1G_SEG 4096
int v1g_compact_count_scan(V1GHandle* h, int kind, const void* x, int n_rows, int64_t n_cols,
                           int time_major_T, int32_t* offsets, int64_t* n_segments_out,
                           cudaStream_t st);
int v1g_compact_fill(V1GHandle* h, int kind, const void* x, int n_rows, int64_t n_cols,
                     int time_major_T, const int32_t* offsets, void* out, int64_t cap,
                     cudaStream_t st);
