/*
 * v1g.h - C ABI of the B200 (sm_100a) implementation of the per-timestep core of the V1 GLIF3
 * model: event-driven spike -> synaptic-current scatter, double-alpha PSC update, GLIF3
 * membrane / after-spike-current / refractory / threshold update, and their BPTT gradients.
 *
 * The reference (JavierGalvan9/V1_GLIF_model) has no FFI: its operator interface for this path
 * is a set of Python callables over TensorFlow tensors in v1_model_utils/models.py.  Each entry
 * point below names the callable (file:line in the reference tree) it stands in for.  Plain
 * pointers and sizes only.  Unless a parameter says "host", pointers are DEVICE pointers on the
 * GPU that was current when the handle was created.  Every call returns 0 on success or a
 * negative V1G_E* code and never aborts; v1g_last_error() gives the message.  A handle is not
 * thread-safe; use one per GPU.  `stream` is a cudaStream_t passed as void*.
 *
 * Tensor layouts at this boundary are the reference's own:
 *   z_buf[B, D*N]   block d-1 (columns (d-1)*N .. d*N) holds the spikes emitted d steps ago
 *   psc, psc_rise, rec_inputs [B, N*R]  index n*R + r      asc[B, N*2]  index n*2 + k
 *   i_flat[B*N, R]  row b*N + n
 *   weights / weight gradients of a source: dense [nnz] in the order of the `indices` rows given
 *   to v1g_set_connectivity (the reference's post-major synapse order, load_sparse.py:15-22)
 */
#ifndef V1G_H_
#define V1G_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define V1G_OK 0
#define V1G_EINVAL (-1)   /* bad argument (the reference raises ValueError, models.py:299-315) */
#define V1G_ECUDA (-2)    /* a CUDA runtime call failed */
#define V1G_ENOMEM (-3)   /* device allocation failed */
#define V1G_ETIMEOUT (-4) /* a bounded device-side wait gave up; results are invalid */
#define V1G_ESTATE (-5)   /* call order violated (e.g. backward without a saved forward) */
#define V1G_ERANGE (-6)   /* size beyond a stated maximum */

/* synaptic sources of the cell */
#define V1G_SRC_REC 0 /* recurrent, delays folded into the presynaptic column (models.py:633-640) */
#define V1G_SRC_LGN 1 /* LGN input, no delay (models.py:707-738) */
#define V1G_SRC_BKG 2 /* background Poisson nodes, no delay, scaled by count (models.py:740-773) */

#define V1G_FLAG_HARD_RESET 1   /* models.py:1020-1023 */
#define V1G_FLAG_PSEUDO_GAUSS 2 /* models.py:36-50, 1106-1107 */

#define V1G_MAX_BATCH 8
#define V1G_MAX_RECEPTORS 8
#define V1G_MAX_DELAY 8

typedef struct V1GHandle V1GHandle;

/* Scalars of V1Column.__init__ (models.py:451-476). */
typedef struct V1GConfig {
  int32_t n_neurons;   /* N */
  int32_t n_receptors; /* R = n_syn_basis (models.py:520), <= V1G_MAX_RECEPTORS */
  int32_t n_syn_types; /* S = rows of synaptic_basis_weights (models.py:620-622), <= 256 */
  int32_t max_delay;   /* D in steps (models.py:529-539), <= V1G_MAX_DELAY */
  int32_t n_lgn;
  int32_t n_bkg;
  int32_t flags;
  float dt;
  float dampening_factor;           /* amplitude of the pseudo-derivative */
  float recurrent_dampening;        /* models.py:1081 */
  float voltage_gradient_dampening; /* models.py:1010 */
  float gauss_std;
  float pseudo_width; /* support half-width of the triangular pseudo-derivative; reference = 1 */
  float lr_scale;     /* models.py:1097 */
  float bkg_firing_rate; /* Hz; Poisson rate per step = bkg_firing_rate * 0.001 (models.py:741) */
} V1GConfig;

/* Cell state, reference layouts and dtypes (models.py:1030-1056).  r is int8. */
typedef struct V1GState {
  float* z_buf;    /* [B, D*N] */
  float* v;        /* [B, N]   */
  int8_t* r;       /* [B, N]   */
  float* asc;      /* [B, N*2] */
  float* psc_rise; /* [B, N*R] */
  float* psc;      /* [B, N*R] */
  int32_t* noise_step; /* [B] step counter of the background sampler (models.py:1042, 1133), may be NULL */
} V1GState;

/* In-kernel loss specification of the training rollout.
 *   rate     : with n_rate_groups == 0 the simplified form of the benchmark configurations,
 *                rate_cost * mean_n (mean_{b,t} z[b,t,n] - target[n])^2, target in spikes/step;
 *              with n_rate_groups > 0 the reference's own firing-rate target
 *              (SpikeRateDistributionTarget.__call__, loss_functions.py:873-889, with
 *              compute_spike_rate_target_loss and huber_quantile_loss, :626-681): rates are the mean
 *              over the batch and the steps [rate_pre_delay, T - rate_post_delay); per population the
 *              sorted rates are compared rank by rank with the sorted target sample through the
 *              quantile-Huber penalty (kappa = rate_kappa, 0 -> 0.002), summed over populations,
 *              divided by the neurons covered and multiplied by rate_cost.  Neurons with equal
 *              rates keep their listed order (the reference orders them at random).
 *   voltage  : voltage_cost * mean_{b,t,n} (relu(v-1)^2 + relu(v_lo[n]-v)^2); with v_lo == NULL
 *              (lower bound 0) this is the reference's "range" penalty relu(|v-.5|-.5)^2, with
 *              voltage_mode == 1 its "threshold" penalty (v-1)^2 (VoltageRegularization,
 *              loss_functions.py:1047-1119)
 *   synchrony: with n_sync_samples == 0 the simplified form of the benchmark configuration,
 *                sync_cost * (mean_b Fano_b - fano_target)^2, Fano_b = var/mean over bins of the
 *                population spike count in bins of sync_bin steps (loss_functions.py:964-981);
 *              with n_sync_samples > 0 the reference's own target (SynchronizationLoss.__call__,
 *              loss_functions.py:983-1044): every sample is one trial and a set of neurons, its
 *              population count over [sync_t_start, sync_t_end) is binned with every bin size below
 *              half the window, Fano = biased variance / max(mean, 1e-7), averaged over samples, and
 *              the loss is sync_cost * mean_k (target_k - Fano_k)^2.  The reference draws trial,
 *              size and members of the samples at random in every call; here they are an input.
 *   OSI/DSI  : the reference's population orientation / direction selectivity target
 *              (OrientationSelectivityLoss with method "crowd_osi", loss_functions.py:1340-1440):
 *              rates per trial over [osi_pre_delay, T - osi_post_delay), optionally divided by a
 *              normaliser; per trial and cell type osi = mean(rates cos 2d) / max(mean rates, 0.0005),
 *              dsi with cos d, d = angle[b] - tuning_angle[n]; averaged over trials;
 *              osi_cost * sum_type count ((osi - target)^2 + (dsi - target)^2) / sum_type count.
 *              Its value is added to the synchrony slot of the returned losses.
 * All costs are multiplied by loss_scale (1/replicas, multi_training.py:427-429). */
typedef struct V1GLossSpec {
  const float* rate_target; /* [N] device, may be NULL when rate_cost == 0 or populations are given */
  const float* v_lo;        /* [N] device, lower voltage bound in scaled units */
  float rate_cost;
  float voltage_cost;
  float sync_cost;
  float fano_target;
  int32_t sync_bin;
  float loss_scale;
  /* populations of the rate-distribution target (all device pointers); the reference's
   * target_rates dictionary flattened: population g owns positions [offsets[g], offsets[g+1]) */
  int32_t n_rate_groups;
  int32_t n_rate_neurons;            /* = offsets[n_rate_groups] */
  const int32_t* rate_group_offsets; /* [n_rate_groups + 1] */
  const int32_t* rate_group_neurons; /* [n_rate_neurons] neuron ids ("neuron_ids") */
  const float* rate_group_targets;   /* [n_rate_neurons] "sorted_target_rates", ascending per population, spikes/step */
  float rate_kappa;
  int32_t rate_pre_delay, rate_post_delay;
  /* samples of the synchrony target in full (see above); sample s = trial sync_sample_trial[s] and the
   * neurons at positions [offsets[s], offsets[s+1]) */
  int32_t n_sync_samples;
  int32_t n_sync_members;             /* = offsets[n_sync_samples] */
  const int32_t* sync_sample_trial;   /* [n_sync_samples] device */
  const int32_t* sync_sample_offsets; /* [n_sync_samples + 1] device */
  const int32_t* sync_sample_neurons; /* [n_sync_members] device */
  int32_t n_sync_bins;
  const int32_t* sync_bin_sizes;      /* [n_sync_bins] HOST, in steps; sizes not below half the window are ignored */
  const float* sync_bin_targets;      /* [n_sync_bins] HOST, the measured Fano factor per bin size */
  int32_t sync_t_start, sync_t_end;   /* window in steps; sync_t_end <= 0: end of the rollout */
  /* population OSI/DSI target (see above), off when osi_cost == 0 or n_osi_types == 0 */
  float osi_cost;
  int32_t n_osi_types;
  const float* osi_angle;          /* [B] device, stimulus direction of each trial in degrees */
  const float* osi_tuning_angle;   /* [N] device, network['tuning_angle'] in degrees */
  const int32_t* osi_type_ids;     /* [N] device, cell type of every neuron ("node_type_ids") */
  const float* osi_normalizer;     /* [N] device or NULL, rate normaliser (floored at 0.0005) */
  const float* osi_targets;        /* [n_osi_types] HOST, measured OSI per cell type */
  const float* dsi_targets;        /* [n_osi_types] HOST */
  const float* osi_type_counts;    /* [n_osi_types] HOST, the weights "cell_type_count" */
  int32_t osi_pre_delay, osi_post_delay;
  int32_t voltage_mode; /* 0: range (above), 1: threshold, voltage_cost * mean (v - 1)^2 */
} V1GLossSpec;

/* Event counters of the last rollout (for the roofline's algorithmic bytes). */
typedef struct V1GCounters {
  unsigned long long spikes;     /* V1 spikes emitted */
  unsigned long long rec_rows;   /* active recurrent source rows walked (spike x delay buckets) */
  unsigned long long rec_events; /* recurrent synapse events delivered */
  unsigned long long lgn_rows;
  unsigned long long lgn_events;
  unsigned long long bkg_rows;
  unsigned long long bkg_events;
  unsigned long long bwd_rows;   /* rows walked by the backward spike-gradient gather */
  unsigned long long bwd_events; /* synapses visited by it */
  unsigned long long dw_events;  /* weight-gradient synapse events */
} V1GCounters;

/* ---- life cycle ------------------------------------------------------------------------ */

/* V1Column.__init__ scalars (models.py:451-541). */
int v1g_create(const V1GConfig* cfg, V1GHandle** out);
int v1g_destroy(V1GHandle* h);
const char* v1g_last_error(const V1GHandle* h);
/* Library build tag, usable without a GPU. */
const char* v1g_version(void);

/* Connectivity of one source.  indices_host[nnz,2] = (post, pre) int64 on the HOST exactly as
 * V1Column stores them (recurrent: pre already holds pre + N*(delay_steps-1), models.py:633-639),
 * syn_ids_host[nnz] on the host.  n_source_cols = D*N (REC), n_lgn, n_bkg.  Builds the
 * presynaptic CSR of make_pre_ind_table (models.py:299-373; same stable order inside a row) and
 * the post-major gather table.  Out-of-range indices -> V1G_EINVAL (models.py:308-314). */
int v1g_set_connectivity(V1GHandle* h, int source, int64_t nnz, const int64_t* indices_host,
                         const uint8_t* syn_ids_host, int64_t n_source_cols);

/* make_pre_ind_table + _validate_inputs (models.py:299-373) on the host, no GPU needed:
 * order[nnz] lists positions of indices_host[nnz,2] grouped by presynaptic column (column 1),
 * original order kept inside a group; row_splits[n_source_cols+1].  V1G_EINVAL for
 * n_source_cols <= 0 or an out-of-range presynaptic index (the reference raises ValueError). */
int v1g_build_pre_ind_table(int64_t nnz, const int64_t* indices_host, int64_t n_source_cols,
                            int64_t* order_host, int64_t* row_splits_host);

/* Read back the presynaptic table: order[nnz] (positions into the caller's synapse arrays) and
 * row_splits[n_source_cols+1], both HOST int64, numbered exactly like the RaggedTensor of
 * make_pre_ind_table (models.py:343-373). */
int v1g_get_pre_ind_table(V1GHandle* h, int source, int64_t* order_host, int64_t* row_splits_host);

/* Per-neuron constants precomputed by V1Column.__init__ (models.py:482-526, 574-611); HOST
 * pointers.  decay[N], current_factor[N], asc_decay[N*2], asc_amps[N*2], t_ref_steps[N] int32,
 * syn_decay[R], psc_initial[R], basis[S*R].  Kernels never recompute an exponential. */
int v1g_set_neuron_params(V1GHandle* h, const float* decay, const float* current_factor,
                          const float* asc_decay, const float* asc_amps,
                          const int32_t* t_ref_steps, const float* syn_decay,
                          const float* psc_initial, const float* basis);

/* Weights of a source in the caller's synapse order; device pointer.  Stands in for the
 * variable read in calculate_synaptic_currents and refresh_recurrent_weight_shadow
 * (models.py:663-682, 966-976). */
int v1g_set_weights(V1GHandle* h, int source, const float* w, void* stream);

/* ---- stochastic inputs on the device -------------------------------------------------------
 * The reference draws the background counts inside the cell with tf.random.stateless_poisson keyed
 * by [noise_seed + replica_id * 1000003, noise_step[0]] (models.py:865-887) and the LGN spikes in its
 * data pipeline as uniform < 1 - exp(-rate / 1000) (stim_dataset.py:182-193).  These entry points do
 * the same with a Philox-4x32-10 generator evaluated as a function of (seed, replica, step, trial,
 * node): equal arguments give equal draws in every call, chunking and replay.  TensorFlow's own
 * random streams are not reproduced. */

/* noise_seed of the cell (models.py:506; advanced once per rollout by the training loop,
 * tf_utils.py:235-237) and the replica id that offsets it (models.py:869-877). */
int v1g_set_noise_seed(V1GHandle* h, int64_t noise_seed, int32_t replica_id);

/* counts_out[B, T, n_bkg] int32 ~ Poisson(bkg_firing_rate * 0.001 * dt) for the steps
 * first_step .. first_step + T - 1 (the values of noise_step[0]).  Rates above 8 per step:
 * V1G_ERANGE. */
int v1g_sample_bkg_counts(V1GHandle* h, int32_t batch, int32_t n_steps, int32_t first_step,
                          int32_t* counts_out, void* stream);

/* x_out[B, T, n_lgn] uint8 = uniform < 1 - exp(-rates / 1000); rates[T, n_lgn] in Hz, one table for
 * all trials (rates_batch_stride = 0) or one per trial (stride in elements between trials). */
int v1g_sample_lgn_spikes(V1GHandle* h, int32_t batch, int32_t n_steps, const float* rates,
                          int64_t rates_batch_stride, int64_t seed, uint8_t* x_out, void* stream);

/* ---- LGN front end: movie -> firing rates (lgn_model/lgn.py:481-528, helpers :54-96) ------------
 * The stage upstream of the cell: every frame is filtered with the Gaussian of each unit's spatial
 * size class (conv2d, padding SAME, divided by the same filter applied to a frame of ones), sampled
 * bilinearly at the unit's position and at that of its non-dominant subfield (spatial_response),
 * then filtered in time per unit, scaled, offset by the spontaneous rate and rectified
 * (firing_rates_from_spatial).  The tables are the arrays the reference's LGN.__init__ prepares and
 * caches (positions already scaled and clamped to the frame, lgn.py:386-393). */
typedef struct V1GLgn V1GLgn;
typedef struct V1GLgnTables {       /* all HOST pointers */
  int32_t n_units, height, width;   /* frame [height, width]; the reference uses 120 x 240 */
  int32_t n_classes;                /* spatial size classes (self.gaussian_filters) */
  const int32_t* filter_sizes;      /* [n_classes] side k of each square filter, odd */
  const float* filters;             /* the filters back to back, row-major k x k each */
  const int32_t* unit_class;        /* [n_units] class of each unit (self.spatial_range_indices) */
  const float *x, *y;               /* [n_units] position in pixels, 0 <= x <= width-1, 0 <= y <= height-1 */
  const float *non_dominant_x, *non_dominant_y;
  int32_t len_dom, len_non_dom;     /* taps of the temporal kernels */
  const float* dom_temporal_kernels;      /* [len_dom, n_units], last tap = current frame */
  const float* non_dom_temporal_kernels;  /* [len_non_dom, n_units] */
  const float *amplitude, *non_dom_amplitude, *is_composite, *spontaneous_firing_rates; /* [n_units] */
  int32_t bmtk_compat;              /* 1: divide by the filtered frame of ones (the reference's default) */
} V1GLgnTables;

int v1g_lgn_create(const V1GLgnTables* tables, V1GLgn** out);
int v1g_lgn_destroy(V1GLgn* lgn);
const char* v1g_lgn_last_error(const V1GLgn* lgn);

/* movie[n_frames, height, width] float32 (device) -> rates_out[n_frames, n_units] in Hz (device,
 * nullable) and, if wanted, the two spatial responses spatial_out[2, n_frames, n_units] (dominant,
 * non-dominant; device, nullable) that LGN.spatial_response returns.  With movie == NULL the
 * spatial responses in spatial_out are an INPUT and only the temporal stage runs
 * (LGN.firing_rates_from_spatial).  The rates feed v1g_sample_lgn_spikes / v1g_rollout_fwd_rates. */
int v1g_lgn_firing_rates(V1GLgn* lgn, const float* movie, int32_t n_frames, float* spatial_out,
                         float* rates_out, void* stream);

/* ---- operator level (one TensorFlow-level callable each) ---------------------------------- */

/* tf.where(x > 0) (models.py:128, 826, 890): row-major coordinates of the positive entries of
 * x[n_rows, n_cols] (float32) as int64 pairs coords[cap,2]; *count gets the number found (device
 * int32).  Entries beyond cap are dropped, count still reports the true number. */
int v1g_compact_spikes(V1GHandle* h, const float* x, int32_t n_rows, int64_t n_cols,
                       int64_t* coords, int64_t cap, int32_t* count, void* stream);

/* Same result as v1g_compact_spikes, for callers that may not allocate device memory.  It has no
 * counterpart in the reference.  Who needs it: code that runs as an op inside TensorFlow or
 * PyTorch (device memory there has to come from the framework's allocator; a cudaMalloc made
 * behind its back is not accounted for and blocks all streams of the GPU while it runs) and
 * programs that work inside a memory budget fixed at start-up.  This entry point takes no handle
 * and calls no cudaMalloc, cudaFree or other allocating routine; its working counters live in a
 * fixed array inside the library (256 KiB on every GPU that loads the library, held until exit).
 * Limit: n_rows * ceil(n_cols / 4096) <= 65536, i.e. up to 268 M input elements; larger inputs are
 * refused with V1G_ERANGE and a message from v1g_last_error(NULL).
 * The first call on each device looks up the array's device address; make that call with the
 * device current and before any stream capture is begun on it.  All calls share the one array:
 * calls that can overlap on the GPU (different streams or threads) race and must be serialised by
 * the caller.  Nothing has to be cleared between calls.  x, coords and count are device pointers
 * as for v1g_compact_spikes; count may be NULL. */
int v1g_compact_spikes_noalloc(const float* x, int32_t n_rows, int64_t n_cols, int64_t* coords,
                               int64_t cap, int32_t* count, void* stream);

/* calculate_synaptic_currents forward (models.py:103-169), calculate_input_current_from_spikes
 * (models.py:814-863) and calculate_noise_current with given counts (models.py:890-940).
 * x[B, n_source_cols] float32: spikes (REC, LGN) or Poisson counts as floats (BKG).
 * i_flat[B*N, R] is overwritten. */
int v1g_syn_currents_fwd(V1GHandle* h, int source, const float* x, int32_t batch, float* i_flat,
                         void* stream);

/* Gradient of the above (models.py:174-261): dy[B*N,R] -> d_x[B, n_source_cols] (nullable;
 * dense over ALL synapses, no dampening applied) and d_w[nnz] in the caller's synapse order
 * (nullable; event-driven, overwritten). */
int v1g_syn_currents_bwd(V1GHandle* h, int source, const float* x, const float* dy, int32_t batch,
                         float* d_x, float* d_w, void* stream);

/* One dense update + spike + refractory gating + buffer shift: update_psc, _dense_update_impl,
 * spike_function and the tail of V1Column.call (models.py:979-1028, 1099-1117).
 * rec_inputs[B, N*R] already holds (i_rec + i_lgn + i_bkg) * lr_scale.  `in` and `out` must not
 * alias.  z_out[B,N] float32 0/1 (nullable). */
int v1g_step_fwd(V1GHandle* h, int32_t batch, const V1GState* in, const float* rec_inputs,
                 V1GState* out, float* z_out, void* stream);

/* Adjoint of v1g_step_fwd.  g_out holds dL/d(new state) (r ignored), g_z / g_v_out the
 * gradients of the two outputs (nullable), new_v / new_r the forward results.  Writes
 * dL/d(old state) to g_in and dL/d rec_inputs to g_rec_inputs.  Stop-gradients and
 * straight-through factors as in models.py:994, 1010-1018, 58-64. */
int v1g_step_bwd(V1GHandle* h, int32_t batch, const V1GState* g_out, const float* g_z,
                 const float* g_v_out, const float* new_v, const int8_t* new_r, V1GState* g_in,
                 float* g_rec_inputs, void* stream);

/* ---- fused rollout (the Keras RNN loop over V1Column.call, models.py:1317-1322) ----------- */

/* T steps from `state` (updated in place; NULL pointers inside mean zero state and nothing is
 * written back).  x[B,T,n_lgn] uint8 LGN spikes, bkg_counts[B,T,n_bkg] int32 Poisson counts; with
 * bkg_counts == NULL the counts are drawn on the device as v1g_sample_bkg_counts draws them, for the
 * steps state->noise_step[0] .. (0 when there is no state or no counter), and state->noise_step is
 * advanced by T (models.py:1133).
 * z_out[B,T,N] uint8 and v_out[B,T,N] float32 are optional.  save_for_bwd != 0 keeps v and the
 * spike/refractory bits of every step, and a copy of bkg_counts, inside the handle for
 * v1g_rollout_bwd; x and bkg_counts may be reused once the call has returned.
 * The call is NOT asynchronous to the host: it waits on `stream` once (cudaStreamSynchronize) to
 * learn the number of LGN events before it sizes their list, so it cannot be captured in a CUDA
 * graph, and everything queued on `stream` before it has finished when it returns. */
int v1g_rollout_fwd(V1GHandle* h, int32_t batch, int32_t n_steps, const uint8_t* x,
                    const int32_t* bkg_counts, V1GState* state, uint8_t* z_out, float* v_out,
                    int32_t save_for_bwd, void* stream);

/* v1g_rollout_fwd with the LGN spikes drawn on the device from firing rates (as
 * v1g_sample_lgn_spikes draws them with `lgn_seed`) directly into the rollout's event list, without
 * materialising x.  rates[T, n_lgn] or [B, T, n_lgn] (rates_batch_stride as above). */
int v1g_rollout_fwd_rates(V1GHandle* h, int32_t batch, int32_t n_steps, const float* rates,
                          int64_t rates_batch_stride, int64_t lgn_seed, const int32_t* bkg_counts,
                          V1GState* state, uint8_t* z_out, float* v_out, int32_t save_for_bwd,
                          void* stream);

/* Same through HOST buffers: copies x and bkg_counts to the device, runs the rollout from the
 * zero state, copies z_out (uint8, nullable) and v_out (nullable) back.  The end-to-end form a
 * forward-only evaluation (osi_dsi_estimator.py:280-305) uses. */
int v1g_rollout_fwd_host(V1GHandle* h, int32_t batch, int32_t n_steps, const uint8_t* x_host,
                         const int32_t* bkg_counts_host, uint8_t* z_out_host, float* v_out_host,
                         int32_t save_for_bwd, void* stream);

/* Forward-only evaluation through HOST buffers at full device speed: the rollout runs from the zero
 * state in chunks of chunk_steps steps (0 = automatic) with the state carried on the device, while
 * the inputs of the next chunk and the spikes of the previous one travel on two further streams.
 * z_format 0: z_out_host[B,T,N] uint8 as the reference's evaluator stores them
 * (osi_dsi_estimator.py:297-305); z_format 1: z_out_host[B,T,ceil(N/32)] uint32 with the spike of
 * neuron n in bit n % 32 of word n / 32 (an eighth of the bytes to copy).  z_out_host may be NULL.
 * The copies overlap with the computation only when the host buffers are pinned (page-locked);
 * pageable buffers work but are copied at the speed of a staged copy.  Returns after all results
 * have arrived. */
int v1g_rollout_fwd_host_pipelined(V1GHandle* h, int32_t batch, int32_t n_steps, const uint8_t* x_host,
                                   const int32_t* bkg_counts_host, void* z_out_host, int32_t z_format,
                                   int32_t chunk_steps, void* stream);

/* BPTT over the saved rollout (tape.gradient in multi_training.py:493).  The loss is the
 * in-kernel specification plus optional explicit gradients g_z[B,T,N], g_v[B,T,N] (nullable).
 * Weight gradients are ACCUMULATED into d_w_* (caller zeroes them), each in its source's synapse
 * order; any may be NULL.  The initial state of the saved rollout is a constant (no gradient is
 * returned for it), but spikes pending in its z_buf do contribute to d_w_rec.  loss_out[4] (device, nullable) = total, rate, voltage, synchrony. */
int v1g_rollout_bwd(V1GHandle* h, const V1GLossSpec* loss, const float* g_z, const float* g_v,
                    float* d_w_rec, float* d_w_lgn, float* d_w_bkg, float* loss_out, void* stream);

/* ExponentiatedAdam.update_step, dense branch (optimizers.py:353-376) followed by the
 * SignedConstraint (models.py:419-427).  positive[n] uint8 is the sign mask fixed at
 * construction; step is the 1-based iteration; grad is multiplied by grad_scale first. */
int v1g_expadam_update(float* w, const float* grad, float* m, float* v, const uint8_t* positive,
                       int64_t n, float lr, float beta1, float beta2, float eps, int64_t step,
                       float grad_scale, void* stream);

/* ---- training in the library's own synapse order ---------------------------------------------
 * The reference's training step (multi_training.py:483-520) is tape.gradient -> cross-replica sum
 * -> ExponentiatedAdam.update_step -> SignedConstraint -> refresh of the compute copy.  These
 * entry points do the same without converting gradients and weights to the caller's synapse
 * order and back every step: gradients, moments and the update live in the internal order
 * (presynaptic CSR for the recurrent and LGN sources, post-major table for the background), which
 * is identical on every replica with the same connectivity, so one flat buffer can be all-reduced
 * as it is.  v1g_get_weights converts back whenever the caller wants the weights. */

/* sizes3[s] = number of synapses of source s; the flat buffers below are [rec | lgn | bkg]. */
int v1g_train_layout(V1GHandle* h, int64_t* sizes3);

/* v1g_rollout_bwd with the three weight gradients ACCUMULATED into grads_flat in internal order. */
int v1g_rollout_bwd_internal(V1GHandle* h, const V1GLossSpec* loss, const float* g_z,
                             const float* g_v, float* grads_flat, float* loss_out, void* stream);

/* Exp-Adam + sign constraint (optimizers.py:353-376, models.py:419-427) on the sources whose bit
 * is set in train_mask (bit 0 recurrent, 1 LGN, 2 background), in place on the weights the
 * kernels read.  The sign mask is the sign of each weight at the first v1g_set_weights call. */
int v1g_expadam_update_internal(V1GHandle* h, const float* grads_flat, float* m_flat, float* v_flat,
                                int32_t train_mask, float lr, float beta1, float beta2, float eps,
                                int64_t step, float grad_scale, void* stream);

/* Weight regularisers of the reference on a weight vector w[n] whose synapses carry an integer group
 * id (the edge type): value ADDED to loss_out[0] (device, nullable), gradient ACCUMULATED into grad[n].
 * w, group_ids and grad share one synapse order, whichever it is.
 *   kind 0  MeanStiffRegularizer (loss_functions.py:171-220): strength * mean_g (mean_g(w) - target[g])^2;
 *           with denominator != NULL (penalize_relative_change, max(|initial mean|, 1e-4))
 *           strength * sqrt(mean_g ((mean_g(w) - target[g]) / denominator[g])^2).  target[n_groups].
 *   kind 1  EarthMoversDistanceRegularizer (loss_functions.py:536-601): strength * mean_g mean_i
 *           |sort(w_g)_i - y_g,i|.  target[n] = the initial weights sorted ascending inside each group,
 *           groups in ascending id order; group_offsets[n_groups + 1] = where each group starts in it.
 * All pointers are device pointers. */
int v1g_weight_regularizer(V1GHandle* h, int32_t kind, const float* w, const int32_t* group_ids, int64_t n,
                           int32_t n_groups, const float* target, const int32_t* group_offsets,
                           const float* denominator, float strength, float* loss_out, float* grad,
                           void* stream);

/* perm_out_host[i] (HOST, [nnz]) = position, in the caller's synapse arrays, of the synapse that the
 * library's internal order of a source holds at position i: what converts per-synapse tables (such as
 * the group ids above) to the order of v1g_rollout_bwd_internal's gradient buffer. */
int v1g_get_internal_order(V1GHandle* h, int source, int32_t* perm_out_host);

/* Device address of the weights the kernels read, in the library's internal order (read-only view;
 * stays valid until the connectivity of the source is set again).  What a regulariser evaluated in
 * the internal order takes as w. */
int v1g_internal_weights(V1GHandle* h, int source, const float** w_out);

/* Current weights of a source in the caller's synapse order (device pointer, [nnz]). */
int v1g_get_weights(V1GHandle* h, int source, float* w_out, void* stream);

int v1g_get_counters(V1GHandle* h, V1GCounters* out_host);

/* Waits for `stream` and returns the device-side status of the launches since the last call:
 * V1G_ETIMEOUT if a bounded grid-barrier wait inside a rollout kernel gave up (the kernel then
 * returned early and its outputs are invalid).  The reference has no counterpart; a TensorFlow
 * op reports errors by raising from session.run. */
int v1g_synchronize(V1GHandle* h, void* stream);

/* Failure-path check without a fault: launches one thread that waits, with the bounded-wait
 * helper of the rollout kernels, for a counter nothing increments.  After `polls` polls it gives
 * up, records the device status and returns normally; the next v1g_synchronize then reports
 * V1G_ETIMEOUT and clears the status, and the handle stays usable.  No counterpart in the
 * reference. */
int v1g_selftest_bounded_wait(V1GHandle* h, long long polls, void* stream);

/* Tuning knobs, mainly for tests: "rollout_chunk" (neurons per thread block in the rollout
 * kernels, multiple of 32, 0 = automatic), "state_in_global" (1 = keep the rollout state in
 * global memory even when it fits in shared memory), "force_smem_kernel" (1 = the general forward
 * kernel even where the register-resident one applies), "spin_limit" (iterations a grid-barrier
 * wait may spin before giving up), "no_meta" (1 = the rollout kernels read the plain post / sid /
 * weight arrays instead of the packed 8-byte synapse records), "no_q_pack" (1 = fp32 rows in the
 * backward ring for a batch of 5 instead of 24-bit floats), "pair_rows" (1 = two steps per 32-byte
 * row in the backward ring, halving the L2 requests of delays >= 2; measured slower, off by default), "phase_timers" (1 = per-block phase
 * times, read with v1g_get_phase_times), "l2_window", "csr_evict_first" (cache-policy
 * experiments).  No counterpart in the reference. */
int v1g_set_option(V1GHandle* h, const char* name, long long value);

/* Device time in ms of the last forward (which = 0) or backward (which = 1) rollout kernel,
 * from CUDA events recorded on the launch stream around that kernel alone; blocks until the
 * kernel has finished.  No counterpart in the reference. */
int v1g_last_kernel_ms(V1GHandle* h, int which, float* ms);

/* Slices of equal scatter work for the forward rollout.  Each thread block of the rollout kernels
 * owns a contiguous slice of neurons; with equal slices the blocks whose neurons fire most set the
 * pace of every step.  This call re-cuts the slices of the one-neuron-per-thread forward kernel so
 * that cost_host[n] (host, [n_neurons], >= 0; e.g. expected spikes x out-degree) sums to about the
 * same in every slice; with cost_host == NULL the cost is taken from the spike counts of the last
 * rollout that was saved for the backward pass.  Results do not depend on the slicing (up to the
 * summation order of the currents).  Connectivity changes and the "rollout_chunk" option reset it.
 * No counterpart in the reference. */
int v1g_balance_slices(V1GHandle* h, const float* cost_host, void* stream);

/* Number of CUDA kernels this library has launched in the process so far (all handles).  No
 * counterpart in the reference. */
long long v1g_launch_count(void);

/* With option "phase_timers" = 1 the rollout kernels record, per thread block, the nanoseconds
 * spent in their dense, scatter and barrier phases and in total; this copies up to max_blocks
 * records of 4 values to the host.  A profiling aid with no counterpart in the reference. */
int v1g_get_phase_times(V1GHandle* h, unsigned long long* out_host, int32_t max_blocks,
                        int32_t* n_blocks);

#ifdef __cplusplus
}
#endif
#endif /* V1G_H_ */
