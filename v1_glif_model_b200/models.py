"""Host-side mirror of the reference's operator interface for the recurrent cell.

Same names, argument meaning and error behaviour as ``v1_model_utils/models.py`` in the
reference, with the arithmetic done by ``libv1g.so`` (hand-written sm_100a kernels behind the C
ABI of ``include/v1g.h``).  PyTorch is used only as the owner of device memory and streams.

=====================================  ==============================================
here                                   reference ``v1_model_utils/models.py``
=====================================  ==============================================
``make_pre_ind_table``                 ``:343-373`` (+ ``_validate_inputs`` ``:299-315``)
``V1Column.__init__``                  ``:451-773``
``V1Column.zero_state`` / ``call``     ``:1044-1056`` / ``:1059-1135``
``calculate_i_rec_with_custom_grad``   ``:942-964`` -> ``calculate_synaptic_currents`` ``:103-263``
``calculate_input_current_from_spikes``  ``:814-863``
``calculate_noise_current``            ``:865-940``
``update_psc`` / ``_dense_update_impl``  ``:979-982`` / ``:985-1028``
``rollout`` / ``rollout_host``         Keras ``RNN(cell)`` loop ``:1317-1322``
``backward``                           ``tape.gradient`` in ``multi_training.py:493``
=====================================  ==============================================

There is no CPU path: without a CUDA device or without the built library every entry raises.
"""
from __future__ import annotations

import ctypes as C
import zlib

import numpy as np
import torch

from . import _lib


def make_pre_ind_table(indices, n_source_neurons=197613):
    """CSR table by presynaptic index: ``(order, row_splits)`` as int64 NumPy arrays.

    The reference wraps the same two arrays in a ``tf.RaggedTensor`` (``models.py:343-373``).
    Raises ``ValueError`` on a non-positive source count, a malformed index array or an
    out-of-range presynaptic index, like ``_validate_inputs`` (``models.py:299-315``).
    Runs on the host inside the library; no GPU is needed.
    """
    n_source_neurons = int(n_source_neurons)
    if n_source_neurons <= 0:
        raise ValueError(f'`n_source_neurons` must be > 0, got {n_source_neurons}.')
    idx = np.asarray(indices)
    if idx.ndim != 2 or idx.shape[1] < 2:
        raise ValueError(f'`indices` must have shape [n_synapses, >=2], got {idx.shape}.')
    idx = np.ascontiguousarray(idx[:, :2], dtype=np.int64)
    pre = idx[:, 1]
    invalid = (pre < 0) | (pre >= n_source_neurons)
    if np.any(invalid):
        bad = int(pre[np.flatnonzero(invalid)[0]])
        raise ValueError(
            f'Presynaptic index {bad} is out of bounds for `n_source_neurons={n_source_neurons}`.')
    order = np.empty((idx.shape[0],), dtype=np.int64)
    row_splits = np.empty((n_source_neurons + 1,), dtype=np.int64)
    rc = _lib.load().v1g_build_pre_ind_table(
        idx.shape[0], idx.ctypes.data, n_source_neurons, order.ctypes.data, row_splits.ctypes.data)
    if rc != _lib.OK:
        raise ValueError(f"v1g_build_pre_ind_table failed with status {rc}")
    return order, row_splits


def _ptr(t):
    if t is None:
        return None
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class V1Column:
    """The V1 GLIF3 recurrent cell on one B200; constructor arguments as the reference's."""

    def __init__(self, network, lgn_input, bkg_input, dt=1.0, gauss_std=0.5,
                 dampening_factor=0.3, recurrent_dampening_factor=0.5,
                 voltage_gradient_dampening=0.5, input_weight_scale=1.0,
                 recurrent_weight_scale=1.0, lr_scale=1.0, spike_gradient=False, max_delay=0,
                 batch_size=1, bkg_firing_rate=250, pseudo_gauss=False, train_recurrent=True,
                 train_recurrent_per_type=True, train_input=False, train_noise=True,
                 noise_seed=0, hard_reset=False, current_input=False, pseudo_width=1.0,
                 device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("V1Column needs a CUDA device (sm_100a); there is no CPU fallback.")
        if current_input:
            raise NotImplementedError("current_input=True (firing-probability input) is outside "
                                      "the accelerated path")
        self._libh = None
        self._lib = _lib.load()
        self.device = torch.device(device if device is not None else
                                   f"cuda:{torch.cuda.current_device()}")
        torch.cuda.set_device(self.device)
        self._dt = float(dt)
        self._n_neurons = n = int(network["n_nodes"])
        self._lr_scale = float(lr_scale)
        self._hard_reset = bool(hard_reset)
        self._pseudo_gauss = bool(pseudo_gauss)
        self.bkg_firing_rate = float(bkg_firing_rate)
        self.noise_seed = int(noise_seed)

        # ---- per-neuron constants (models.py:482-526, 574-611), fp32 like the TF graph ----
        p = {k: np.asarray(v, dtype=np.float64) for k, v in network["node_params"].items()}
        type_ids = np.asarray(network["node_type_ids"]).astype(np.int64)
        voltage_scale = p["V_th"] - p["E_L"]
        self.voltage_scale = voltage_scale[type_ids]
        asc_amps = (p["asc_amps"] / voltage_scale[..., None])[type_ids]
        membrane_decay = np.exp(-dt / (p["C_m"] / p["g"]))
        current_factor = ((1 - membrane_decay) / p["g"])[type_ids]
        membrane_decay = membrane_decay[type_ids]
        tau_syn = np.asarray(network["tau_syn"], dtype=np.float64)
        self._n_syn_basis = r = int(tau_syn.size)
        syn_decay = np.exp(-dt / tau_syn).astype(np.float32)
        psc_initial = (np.e / tau_syn).astype(np.float32)
        t_ref_steps = np.maximum(np.ceil(p["t_ref"][type_ids] / dt).astype(np.int16), 1)
        # k goes through inverse-sigmoid and sigmoid in fp32 before exp (models.py:556-593)
        k32 = torch.from_numpy(p["k"]).to(torch.float32)[torch.from_numpy(type_ids)]
        k32 = torch.sigmoid(torch.log(k32 / (1 - k32)))
        asc_decay = torch.exp(-torch.tensor(dt, dtype=torch.float32) * k32).numpy()
        basis = np.ascontiguousarray(np.asarray(network["synaptic_basis_weights"], dtype=np.float32))
        if basis.ndim != 2 or basis.shape[1] != r:
            raise ValueError(f"synaptic_basis_weights must be [S, {r}], got {basis.shape}")

        # ---- delays (models.py:529-539, 633-636) ----
        rec_delays = np.asarray(network["synapses"]["delays"])
        all_delays = [rec_delays] + [np.asarray(d["delays"]) for d in (lgn_input, bkg_input)
                                     if "delays" in d]
        data_max_delay = int(np.ceil(np.max(np.concatenate(all_delays)) / dt))
        self.max_delay = min(data_max_delay, max_delay) if max_delay > 0 else data_max_delay

        self.input_dim = int(lgn_input["n_inputs"])
        self.n_bkg = int(bkg_input["n_inputs"])
        cfg = _lib.V1GConfig(
            n_neurons=n, n_receptors=r, n_syn_types=basis.shape[0], max_delay=self.max_delay,
            n_lgn=self.input_dim, n_bkg=self.n_bkg,
            flags=(_lib.FLAG_HARD_RESET if hard_reset else 0) |
                  (_lib.FLAG_PSEUDO_GAUSS if pseudo_gauss else 0),
            dt=dt, dampening_factor=dampening_factor,
            recurrent_dampening=recurrent_dampening_factor,
            voltage_gradient_dampening=voltage_gradient_dampening, gauss_std=gauss_std,
            pseudo_width=pseudo_width, lr_scale=lr_scale, bkg_firing_rate=bkg_firing_rate)
        hp = C.c_void_p()
        rc = self._lib.v1g_create(C.byref(cfg), C.byref(hp))
        if rc != _lib.OK:
            _lib.check(None, rc)
        self._libh = hp

        f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
        tref32 = np.ascontiguousarray(t_ref_steps, dtype=np.int32)
        arrs = [f32(membrane_decay), f32(current_factor), f32(asc_decay), f32(asc_amps), tref32,
                syn_decay, psc_initial, basis]
        self._check(self._lib.v1g_set_neuron_params(self._libh, *[a.ctypes.data for a in arrs]))
        self.t_ref_steps = tref32
        self.synaptic_basis_weights = basis

        # ---- connectivity (models.py:625-640, 707-773) ----
        def _source(src, indices, weights, syn_ids, n_cols, scale):
            indices = np.ascontiguousarray(indices, dtype=np.int64)
            syn_ids = np.ascontiguousarray(syn_ids, dtype=np.uint8)
            w = np.asarray(weights, dtype=np.float64) / voltage_scale[type_ids[indices[:, 0]]]
            self._check(self._lib.v1g_set_connectivity(
                self._libh, src, indices.shape[0], indices.ctypes.data, syn_ids.ctypes.data, n_cols))
            positive = torch.from_numpy(w >= 0).to(self.device)
            values = torch.from_numpy((w * scale / lr_scale).astype(np.float32)).to(self.device)
            return indices, values, positive

        rec_idx = np.array(network["synapses"]["indices"], dtype=np.int64)
        delays = np.round(np.clip(rec_delays, dt, self.max_delay) / dt).astype(np.int32)
        rec_idx[:, 1] = rec_idx[:, 1] + n * (delays - 1)
        self.recurrent_dense_shape = (n, self.max_delay * n)
        self.recurrent_indices, self.recurrent_weight_values, self.recurrent_weight_positive = \
            _source(_lib.SRC_REC, rec_idx, network["synapses"]["weights"],
                    network["synapses"]["syn_ids"], self.recurrent_dense_shape[1],
                    recurrent_weight_scale)
        self.lgn_input_dense_shape = (n, self.input_dim)
        self.input_indices, self.input_weight_values, self.input_weight_positive = \
            _source(_lib.SRC_LGN, lgn_input["indices"], lgn_input["weights"], lgn_input["syn_ids"],
                    self.input_dim, input_weight_scale)
        self.bkg_input_dense_shape = (n, self.n_bkg)
        self.bkg_input_indices, self.bkg_input_weights, self.bkg_input_weight_positive = \
            _source(_lib.SRC_BKG, bkg_input["indices"], bkg_input["weights"], bkg_input["syn_ids"],
                    self.n_bkg, input_weight_scale)
        self.refresh_weights()
        # keys of the device-side background sampler: noise_seed + replica_id * 1000003
        # (models.py:869-877); one process drives one GPU here, so the replica is the process rank
        replica = 0
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            replica = torch.distributed.get_rank()
        self.set_noise_seed(self.noise_seed, replica)

    # ---- plumbing ----------------------------------------------------------------------
    def _check(self, rc):
        _lib.check(self._libh, rc)

    def __del__(self):
        if getattr(self, "_libh", None):
            self._lib.v1g_destroy(self._libh)
            self._libh = None

    def set_noise_seed(self, noise_seed, replica_id=None):
        """Seed of the background sampler (``models.py:506``; the reference's training loop advances
        it once per rollout, ``tf_utils.py:235-237``) and, optionally, the replica id that offsets it."""
        self.noise_seed = int(noise_seed)
        if replica_id is not None:
            self.replica_id = int(replica_id)
        self._check(self._lib.v1g_set_noise_seed(self._libh, self.noise_seed, self.replica_id))

    def set_option(self, name, value):
        self._check(self._lib.v1g_set_option(self._libh, name.encode(), int(value)))

    def synchronize(self):
        self._check(self._lib.v1g_synchronize(self._libh, _stream()))

    def counters(self):
        c = _lib.V1GCounters()
        self._check(self._lib.v1g_get_counters(self._libh, C.byref(c)))
        return {n: int(getattr(c, n)) for n, _ in c._fields_}

    def last_kernel_ms(self, which):
        """Device milliseconds of the last forward (0) or backward (1) rollout kernel alone."""
        ms = C.c_float(0.0)
        self._check(self._lib.v1g_last_kernel_ms(self._libh, which, C.byref(ms)))
        return ms.value

    def balance_slices(self, cost=None):
        """Re-cut the thread blocks' slices of the forward rollout so that every slice carries about the
        same scatter work (``v1g_balance_slices``): ``cost`` = per-neuron weights (NumPy ``[n_neurons]``),
        or ``None`` to use the spike counts of the last rollout saved for the backward pass."""
        ptr = None
        if cost is not None:
            cost = np.ascontiguousarray(cost, dtype=np.float32)
            assert cost.shape == (self._n_neurons,)
            ptr = cost.ctypes.data
        self._check(self._lib.v1g_balance_slices(self._libh, ptr, _stream()))

    def phase_times(self):
        """Per-block (dense, scatter, barrier, total) nanoseconds of the last rollout kernel
        (needs ``set_option('phase_timers', 1)``)."""
        buf = np.zeros((1024, 4), dtype=np.uint64)
        n = C.c_int32(0)
        self._check(self._lib.v1g_get_phase_times(self._libh, buf.ctypes.data, 1024, C.byref(n)))
        return buf[:n.value]

    def pre_ind_table(self, source=_lib.SRC_REC):
        """``(order, row_splits)`` of a source as built inside the library."""
        nnz = {0: self.recurrent_indices, 1: self.input_indices, 2: self.bkg_input_indices}[source].shape[0]
        ncols = {0: self.recurrent_dense_shape[1], 1: self.input_dim, 2: self.n_bkg}[source]
        order = np.empty((nnz,), np.int64)
        splits = np.empty((ncols + 1,), np.int64)
        self._check(self._lib.v1g_get_pre_ind_table(self._libh, source, order.ctypes.data,
                                                    splits.ctypes.data))
        return order, splits

    def refresh_weights(self):
        """Push the three weight variables to the kernels' layouts.

        Stands in for ``refresh_recurrent_weight_shadow`` (``models.py:966-976``); call it after
        changing a weight tensor in place.
        """
        for src, w in ((_lib.SRC_REC, self.recurrent_weight_values),
                       (_lib.SRC_LGN, self.input_weight_values),
                       (_lib.SRC_BKG, self.bkg_input_weights)):
            self._check(self._lib.v1g_set_weights(self._libh, src, _ptr(w), _stream()))

    refresh_recurrent_weight_shadow = refresh_weights

    def pull_weights(self):
        """Copy the weights the kernels currently use back into the three weight tensors (needed
        after updates made in the library's internal order, see ``training.Trainer``)."""
        for src, w in ((_lib.SRC_REC, self.recurrent_weight_values),
                       (_lib.SRC_LGN, self.input_weight_values),
                       (_lib.SRC_BKG, self.bkg_input_weights)):
            self._check(self._lib.v1g_get_weights(self._libh, src, _ptr(w), _stream()))

    def train_layout(self):
        sizes = (C.c_int64 * 3)()
        self._check(self._lib.v1g_train_layout(self._libh, sizes))
        return [int(v) for v in sizes]

    def _loss_spec(self, loss):
        """``V1GLossSpec`` from a dict with any of ``rate_target`` (tensor [N], spikes/step),
        ``v_lo`` (tensor [N]), ``rate_cost``, ``voltage_cost``, ``sync_cost``, ``fano_target``,
        ``sync_bin``, ``loss_scale``, ``voltage_mode`` ("range" or "threshold") and, for the reference's rate-distribution target
        (``loss_functions.py:782-889``), ``rate_groups`` = list of ``(neuron_ids, sorted_targets)``
        with ``rate_kappa``, ``rate_pre_delay``, ``rate_post_delay``; and, for the reference's
        synchrony target (``loss_functions.py:983-1044``), ``sync_samples`` = list of
        ``(trial, neuron_ids)`` with ``sync_bin_sizes`` (steps), ``sync_bin_targets`` (measured Fano
        factors), ``sync_t_start``, ``sync_t_end``; and, for its population OSI/DSI target
        (``loss_functions.py:1340-1440``), ``osi_cost``, ``osi_angle`` [B] (degrees),
        ``osi_tuning_angle`` [N], ``osi_type_ids`` [N], ``osi_targets`` / ``dsi_targets`` /
        ``osi_type_counts`` [types], optional ``osi_normalizer`` [N], ``osi_pre_delay``,
        ``osi_post_delay``."""
        loss = dict(loss or {})
        spec = _lib.V1GLossSpec(
            rate_target=loss["rate_target"].data_ptr() if loss.get("rate_target") is not None else None,
            v_lo=loss["v_lo"].data_ptr() if loss.get("v_lo") is not None else None,
            rate_cost=loss.get("rate_cost", 0.0), voltage_cost=loss.get("voltage_cost", 0.0),
            sync_cost=loss.get("sync_cost", 0.0), fano_target=loss.get("fano_target", 1.0),
            sync_bin=int(loss.get("sync_bin", 50)), loss_scale=loss.get("loss_scale", 1.0))
        spec.voltage_mode = 1 if loss.get("voltage_mode") == "threshold" else 0
        groups = loss.get("rate_groups")
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.device)
        if groups:
            # constant over a training run, so the device copy is cached; the key is the CONTENT
            # (an object's id can be reused by a new list once the old one is freed)
            sizes = [len(g[0]) for g in groups]
            offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
            ids = np.concatenate([np.asarray(g[0], dtype=np.int32) for g in groups])
            tgt = np.concatenate([np.asarray(g[1], dtype=np.float32) for g in groups])
            key = (tuple(sizes), zlib.crc32(ids.tobytes()), zlib.crc32(tgt.tobytes()))
            if getattr(self, "_rate_groups_key", None) != key:
                self._rate_groups_dev = (dev(offs), dev(ids), dev(tgt), len(sizes), int(offs[-1]))
                self._rate_groups_key = key
            offs, ids, tgt, ng, nn = self._rate_groups_dev
            spec.n_rate_groups, spec.n_rate_neurons = ng, nn
            spec.rate_group_offsets = offs.data_ptr()
            spec.rate_group_neurons = ids.data_ptr()
            spec.rate_group_targets = tgt.data_ptr()
            spec.rate_kappa = float(loss.get("rate_kappa", 0.002))
            spec.rate_pre_delay = int(loss.get("rate_pre_delay", 0) or 0)
            spec.rate_post_delay = int(loss.get("rate_post_delay", 0) or 0)
        samples = loss.get("sync_samples")
        if samples:
            # the reference redraws the samples in every call (loss_functions.py:997-1024), so they are
            # uploaded on every call (a few KB); the tensors are kept alive until the next call
            sizes = [len(smp[1]) for smp in samples]
            offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
            trial = np.asarray([smp[0] for smp in samples], dtype=np.int32)
            ids = np.concatenate([np.asarray(smp[1], dtype=np.int32) for smp in samples])
            self._sync_samples_dev = (dev(trial), dev(offs), dev(ids), len(sizes), int(offs[-1]))
            trial, offs, ids, ns, nm = self._sync_samples_dev
            self._sync_bins_host = (np.ascontiguousarray(loss["sync_bin_sizes"], dtype=np.int32),
                                    np.ascontiguousarray(loss["sync_bin_targets"], dtype=np.float32))
            spec.n_sync_samples, spec.n_sync_members = ns, nm
            spec.sync_sample_trial = trial.data_ptr()
            spec.sync_sample_offsets = offs.data_ptr()
            spec.sync_sample_neurons = ids.data_ptr()
            spec.n_sync_bins = len(self._sync_bins_host[0])
            spec.sync_bin_sizes = self._sync_bins_host[0].ctypes.data
            spec.sync_bin_targets = self._sync_bins_host[1].ctypes.data
            spec.sync_t_start = int(loss.get("sync_t_start", 0) or 0)
            spec.sync_t_end = int(loss.get("sync_t_end", 0) or 0)
        if loss.get("osi_cost"):
            dev_f = lambda a: torch.as_tensor(np.asarray(a, dtype=np.float32)).to(self.device)
            tuning_h = np.ascontiguousarray(loss["osi_tuning_angle"], dtype=np.float32)
            types_h = np.ascontiguousarray(loss["osi_type_ids"], dtype=np.int32)
            norm_h = (np.ascontiguousarray(loss["osi_normalizer"], dtype=np.float32)
                      if loss.get("osi_normalizer") is not None else None)
            key = (zlib.crc32(tuning_h.tobytes()), zlib.crc32(types_h.tobytes()),
                   zlib.crc32(norm_h.tobytes()) if norm_h is not None else None)
            if getattr(self, "_osi_key", None) != key:
                self._osi_dev = (dev(tuning_h), dev(types_h), dev(norm_h) if norm_h is not None else None)
                self._osi_key = key
            tuning, types, norm = self._osi_dev
            self._osi_angle_dev = dev_f(loss["osi_angle"])
            self._osi_host = tuple(np.ascontiguousarray(loss[k], dtype=np.float32)
                                   for k in ("osi_targets", "dsi_targets", "osi_type_counts"))
            spec.osi_cost = float(loss["osi_cost"])
            spec.n_osi_types = len(self._osi_host[0])
            spec.osi_angle = self._osi_angle_dev.data_ptr()
            spec.osi_tuning_angle = tuning.data_ptr()
            spec.osi_type_ids = types.data_ptr()
            spec.osi_normalizer = norm.data_ptr() if norm is not None else None
            spec.osi_targets, spec.dsi_targets, spec.osi_type_counts = (a.ctypes.data for a in self._osi_host)
            spec.osi_pre_delay = int(loss.get("osi_pre_delay", 0) or 0)
            spec.osi_post_delay = int(loss.get("osi_post_delay", 0) or 0)
        return spec

    def backward_internal(self, loss, grads_flat, losses=None):
        """BPTT with the gradients accumulated into ``grads_flat`` ([rec | lgn | bkg]) in the
        library's internal synapse order."""
        spec = self._loss_spec(loss)
        if losses is None:
            losses = torch.zeros((4,), dtype=torch.float32, device=self.device)
        self._check(self._lib.v1g_rollout_bwd_internal(self._libh, C.byref(spec), None, None,
                                                       _ptr(grads_flat), _ptr(losses), _stream()))
        return losses

    def _state_struct(self, state):
        z_buf, v, r, asc, psc_rise, psc = state[:6]
        for t in (z_buf, v, r, asc, psc_rise, psc):
            assert t.is_cuda and t.is_contiguous()
        assert r.dtype == torch.int8
        noise_step = None
        if len(state) > 6 and isinstance(state[6], torch.Tensor) and state[6].is_cuda:
            assert state[6].dtype == torch.int32 and state[6].is_contiguous()
            noise_step = state[6].data_ptr()
        return _lib.V1GState(z_buf.data_ptr(), v.data_ptr(), r.data_ptr(), asc.data_ptr(),
                             psc_rise.data_ptr(), psc.data_ptr(), noise_step)

    # ---- reference operator interface ---------------------------------------------------
    @property
    def state_size(self):
        n, r = self._n_neurons, self._n_syn_basis
        return (n * self.max_delay, n, n, n * 2, n * r, n * r, ())

    def zero_state(self, batch_size, dtype=torch.float32):
        n, r, d = self._n_neurons, self._n_syn_basis, self.max_delay
        z = lambda *s: torch.zeros(s, dtype=torch.float32, device=self.device)
        return (z(batch_size, n * d), z(batch_size, n),
                torch.zeros((batch_size, n), dtype=torch.int8, device=self.device),
                z(batch_size, n * 2), z(batch_size, n * r), z(batch_size, n * r),
                torch.zeros((batch_size,), dtype=torch.int32, device=self.device))

    def compact_spikes(self, x):
        """``tf.where(x > 0)`` -> int64 ``[n, 2]`` coordinates, row-major order."""
        x = x.to(torch.float32).contiguous()
        rows, cols = x.shape
        coords = torch.empty((rows * cols, 2), dtype=torch.int64, device=self.device)
        count = torch.zeros((1,), dtype=torch.int32, device=self.device)
        self._check(self._lib.v1g_compact_spikes(self._libh, _ptr(x), rows, cols, _ptr(coords),
                                                 rows * cols, _ptr(count), _stream()))
        return coords[:int(count.item())]

    def _syn_currents(self, source, x):
        x = x.to(torch.float32).contiguous()
        b = x.shape[0]
        out = torch.empty((b * self._n_neurons, self._n_syn_basis), dtype=torch.float32,
                          device=self.device)
        self._check(self._lib.v1g_syn_currents_fwd(self._libh, source, _ptr(x), b, _ptr(out),
                                                   _stream()))
        return out

    def syn_currents_grad(self, source, x, dy, want_dx=True, want_dw=True):
        """Gradient of a current computation: ``(d_x or None, d_w or None)`` (``models.py:174-261``)."""
        x = x.to(torch.float32).contiguous()
        dy = dy.contiguous()
        b = x.shape[0]
        nnz = {0: self.recurrent_weight_values, 1: self.input_weight_values,
               2: self.bkg_input_weights}[source].numel()
        d_x = torch.empty_like(x) if want_dx else None
        d_w = torch.empty((nnz,), dtype=torch.float32, device=self.device) if want_dw else None
        self._check(self._lib.v1g_syn_currents_bwd(self._libh, source, _ptr(x), _ptr(dy), b,
                                                   _ptr(d_x), _ptr(d_w), _stream()))
        return d_x, d_w

    def calculate_i_rec_with_custom_grad(self, rec_z_buf):
        return self._syn_currents(_lib.SRC_REC, rec_z_buf)

    def calculate_input_current_from_spikes(self, x_t):
        return self._syn_currents(_lib.SRC_LGN, x_t)

    def sample_bkg_counts(self, batch_size, n_steps=None, first_step=0):
        """Poisson counts of the background nodes at ``bkg_firing_rate * dt / 1000`` per step, drawn by
        the library's Philox sampler from ``(noise_seed + replica_id * 1000003, step)``, the key the
        reference gives ``tf.random.stateless_poisson`` (``models.py:867-887``).  TensorFlow's random
        stream itself is not reproduced, so runs that must match another implementation pass the
        counts in explicitly.  ``[B, n_bkg]`` for ``n_steps=None``, else ``[B, n_steps, n_bkg]``."""
        t_len = 1 if n_steps is None else int(n_steps)
        out = torch.empty((batch_size, t_len, self.n_bkg), dtype=torch.int32, device=self.device)
        self._check(self._lib.v1g_sample_bkg_counts(self._libh, batch_size, t_len, int(first_step),
                                                    _ptr(out), _stream()))
        return out[:, 0] if n_steps is None else out

    def sample_lgn_spikes(self, rates, batch_size, seed):
        """LGN spikes ``uniform < 1 - exp(-rates / 1000)`` (``stim_dataset.py:182-193``) as uint8
        ``[B, T, n_lgn]`` from ``rates[T, n_lgn]`` (one table for all trials) or ``[B, T, n_lgn]``."""
        rates = rates.to(torch.float32).contiguous()
        stride = 0 if rates.dim() == 2 else rates.shape[1] * rates.shape[2]
        t_len = rates.shape[-2]
        out = torch.empty((batch_size, t_len, self.input_dim), dtype=torch.uint8, device=self.device)
        self._check(self._lib.v1g_sample_lgn_spikes(self._libh, batch_size, t_len, _ptr(rates), stride,
                                                    int(seed), _ptr(out), _stream()))
        return out

    def calculate_noise_current(self, batch_size, noise_step=None, counts=None):
        if counts is None:
            step = int(noise_step[0]) if noise_step is not None else 0
            counts = self.sample_bkg_counts(batch_size, first_step=step)
        return self._syn_currents(_lib.SRC_BKG, counts)

    def _dense_update_impl(self, batch_size, prev_z, v, r, asc, psc_rise, psc, rec_inputs):
        """``(new_v, new_r, new_asc, new_psc_rise, new_psc)`` (``models.py:985-1028``)."""
        n, d = self._n_neurons, self.max_delay
        z_buf = torch.zeros((batch_size, n * d), dtype=torch.float32, device=self.device)
        z_buf[:, :n] = prev_z
        state = (z_buf, v.contiguous(), r.contiguous(), asc.contiguous(), psc_rise.contiguous(),
                 psc.contiguous())
        new_state, _ = self._step(batch_size, state, rec_inputs)
        return new_state[1], new_state[2], new_state[3], new_state[4], new_state[5]

    def update_psc(self, psc, psc_rise, rec_inputs):
        """``(new_psc, new_psc_rise)`` (``models.py:979-982``)."""
        b = psc.shape[0]
        zs = self.zero_state(b)
        state = (zs[0], zs[1], zs[2], zs[3], psc_rise.contiguous(), psc.contiguous())
        new_state, _ = self._step(b, state, rec_inputs)
        return new_state[5], new_state[4]

    def _step(self, batch_size, state, rec_inputs):
        out = tuple(torch.empty_like(t) for t in state[:6])
        z = torch.empty((batch_size, self._n_neurons), dtype=torch.float32, device=self.device)
        s_in, s_out = self._state_struct(state), self._state_struct(out)
        rec_inputs = rec_inputs.contiguous()
        self._check(self._lib.v1g_step_fwd(self._libh, batch_size, C.byref(s_in), _ptr(rec_inputs),
                                           C.byref(s_out), _ptr(z), _stream()))
        return out, z

    def call(self, inputs, state, constants=None, bkg_counts=None):
        """One timestep: ``((z, v), new_state)`` (``models.py:1059-1135``), operator by operator."""
        batch_size = inputs.shape[0]
        z_buf, v, r, asc, psc_rise, psc, noise_step = state
        lgn_input = inputs[:, :self.input_dim]
        i_rec = self.calculate_i_rec_with_custom_grad(z_buf)
        external_current = self.calculate_input_current_from_spikes(lgn_input)
        i_noise = self.calculate_noise_current(batch_size, noise_step, counts=bkg_counts)
        rec_inputs = (i_rec + external_current + i_noise).reshape(
            batch_size, self._n_neurons * self._n_syn_basis) * self._lr_scale
        new_state, new_z = self._step(batch_size, state, rec_inputs)
        self.last_rec_inputs = rec_inputs
        return (new_z, new_state[1]), new_state + (noise_step + 1,)

    # ---- fused rollout -------------------------------------------------------------------
    def rollout(self, x, bkg_counts=None, state=None, return_z=True, return_v=True,
                save_for_bwd=False):
        """``T`` steps in one persistent kernel.

        ``x[B,T,n_lgn]`` uint8/bool LGN spikes, ``bkg_counts[B,T,n_bkg]`` int32; without counts they
        are drawn inside the library for the steps ``state[6][0]`` .. (``noise_step``; 0 without a
        state).  ``state`` (a ``zero_state``-shaped tuple) is updated IN PLACE when given.
        Returns ``(z uint8 [B,T,N] or None, v float32 [B,T,N] or None)``.
        """
        b, t_len = x.shape[0], x.shape[1]
        x = x.to(torch.uint8).contiguous()
        if bkg_counts is not None:
            bkg_counts = bkg_counts.to(torch.int32).contiguous()
        n = self._n_neurons
        z = torch.empty((b, t_len, n), dtype=torch.uint8, device=self.device) if return_z else None
        v = torch.empty((b, t_len, n), dtype=torch.float32, device=self.device) if return_v else None
        if b > _lib.MAX_BATCH:
            return self._rollout_wide(x, bkg_counts, state, z, v, save_for_bwd)
        st = C.byref(self._state_struct(state)) if state is not None else None
        self._saved = (x, bkg_counts) if save_for_bwd else None
        self._check(self._lib.v1g_rollout_fwd(self._libh, b, t_len, _ptr(x), _ptr(bkg_counts), st,
                                              _ptr(z), _ptr(v), int(save_for_bwd), _stream()))
        return z, v

    def _rollout_wide(self, x, bkg_counts, state, z, v, save_for_bwd):
        """Forward rollout of more trials than one kernel launch takes (``V1G_MAX_BATCH``; the reference
        evaluates 10 trials per angle, ``osi_dsi_estimator.py:424``): trials are independent, so the
        batch runs as consecutive groups of at most 8, each on its rows of the inputs, outputs and state.
        Counts that the library is to draw are drawn for the whole batch first, so that row ``i`` gets the
        noise of batch row ``i`` and not that of its position inside a group."""
        if save_for_bwd:
            raise ValueError(f"a rollout saved for the backward pass holds at most {_lib.MAX_BATCH} trials per GPU")
        b, t_len = x.shape[0], x.shape[1]
        if bkg_counts is None:
            first = 0
            if state is not None and len(state) > 6 and isinstance(state[6], torch.Tensor):
                first = int(state[6][0])
            bkg_counts = self.sample_bkg_counts(b, t_len, first_step=first)
        for lo in range(0, b, _lib.MAX_BATCH):
            hi = min(b, lo + _lib.MAX_BATCH)
            sub = tuple(s[lo:hi] for s in state) if state is not None else None
            st = C.byref(self._state_struct(sub)) if sub is not None else None
            self._check(self._lib.v1g_rollout_fwd(
                self._libh, hi - lo, t_len, _ptr(x[lo:hi]), _ptr(bkg_counts[lo:hi]), st,
                _ptr(z[lo:hi]) if z is not None else None, _ptr(v[lo:hi]) if v is not None else None, 0, _stream()))
        self._saved = None
        return z, v

    def rollout_rates(self, rates, lgn_seed, batch_size, bkg_counts=None, state=None, return_z=True,
                      return_v=True, save_for_bwd=False):
        """``rollout`` with the LGN spikes drawn on the device from firing rates (``rates[T,n_lgn]``
        for all trials or ``[B,T,n_lgn]``, Hz) straight into the kernels' event list; nothing but the
        seed comes from the host."""
        rates = rates.to(torch.float32).contiguous()
        stride = 0 if rates.dim() == 2 else rates.shape[1] * rates.shape[2]
        b, t_len, n = int(batch_size), rates.shape[-2], self._n_neurons
        if bkg_counts is not None:
            bkg_counts = bkg_counts.to(torch.int32).contiguous()
        z = torch.empty((b, t_len, n), dtype=torch.uint8, device=self.device) if return_z else None
        v = torch.empty((b, t_len, n), dtype=torch.float32, device=self.device) if return_v else None
        st = C.byref(self._state_struct(state)) if state is not None else None
        self._saved = (rates, bkg_counts) if save_for_bwd else None
        self._check(self._lib.v1g_rollout_fwd_rates(self._libh, b, t_len, _ptr(rates), stride, int(lgn_seed),
                                                    _ptr(bkg_counts), st, _ptr(z), _ptr(v), int(save_for_bwd),
                                                    _stream()))
        return z, v

    def rollout_host(self, x_host, bkg_counts_host, want_z=True, want_v=False):
        """End-to-end form with HOST (NumPy) buffers; copies in, runs, copies the results out."""
        x_host = np.ascontiguousarray(x_host, dtype=np.uint8)
        bkg_counts_host = np.ascontiguousarray(bkg_counts_host, dtype=np.int32)
        b, t_len = x_host.shape[0], x_host.shape[1]
        n = self._n_neurons
        z = np.empty((b, t_len, n), dtype=np.uint8) if want_z else None
        v = np.empty((b, t_len, n), dtype=np.float32) if want_v else None
        self._check(self._lib.v1g_rollout_fwd_host(
            self._libh, b, t_len, x_host.ctypes.data, bkg_counts_host.ctypes.data,
            z.ctypes.data if want_z else None, v.ctypes.data if want_v else None, 0, _stream()))
        return z, v

    def rollout_host_pipelined(self, x_host, bkg_counts_host, z_format="uint8", chunk_steps=0):
        """Forward-only evaluation from host buffers (``osi_dsi_estimator.py:280-305``) with input
        copies, computation and result copies overlapped.  ``x_host`` / ``bkg_counts_host``: NumPy
        arrays or CPU tensors, ``[B,T,n_lgn]`` uint8 and ``[B,T,n_bkg]`` int32; pinned tensors are
        copied at full speed.  Returns a PINNED CPU tensor that the cell reuses on the next call with
        the same shape: ``[B,T,N]`` uint8, or for ``z_format="bits"`` ``[B,T,ceil(N/32)]`` int32 with
        the spike of neuron ``n`` in bit ``n % 32`` of word ``n // 32``."""
        xt = x_host if isinstance(x_host, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(x_host, dtype=np.uint8))
        ct = bkg_counts_host if isinstance(bkg_counts_host, torch.Tensor) else \
            torch.from_numpy(np.ascontiguousarray(bkg_counts_host, dtype=np.int32))
        assert xt.dtype == torch.uint8 and ct.dtype == torch.int32 and xt.is_contiguous() and ct.is_contiguous()
        b, t_len, n = xt.shape[0], xt.shape[1], self._n_neurons
        bits = z_format == "bits"
        shape = (b, t_len, (n + 31) // 32) if bits else (b, t_len, n)
        cache = self.__dict__.setdefault("_host_out", {})
        out = cache.get((bits, shape))
        if out is None:
            out = torch.empty(shape, dtype=torch.int32 if bits else torch.uint8).pin_memory()
            cache.clear()
            cache[(bits, shape)] = out
        self._check(self._lib.v1g_rollout_fwd_host_pipelined(
            self._libh, b, t_len, xt.data_ptr(), ct.data_ptr(), out.data_ptr(), 1 if bits else 0,
            int(chunk_steps), _stream()))
        return out

    def backward(self, loss=None, g_z=None, g_v=None, accumulate_into=None):
        """BPTT over the rollout saved by ``rollout(..., save_for_bwd=True)``.

        ``loss``: see ``_loss_spec``.  Returns ``(dW_rec, dW_lgn, dW_bkg, losses[4])`` in the synapse
        order of the constructor's arrays.
        """
        spec = self._loss_spec(loss)
        if accumulate_into is None:
            grads = [torch.zeros_like(w) for w in (self.recurrent_weight_values,
                                                   self.input_weight_values,
                                                   self.bkg_input_weights)]
        else:
            grads = list(accumulate_into)
        losses = torch.zeros((4,), dtype=torch.float32, device=self.device)
        self._check(self._lib.v1g_rollout_bwd(
            self._libh, C.byref(spec), _ptr(g_z.contiguous() if g_z is not None else None),
            _ptr(g_v.contiguous() if g_v is not None else None), _ptr(grads[0]), _ptr(grads[1]),
            _ptr(grads[2]), _ptr(losses), _stream()))
        return grads[0], grads[1], grads[2], losses
