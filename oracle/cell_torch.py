"""CPU oracle of the V1 GLIF3 recurrent cell.  TEST INFRASTRUCTURE ONLY.

This file restates, operation for operation, the per-timestep cell of the reference
(``v1_model_utils/models.py``) with PyTorch CPU tensors standing in for the TensorFlow ops the
reference calls.  Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import it; no product code path does.

PARITY PINNING: the reference ships no tests, golden vectors or fixtures for this path, and
TensorFlow, which it needs, is not installable where this was written.  The oracle is pinned
against the reference's OWN cell instead: ``tests/golden/run_reference_models.py`` imports the
unmodified ``v1_model_utils/models.py`` from the reference tree over ``tests/golden/tf_standin.py``
(a torch-backed stand-in for the TensorFlow calls the file makes), steps its ``V1Column.call`` and
back-propagates through its custom gradients; the outputs are committed as
``tests/golden/reference_*.npz`` and ``tests/test_oracle_pinning.py`` requires this oracle to
reproduce them (spikes, refractory counters and the CSR table exactly; voltages and state to
1e-12; the three weight gradients to 1e-10, all in fp64).  Not pinned: TensorFlow's own kernels
(summation order of ``unsorted_segment_sum``, the Philox Poisson sampler), which never ran.

Correspondence (reference ``v1_model_utils/models.py`` line numbers):

=============================  =====================================================
here                           reference
=============================  =====================================================
``pseudo_derivative``          ``:23-28``
``SpikeFunction``              ``:52-66`` (``spike_function``), ``:36-50`` (gauss)
``make_pre_ind_table``         ``:299-373``
``get_new_inds_table``         ``:400-417``
``SynapticCurrents``           ``:103-263`` (``calculate_synaptic_currents`` + grad)
``straight_through_dampen``    ``:284-296``
``OracleV1Column.__init__``    ``:482-773``
``...input_current_from_spikes``  ``:814-863``
``...noise_current``           ``:865-940`` (counts are an input, see below)
``update_psc``                 ``:979-982``
``_dense_update_impl``         ``:985-1028``
``zero_state`` / ``call``      ``:1044-1056`` / ``:1059-1135``
=============================  =====================================================

Third-party arithmetic that is not restated: ``tf.random.stateless_poisson`` (TensorFlow
2.15.0.post1 Philox stream, ``models.py:882-887``).  Background spike counts are therefore an
explicit input of ``call`` here and of every parity test.
"""
from __future__ import annotations

import numpy as np
import torch

# the backward pass builds COO tensors from indices that are valid by construction
torch.sparse.check_sparse_tensor_invariants.disable()


# --------------------------------------------------------------------------------------
# spike function and its surrogate gradient
# --------------------------------------------------------------------------------------
def pseudo_derivative(v_scaled, dampening_factor, width=1.0):
    """``dampening * max(1 - |v_scaled|/width, 0)``; the reference has width == 1 (``:23-28``)."""
    one = torch.ones((), dtype=v_scaled.dtype)
    zero = torch.zeros((), dtype=v_scaled.dtype)
    if width == 1.0:
        a = torch.abs(v_scaled)
    else:
        a = torch.abs(v_scaled) / torch.tensor(width, dtype=v_scaled.dtype)
    return torch.tensor(dampening_factor, dtype=v_scaled.dtype) * torch.maximum(one - a, zero)


def gauss_pseudo(v_scaled, sigma, amplitude):
    """``exp(-v^2/sigma^2) * amplitude`` (``:17-21``)."""
    s = torch.tensor(sigma, dtype=v_scaled.dtype)
    return torch.exp(-torch.square(v_scaled) / torch.square(s)) * torch.tensor(
        amplitude, dtype=v_scaled.dtype)


class SpikeFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, v_scaled, dampening_factor, width, gauss_std):
        ctx.save_for_backward(v_scaled)
        ctx.dampening_factor = dampening_factor
        ctx.width = width
        ctx.gauss_std = gauss_std
        return (v_scaled > 0).to(v_scaled.dtype)

    @staticmethod
    def backward(ctx, dy):
        (v_scaled,) = ctx.saved_tensors
        if ctx.gauss_std is not None:
            dz_dv = gauss_pseudo(v_scaled, ctx.gauss_std, ctx.dampening_factor)
        else:
            dz_dv = pseudo_derivative(v_scaled, ctx.dampening_factor, ctx.width)
        return dy * dz_dv, None, None, None


def straight_through_dampen(x, dampening):
    """Forward ``x*(1-d) + stop_gradient(x*d)``; backward scales by ``1-d`` (``:284-296``)."""
    d = torch.clamp(torch.tensor(dampening, dtype=x.dtype), 0.0, 1.0)
    one = torch.ones((), dtype=x.dtype)
    return x * (one - d) + (x * d).detach()


# --------------------------------------------------------------------------------------
# CSR-by-presynaptic table
# --------------------------------------------------------------------------------------
def _validate_inputs(indices, n_source_neurons):
    n_source_neurons = int(n_source_neurons)
    if n_source_neurons <= 0:
        raise ValueError(f'`n_source_neurons` must be > 0, got {n_source_neurons}.')
    indices_np = np.asarray(indices)
    if indices_np.ndim != 2 or indices_np.shape[1] < 2:
        raise ValueError(f'`indices` must have shape [n_synapses, >=2], got {indices_np.shape}.')
    pre_ids = indices_np[:, 1].astype(np.int64, copy=False)
    invalid = (pre_ids < 0) | (pre_ids >= n_source_neurons)
    if np.any(invalid):
        bad = int(pre_ids[np.flatnonzero(invalid)[0]])
        raise ValueError(
            f'Presynaptic index {bad} is out of bounds for `n_source_neurons={n_source_neurons}`.')
    return pre_ids, n_source_neurons


def make_pre_ind_table(indices, n_source_neurons):
    """Stable bucket sort of synapse positions by presynaptic index -> ``(order, row_splits)``.

    Same result as the reference's numba counting sort and as its NumPy fallback
    (``:317-341`` and ``:359-365``): ``order`` lists synapse-array positions grouped by
    presynaptic index, original order kept inside a group; ``row_splits`` has one row per source,
    empty rows included.
    """
    pre_ids, n_source_neurons = _validate_inputs(indices, n_source_neurons)
    if pre_ids.size == 0:
        return np.empty((0,), np.int64), np.zeros((n_source_neurons + 1,), np.int64)
    order = np.argsort(pre_ids, kind='stable').astype(np.int64)
    counts = np.bincount(pre_ids, minlength=n_source_neurons)
    row_splits = np.zeros((n_source_neurons + 1,), np.int64)
    np.cumsum(counts, out=row_splits[1:])
    return order, row_splits


class PreIndTable:
    """Ragged table with the two accessors the cell needs (gather rows, row lengths)."""

    def __init__(self, indices, n_source_neurons):
        order, row_splits = make_pre_ind_table(indices, n_source_neurons)
        self.order = torch.from_numpy(order)
        self.row_splits = torch.from_numpy(row_splits)

    def gather(self, cols):
        """``tf.gather(ragged, cols)`` -> (flat_values, row_lengths)."""
        start = self.row_splits[cols]
        length = self.row_splits[cols + 1] - start
        total = int(length.sum())
        if total == 0:
            return torch.empty((0,), dtype=torch.int64), length
        excl = torch.cumsum(length, 0) - length
        pos = torch.arange(total, dtype=torch.int64) + torch.repeat_interleave(start - excl, length)
        return self.order[pos], length


def get_new_inds_table(indices, weights, syn_ids, non_zero_cols, pre_ind_table):
    """(``:400-417``)"""
    all_synapse_inds, post_in_degree = pre_ind_table.gather(non_zero_cols)
    new_indices = indices[all_synapse_inds]
    new_weights = weights[all_synapse_inds]
    new_syn_ids = syn_ids[all_synapse_inds]
    return new_indices, new_weights, new_syn_ids, post_in_degree, all_synapse_inds


# --------------------------------------------------------------------------------------
# recurrent synaptic currents with the reference's custom gradient
# --------------------------------------------------------------------------------------
class SynapticCurrents(torch.autograd.Function):
    """``calculate_synaptic_currents`` (``:103-263``).

    forward: ``I[b,post,r] = sum over synapses whose delayed presynaptic column is active of
    w*basis[sid,r]``; backward: spike gradient as R sequential sparse products over ALL synapses
    (``:187-202``), weight gradient event-driven over the active ones (``:226-240``).
    """

    @staticmethod
    def forward(ctx, rec_z_buf, weight_values, synapse_indices, dense_shape,
                synaptic_basis_weights, syn_ids, pre_ind_table, scatter_transpose=False):
        batch_size = rec_z_buf.shape[0]
        ctx.scatter_transpose = scatter_transpose
        n_post = int(dense_shape[0])
        nz = torch.nonzero(rec_z_buf > 0)                       # row-major, like tf.where
        batch_indices = nz[:, 0]
        pre_neuron_indices = nz[:, 1]
        new_indices, new_weights, new_syn_ids, post_in_degree, all_synaptic_inds = \
            get_new_inds_table(synapse_indices, weight_values, syn_ids, pre_neuron_indices,
                               pre_ind_table)
        batch_per_conn = torch.repeat_interleave(batch_indices, post_in_degree)
        segment_ids = batch_per_conn * n_post + new_indices[:, 0]
        basis_factors = synaptic_basis_weights[new_syn_ids]
        weighted_basis = new_weights[:, None] * basis_factors
        i_rec_flat = torch.zeros((batch_size * n_post, synaptic_basis_weights.shape[1]),
                                 dtype=rec_z_buf.dtype)
        i_rec_flat.index_add_(0, segment_ids, weighted_basis)
        ctx.save_for_backward(weight_values, synapse_indices, synaptic_basis_weights, syn_ids,
                              segment_ids, new_syn_ids, all_synaptic_inds)
        ctx.dense_shape = (int(dense_shape[0]), int(dense_shape[1]))
        ctx.batch_size = batch_size
        # exposed for the indexing parity tests
        ctx.active = nz
        return i_rec_flat

    @staticmethod
    def backward(ctx, dy):
        (weight_values, synapse_indices, basis, syn_ids, segment_ids, new_syn_ids,
         all_synaptic_inds) = ctx.saved_tensors
        n_post, n_pre = ctx.dense_shape
        b = ctx.batch_size
        de_dv = torch.zeros((b, n_pre), dtype=dy.dtype)
        idx_t = torch.stack([synapse_indices[:, 1], synapse_indices[:, 0]])   # (pre_d, post)
        for r_id in range(basis.shape[1]):
            dy_r = dy[:, r_id].reshape(b, n_post)
            w_r = weight_values * basis[:, r_id][syn_ids]
            if ctx.scatter_transpose:
                # the same product written as a scatter over the synapse list (the terms of every
                # output element are the same, only their summation order differs): several times
                # faster than building a sparse tensor per channel and step, which matters for the
                # full-length parity runs at the benchmark shapes
                contrib = w_r[None, :] * dy_r[:, synapse_indices[:, 0]]
                de_dv = de_dv + torch.zeros_like(de_dv).scatter_add_(
                    1, synapse_indices[:, 1][None, :].expand(b, -1), contrib)
                continue
            # dy_r @ W_r  ==  (W_r^T @ dy_r^T)^T with W_r of shape [n_post, n_pre]
            w_t = torch.sparse_coo_tensor(idx_t, w_r, (n_pre, n_post))
            de_dv = de_dv + torch.sparse.mm(w_t, dy_r.t().contiguous()).t()
        dnew_weights = dy[segment_ids]
        basis_factors_grad = basis[new_syn_ids]
        de_dw_conn = torch.einsum('cr,cr->c', dnew_weights, basis_factors_grad)
        de_dw = torch.zeros_like(weight_values)
        de_dw.index_add_(0, all_synaptic_inds, de_dw_conn)
        return de_dv, de_dw, None, None, None, None, None, None


# --------------------------------------------------------------------------------------
# the cell
# --------------------------------------------------------------------------------------
def prepare_parameters(network, dt, dtype):
    """Per-neuron constants of ``V1Column.__init__`` (``:482-526, 574-611``)."""
    p = {k: np.asarray(v, dtype=np.float64) for k, v in network["node_params"].items()}
    node_type_ids = np.asarray(network["node_type_ids"])
    voltage_scale = p["V_th"] - p["E_L"]
    asc_amps = p["asc_amps"] / voltage_scale[..., None]
    tau = p["C_m"] / p["g"]
    membrane_decay = np.exp(-dt / tau)
    current_factor = (1 - membrane_decay) / p["g"]
    tau_syns = np.asarray(network["tau_syn"], dtype=np.float64)
    syn_decay = np.exp(-dt / tau_syns)
    psc_initial = np.e / tau_syns
    t_ref_steps = np.maximum(np.ceil(p["t_ref"][node_type_ids] / dt).astype(np.int16), 1)

    def _f(v):
        return torch.from_numpy(np.asarray(v)[node_type_ids]).to(dtype)

    # k passes through inverse-sigmoid / sigmoid in the compute dtype (``:556-593``)
    k = torch.from_numpy(p["k"]).to(dtype)[torch.from_numpy(node_type_ids)]
    k = torch.sigmoid(torch.log(k / (1 - k)))
    asc_decay = torch.exp(-torch.tensor(dt, dtype=dtype) * k)
    return dict(
        voltage_scale=voltage_scale,
        node_type_ids=node_type_ids,
        asc_amps=_f(asc_amps),
        asc_decay=asc_decay,
        decay=_f(membrane_decay),
        current_factor=_f(current_factor),
        syn_decay=torch.from_numpy(syn_decay).to(dtype),
        psc_initial=torch.from_numpy(psc_initial).to(dtype),
        t_ref_steps=torch.from_numpy(t_ref_steps.astype(np.int64)),
    )


class OracleV1Column:
    """``V1Column`` (``:450-1135``) over torch CPU tensors; constructor arguments as the reference."""

    def __init__(self, network, lgn_input, bkg_input, dt=1.0, gauss_std=0.5,
                 dampening_factor=0.3, recurrent_dampening_factor=0.5,
                 voltage_gradient_dampening=0.5, input_weight_scale=1.0,
                 recurrent_weight_scale=1.0, lr_scale=1.0, max_delay=0, pseudo_gauss=False,
                 hard_reset=False, pseudo_width=1.0, dtype=torch.float32, scatter_transpose=False):
        self.dtype = dtype
        # scatter_transpose: evaluate the transposed product of the spike gradient as one scatter
        # per channel instead of the reference's sparse_dense_matmul (same terms, faster on CPU)
        self._scatter_transpose = scatter_transpose
        self._dt = dt
        self._n_neurons = n = int(network["n_nodes"])
        self._lr_scale = lr_scale
        self._dampening_factor = dampening_factor
        self._recurrent_dampening = recurrent_dampening_factor
        self._voltage_gradient_dampening = voltage_gradient_dampening
        self._pseudo_gauss = pseudo_gauss
        self._gauss_std = gauss_std
        self._hard_reset = hard_reset
        self._pseudo_width = pseudo_width

        prm = prepare_parameters(network, dt, dtype)
        self.params = prm
        voltage_scale = prm["voltage_scale"]
        node_type_ids = prm["node_type_ids"]
        self.asc_amps = prm["asc_amps"]
        self.asc_decay = prm["asc_decay"]
        self.decay = prm["decay"]
        self.current_factor = prm["current_factor"]
        self.t_ref_steps = prm["t_ref_steps"]
        self._n_syn_basis = r = prm["syn_decay"].numel()
        self.syn_decay = prm["syn_decay"].repeat(n)[None, :]        # index n*R + r (``:521-526``)
        self.psc_initial = prm["psc_initial"].repeat(n)[None, :]

        rec_delays = np.asarray(network["synapses"]["delays"])
        all_delays = [rec_delays]
        for d_in in (lgn_input, bkg_input):
            if "delays" in d_in:
                all_delays.append(np.asarray(d_in["delays"]))
        data_max_delay = int(np.ceil(np.max(np.concatenate(all_delays)) / dt))
        self.max_delay = min(data_max_delay, max_delay) if max_delay > 0 else data_max_delay

        self.synaptic_basis_weights = torch.as_tensor(
            np.asarray(network["synaptic_basis_weights"]), dtype=dtype)

        # recurrent connectivity (``:625-640``)
        indices = np.array(network["synapses"]["indices"], dtype=np.int64)
        weights = np.asarray(network["synapses"]["weights"], dtype=np.float64)
        weights = weights / voltage_scale[node_type_ids[indices[:, 0]]]
        delays = np.round(np.clip(rec_delays, dt, self.max_delay) / dt).astype(np.int32)
        indices[:, 1] = indices[:, 1] + n * (delays - 1)
        self.recurrent_dense_shape = (n, self.max_delay * n)
        self.recurrent_indices = torch.from_numpy(indices)
        self.pre_ind_table = PreIndTable(indices, self.recurrent_dense_shape[1])
        self.recurrent_weight_positive = torch.from_numpy(weights >= 0)
        self.recurrent_weight_values = torch.from_numpy(
            weights * recurrent_weight_scale / lr_scale).to(dtype).requires_grad_(True)
        self.syn_ids = torch.from_numpy(np.asarray(network["synapses"]["syn_ids"]).astype(np.int64))

        # LGN connectivity, no delays (``:707-738``)
        self.input_dim = int(lgn_input["n_inputs"])
        in_idx = np.array(lgn_input["indices"], dtype=np.int64)
        in_w = np.asarray(lgn_input["weights"], dtype=np.float64)
        in_w = in_w / voltage_scale[node_type_ids[in_idx[:, 0]]]
        self.input_indices = torch.from_numpy(in_idx)
        self.input_weight_positive = torch.from_numpy(in_w >= 0)
        self.input_weight_values = torch.from_numpy(
            in_w * input_weight_scale / lr_scale).to(dtype).requires_grad_(True)
        self.input_syn_ids = torch.from_numpy(np.asarray(lgn_input["syn_ids"]).astype(np.int64))
        self.pre_input_ind_table = PreIndTable(in_idx, self.input_dim)

        # background connectivity (``:740-773``)
        self.n_bkg = int(bkg_input["n_inputs"])
        bk_idx = np.array(bkg_input["indices"], dtype=np.int64)
        bk_w = np.asarray(bkg_input["weights"], dtype=np.float64)
        bk_w = bk_w / voltage_scale[node_type_ids[bk_idx[:, 0]]]
        self.bkg_input_indices = torch.from_numpy(bk_idx)
        self.bkg_input_weight_positive = torch.from_numpy(bk_w >= 0)
        self.bkg_input_weights = torch.from_numpy(
            bk_w * input_weight_scale / lr_scale).to(dtype).requires_grad_(True)
        self.bkg_input_syn_ids = torch.from_numpy(np.asarray(bkg_input["syn_ids"]).astype(np.int64))
        self.pre_bkg_ind_table = PreIndTable(bk_idx, self.n_bkg)

    # ---- currents ------------------------------------------------------------------
    def calculate_i_rec_with_custom_grad(self, rec_z_buf):
        return SynapticCurrents.apply(
            rec_z_buf, self.recurrent_weight_values, self.recurrent_indices,
            self.recurrent_dense_shape, self.synaptic_basis_weights, self.syn_ids,
            self.pre_ind_table, self._scatter_transpose)

    def calculate_input_current_from_spikes(self, x_t):
        """(``:814-863``)"""
        batch_size = x_t.shape[0]
        n_post = self._n_neurons
        nz = torch.nonzero(x_t if x_t.dtype == torch.bool else x_t > 0)
        new_indices, new_weights, new_syn_ids, post_in_degree, _ = get_new_inds_table(
            self.input_indices, self.input_weight_values, self.input_syn_ids, nz[:, 1],
            self.pre_input_ind_table)
        batch_per_conn = torch.repeat_interleave(nz[:, 0], post_in_degree)
        segment_ids = batch_per_conn * n_post + new_indices[:, 0]
        basis_factors = self.synaptic_basis_weights[new_syn_ids]
        new_weights_final = new_weights[:, None] * basis_factors
        out = torch.zeros((batch_size * n_post, self._n_syn_basis), dtype=self.dtype)
        return out.index_add(0, segment_ids, new_weights_final)

    def calculate_noise_current(self, batch_size, rest_of_brain):
        """(``:865-940``) with the Poisson counts ``rest_of_brain[B, n_bkg]`` given."""
        n_post = self._n_neurons
        nz = torch.nonzero(rest_of_brain > 0)
        new_indices, new_weights, new_syn_ids, post_in_degree, _ = get_new_inds_table(
            self.bkg_input_indices, self.bkg_input_weights, self.bkg_input_syn_ids, nz[:, 1],
            self.pre_bkg_ind_table)
        batch_per_conn = torch.repeat_interleave(nz[:, 0], post_in_degree)
        segment_ids = batch_per_conn * n_post + new_indices[:, 0]
        n_pre_spikes = rest_of_brain[batch_per_conn, new_indices[:, 1]].to(self.dtype)
        basis_factors = self.synaptic_basis_weights[new_syn_ids]
        new_weights_final = (new_weights * n_pre_spikes)[:, None] * basis_factors
        out = torch.zeros((batch_size * n_post, self._n_syn_basis), dtype=self.dtype)
        return out.index_add(0, segment_ids, new_weights_final)

    # ---- dense update --------------------------------------------------------------
    def update_psc(self, psc, psc_rise, rec_inputs):
        new_psc_rise = psc_rise * self.syn_decay + rec_inputs * self.psc_initial
        new_psc = psc * self.syn_decay + self._dt * self.syn_decay * psc_rise
        return new_psc, new_psc_rise

    def _dense_update_impl(self, batch_size, prev_z, v, r, asc, psc_rise, psc, rec_inputs):
        n, rr = self._n_neurons, self._n_syn_basis
        new_psc, new_psc_rise = self.update_psc(psc, psc_rise, rec_inputs)
        asc = asc.reshape(batch_size, n, 2)
        new_asc = self.asc_decay * asc + prev_z.detach()[..., None] * self.asc_amps
        new_asc = new_asc.reshape(batch_size, n * 2)
        input_current = _sum_last(psc.reshape(batch_size, n, rr))
        c1 = input_current + _sum_last(asc)
        dampened_v = straight_through_dampen(v, self._voltage_gradient_dampening)
        new_v = self.decay * dampened_v + self.current_factor * c1 - prev_z.detach()
        prev_spike = prev_z.detach().to(torch.int64)
        new_r = torch.clamp(r + prev_spike * self.t_ref_steps - 1, min=0)
        if self._hard_reset:
            new_v = torch.where(new_r > 0, torch.zeros_like(new_v), new_v)
        return new_v, new_r, new_asc, new_psc_rise, new_psc

    def zero_state(self, batch_size):
        n, r, d = self._n_neurons, self._n_syn_basis, self.max_delay
        z = lambda *s: torch.zeros(s, dtype=self.dtype)
        return (z(batch_size, n * d), z(batch_size, n), torch.zeros((batch_size, n), dtype=torch.int64),
                z(batch_size, n * 2), z(batch_size, n * r), z(batch_size, n * r),
                torch.zeros((batch_size,), dtype=torch.int32))

    def call(self, inputs, state, bkg_counts):
        """One timestep (``:1059-1135``).  ``bkg_counts[B, n_bkg]`` replaces the in-cell sampler."""
        n = self._n_neurons
        lgn_input = inputs[:, :self.input_dim]
        batch_size = inputs.shape[0]
        z_buf, v, r, asc, psc_rise, psc, noise_step = state
        prev_z = z_buf[:, :n]
        rec_z_buf = straight_through_dampen(z_buf, 1 - self._recurrent_dampening)
        i_rec = self.calculate_i_rec_with_custom_grad(rec_z_buf)
        external_current = self.calculate_input_current_from_spikes(lgn_input)
        i_noise = self.calculate_noise_current(batch_size, bkg_counts)
        rec_inputs = i_rec + external_current + i_noise
        rec_inputs = rec_inputs.reshape(batch_size, n * self._n_syn_basis)
        rec_inputs = rec_inputs * self._lr_scale
        new_v, new_r, new_asc, new_psc_rise, new_psc = self._dense_update_impl(
            batch_size, prev_z, v, r, asc, psc_rise, psc, rec_inputs)
        v_sc = new_v - 1.0
        new_z = SpikeFunction.apply(v_sc, self._dampening_factor, self._pseudo_width,
                                    self._gauss_std if self._pseudo_gauss else None)
        new_z = torch.where(new_r > 0, torch.zeros_like(new_z), new_z)
        new_z_buf = torch.cat([new_z, z_buf[:, :-n]], dim=1) if self.max_delay > 1 else new_z
        new_state = (new_z_buf, new_v, new_r, new_asc, new_psc_rise, new_psc, noise_step + 1)
        self.last_rec_inputs = rec_inputs
        return (new_z, new_v), new_state

    def rollout(self, x, bkg_counts, state=None, collect_states=False):
        """Keras ``RNN(cell, return_sequences=True)`` (``:1317-1322``): loop ``call`` over time.

        ``x[B,T,n_lgn]``, ``bkg_counts[B,T,n_bkg]`` -> ``z[B,T,N]``, ``v[B,T,N]``, final state.
        """
        b, t_len = x.shape[0], x.shape[1]
        if state is None:
            state = self.zero_state(b)
        zs, vs, states = [], [], []
        xf = x if x.dtype == torch.bool else x.to(self.dtype)
        for t in range(t_len):
            (z, v), state = self.call(xf[:, t], state, bkg_counts[:, t])
            zs.append(z)
            vs.append(v)
            if collect_states:
                states.append(tuple(s.detach().clone() for s in state) + (self.last_rec_inputs.detach().clone(),))
        out = (torch.stack(zs, 1), torch.stack(vs, 1), state)
        return out + (states,) if collect_states else out


def _sum_last(x):
    """Left-to-right sum over the last axis (the GPU kernels add channels in this order)."""
    acc = x[..., 0]
    for i in range(1, x.shape[-1]):
        acc = acc + x[..., i]
    return acc
