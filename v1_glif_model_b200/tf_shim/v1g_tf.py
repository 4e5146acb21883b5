"""TensorFlow glue over the custom ops of ``v1g_tf_ops.cc``: the reference's callables with their
own signatures, backed by ``libv1g.so``.

A maintainer of the reference replaces three things in ``v1_model_utils/models.py``:

* ``calculate_synaptic_currents`` (``:103-263``) by :func:`calculate_synaptic_currents` below - same
  nine positional arguments, same ``tf.custom_gradient`` contract: the gradient list has nine
  entries, of which entry 0 (``d rec_z_buf``, dense over all synapses) and entry 2 (``dW``, dense
  ``[nnz]`` in the reference's synapse order, master dtype) are tensors and the rest ``None``
  (``:251-261``);
* the bodies of ``calculate_input_current_from_spikes`` (``:814-863``), ``calculate_noise_current``
  (``:865-940``) and ``_dense_update_impl`` (``:985-1028``) by :func:`input_current`,
  :func:`noise_current` and :func:`dense_update`;
* or the whole ``tf.keras.layers.RNN(cell)`` loop (``:1317-1322``) by :func:`rollout`.

The library handle is created once per ``V1Column`` with :func:`create_handle` (ctypes, the same
calls as ``v1_glif_model_b200/models.py`` makes) and passed to the ops as its integer address.
This module imports TensorFlow and is therefore usable only where TensorFlow is installed; the ops
library is built by ``build_tf_shim.py``.
"""
import ctypes
import os

import tensorflow as tf

HERE = os.path.dirname(os.path.abspath(__file__))
_ops = tf.load_op_library(os.path.join(HERE, "libv1g_tf_ops.so"))

SRC_REC, SRC_LGN, SRC_BKG = 0, 1, 2


def create_handle(cell_kwargs):
    """A ``V1GHandle`` for one ``V1Column``; ``cell_kwargs`` = the dictionaries and scalars that
    ``v1_glif_model_b200.models.V1Column`` takes.  Returns ``(address, column)``; keep ``column``
    alive for as long as ops use the address."""
    from v1_glif_model_b200.models import V1Column
    column = V1Column(**cell_kwargs)
    return ctypes.cast(column._libh, ctypes.c_void_p).value, column


def _currents(handle, source, n_neurons, n_receptors, nnz):
    """``x -> i_flat`` with the reference's gradient ``[d_x, dW]`` for one synaptic source."""
    @tf.custom_gradient
    def op(x, weight_values):
        i_flat = _ops.v1g_syn_currents(x=x, handle=handle, source=source, n_neurons=n_neurons,
                                       n_receptors=n_receptors)

        def grad(dy):
            d_x, d_w = _ops.v1g_syn_currents_grad(x=x, dy=dy, handle=handle, source=source, nnz=nnz)
            return d_x, tf.cast(d_w, weight_values.dtype)
        return i_flat, grad
    return op


def calculate_synaptic_currents(handle, n_neurons):
    """The replacement for ``calculate_synaptic_currents`` (``models.py:103-263``), bound to a handle."""
    @tf.custom_gradient
    def fn(rec_z_buf, synapse_indices, weight_values, weight_values_compute, dense_shape,
           synaptic_basis_weights, syn_ids, pre_ind_table):
        n_receptors = int(synaptic_basis_weights.shape[1])
        nnz = int(weight_values.shape[0])
        i_rec_flat = _ops.v1g_syn_currents(x=rec_z_buf, handle=handle, source=SRC_REC, n_neurons=n_neurons,
                                           n_receptors=n_receptors)

        def grad(dy):
            d_z, d_w = _ops.v1g_syn_currents_grad(x=rec_z_buf, dy=dy, handle=handle, source=SRC_REC, nnz=nnz)
            # nine entries, one per argument (models.py:251-261)
            return [d_z, None, tf.cast(d_w, weight_values.dtype), None, None, None, None, None, None]
        return i_rec_flat, grad
    return fn


def input_current(handle, n_neurons, n_receptors, nnz):
    """``calculate_input_current_from_spikes(x_t)`` (``models.py:814-863``): ``fn(x_t, input_weight_values)``."""
    return _currents(handle, SRC_LGN, n_neurons, n_receptors, nnz)


def noise_current(handle, n_neurons, n_receptors, nnz):
    """``calculate_noise_current`` with the counts given (``models.py:890-940``): ``fn(counts, bkg_input_weights)``."""
    return _currents(handle, SRC_BKG, n_neurons, n_receptors, nnz)


def dense_update(handle):
    """``_dense_update_impl`` + ``spike_function`` + the tail of ``call`` (``models.py:985-1028, 1099-1117``):
    ``fn(z_buf, v, r, asc, psc_rise, psc, rec_inputs) -> (new state..., z)`` with the adjoint of
    ``v1g_step_bwd`` (stop-gradients and straight-through factors of ``models.py:994, 1010-1018, 58-64``)."""
    @tf.custom_gradient
    def fn(z_buf, v, r, asc, psc_rise, psc, rec_inputs):
        out = _ops.v1g_step(z_buf=z_buf, v=v, r=r, asc=asc, psc_rise=psc_rise, psc=psc, rec_inputs=rec_inputs,
                            handle=handle)
        new_v, new_r = out[1], out[2]

        def grad(g_z_buf, g_v, g_r, g_asc, g_psc_rise, g_psc, g_z):
            d = _ops.v1g_step_grad(g_z_buf=g_z_buf, g_v=g_v, g_r=tf.zeros_like(new_r), g_asc=g_asc,
                                   g_psc_rise=g_psc_rise, g_psc=g_psc, g_z=g_z, g_v_out=tf.zeros_like(g_v),
                                   new_v=new_v, new_r=new_r, handle=handle)
            return [d[0], d[1], None, d[3], d[4], d[5], d[6]]
        return tuple(out), grad
    return fn


def compact_spikes(x):
    """``tf.where(x > 0)`` as int64 ``[n, 2]`` (``models.py:128``)."""
    coords, count = _ops.v1g_compact_spikes(x=x)
    return coords[:count[0]]


def rollout(handle, n_neurons, nnz):
    """The RNN loop (``models.py:1317-1322``) from the zero state: ``fn(x, bkg_counts, w_rec, w_lgn, w_bkg)
    -> (z, v)`` with weight gradients from BPTT inside the library.  ``nnz`` = the three synapse counts."""
    @tf.custom_gradient
    def fn(x, bkg_counts, w_rec, w_lgn, w_bkg):
        z, v = _ops.v1g_rollout(x=x, bkg_counts=bkg_counts, handle=handle, n_neurons=n_neurons, save_for_bwd=True)

        def grad(g_z, g_v):
            d = _ops.v1g_rollout_grad(g_z=g_z, g_v=g_v, handle=handle, nnz_rec=nnz[0], nnz_lgn=nnz[1], nnz_bkg=nnz[2])
            return [None, None, d[0], d[1], d[2]]
        # spikes leave as float so that the gradient is not cut (models.py:1125)
        return (tf.cast(z, v.dtype), v), grad
    return fn
