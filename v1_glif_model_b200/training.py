"""Data-parallel training step around the fused rollouts.

Mirrors the reference's ``train_step_combined`` (``multi_training.py:483-560``): one forward
rollout, BPTT, a sum of the dense fp32 weight gradients over replicas, then an
``ExponentiatedAdam`` step (``v1_model_utils/optimizers.py:353-376``) followed by the sign
constraint (``models.py:419-427``) and a refresh of the kernels' weight copies
(``models.py:966-976``).  The reference reduces gradients inside
``optimizer.apply_gradients`` under ``MirroredStrategy`` with ``HierarchicalCopyAllReduce``
(``tf_utils.py:131-139``); here every rank is one process with one GPU and the three gradients
live in ONE flat buffer that is all-reduced in place with a single NCCL call.  Losses are
pre-scaled by ``1/world_size`` as in ``multi_training.py:427-429``, so the reduction is a sum.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib


class FlatGradients:
    """One flat fp32 buffer holding the gradients of several weight vectors back to back.

    ``views[i]`` aliases the slice of weight vector ``i``; ``all_reduce`` sums the whole buffer
    over the process group in one collective (a no-op for a single process).
    """

    def __init__(self, sizes, device):
        self.sizes = [int(s) for s in sizes]
        self.flat = torch.zeros(sum(self.sizes), dtype=torch.float32, device=device)
        self.views = []
        off = 0
        for s in self.sizes:
            self.views.append(self.flat[off:off + s])
            off += s

    def zero_(self):
        self.flat.zero_()

    def all_reduce(self, group=None):
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
        return self.flat


class ExponentiatedAdam:
    """Exponentiated-gradient Adam on flat fp32 weights (``optimizers.py:353-376``).

    ``m += (g - m)(1 - b1)``, ``v += (g^2 - v)(1 - b2)``,
    ``alpha = lr * sqrt(1 - b2^t) / (1 - b1^t)``,
    ``w <- w * exp(-alpha * m / (sqrt(v) + eps) * sign(w))`` with ``sign(0) = +1``, then the sign
    constraint ``where(positive, relu(w), -relu(-w))``.  The arithmetic runs in one CUDA kernel of
    ``libv1g.so``.
    """

    def __init__(self, params, positives, learning_rate=1e-3, beta_1=0.9, beta_2=0.999,
                 epsilon=1e-11):
        self.params = list(params)
        self.positives = [p.to(torch.uint8).contiguous() for p in positives]
        self.lr, self.b1, self.b2, self.eps = learning_rate, beta_1, beta_2, epsilon
        self.m = [torch.zeros_like(p) for p in self.params]
        self.v = [torch.zeros_like(p) for p in self.params]
        self.iterations = 0

    def apply_gradients(self, grads, grad_scale=1.0):
        lib = _lib.load()
        self.iterations += 1
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        for p, g, m, v, pos in zip(self.params, grads, self.m, self.v, self.positives):
            if not p.is_cuda:
                raise RuntimeError("ExponentiatedAdam runs on the GPU only")
            rc = lib.v1g_expadam_update(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(),
                                        pos.data_ptr(), p.numel(), self.lr, self.b1, self.b2,
                                        self.eps, self.iterations, grad_scale, stream)
            if rc != _lib.OK:
                raise _lib.V1GError(rc, "v1g_expadam_update failed")


class _DevicePointer:
    """A raw device address with a length, duck-typed like the two tensor methods the regulariser uses."""

    def __init__(self, address, n):
        self._address, self._n = address, n

    def data_ptr(self):
        return self._address

    def numel(self):
        return self._n


class WeightRegularizer:
    """A weight regulariser of the reference on the device: ``kind="mean_stiff"``
    (``MeanStiffRegularizer``, ``loss_functions.py:171-220``; ``relative`` = ``penalize_relative_change``)
    or ``kind="emd"`` (``EarthMoversDistanceRegularizer``, ``:536-601``).

    ``edge_type_ids`` and ``initial_weights`` (the weights after division by the voltage scale, as the
    reference prepares them) are per recurrent synapse in the caller's order.  ``order="internal"``
    converts both to the library's own synapse order, the order of ``Trainer``'s gradient buffer.
    Calling the object adds ``strength * value`` to ``loss[0]`` and the gradient to ``grad``."""

    def __init__(self, cell, kind, edge_type_ids, initial_weights, strength, relative=False, order="reference",
                 source=_lib.SRC_REC):
        import numpy as np
        self.cell, self.kind, self.strength = cell, {"mean_stiff": 0, "emd": 1}[kind], float(strength)
        ids = np.asarray(edge_type_ids)
        w0 = np.asarray(initial_weights, dtype=np.float64)
        if order == "internal":
            perm = np.empty(ids.shape[0], dtype=np.int32)
            cell._check(cell._lib.v1g_get_internal_order(cell._libh, source, perm.ctypes.data))
            ids, w0 = ids[perm], w0[perm]
        _, idx = np.unique(ids, return_inverse=True)
        self.n_groups = int(idx.max()) + 1
        counts = np.bincount(idx, minlength=self.n_groups)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cell.device)
        self.group_ids = dev(idx.astype(np.int32))
        self.offsets, self.denominator = None, None
        if self.kind == 0:
            target = np.bincount(idx, weights=w0, minlength=self.n_groups) / counts
            self.target = dev(target.astype(np.float32))
            if relative:
                self.denominator = dev(np.maximum(np.abs(target), 1e-4).astype(np.float32))
        else:
            by_group = np.lexsort((w0, idx))            # groups ascending, weights ascending inside
            self.target = dev(w0[by_group].astype(np.float32))
            self.offsets = dev(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32))

    def __call__(self, w, grad, loss=None):
        c = self.cell
        p = lambda t: t.data_ptr() if t is not None else None
        c._check(c._lib.v1g_weight_regularizer(
            c._libh, self.kind, w.data_ptr(), self.group_ids.data_ptr(), w.numel(), self.n_groups,
            self.target.data_ptr(), p(self.offsets), p(self.denominator), self.strength, p(loss), grad.data_ptr(),
            C.c_void_p(torch.cuda.current_stream().cuda_stream)))


class Trainer:
    """One replica of the data-parallel training loop (batch sharded over ranks).

    ``order="internal"`` (default) keeps gradients, Adam moments and the update in the synapse
    order of the kernels, which is the same on every replica, and skips the per-step conversions
    to and from the caller's order; ``cell.pull_weights()`` (called by ``weights()``) converts
    back on demand.  ``order="reference"`` goes through the caller's order every step.
    """

    def __init__(self, cell, loss, learning_rate=1e-3, train_input=True, train_noise=False,
                 group=None, order="internal", regularizers=()):
        self.cell = cell
        # weight regularisers of the recurrent weights (WeightRegularizer objects built with the same
        # `order`); their gradient joins the reduced gradient once, their value the total loss
        self.regularizers = tuple(regularizers)
        self.order = order
        self.lr = learning_rate
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.loss = dict(loss)
        self.loss["loss_scale"] = self.loss.get("loss_scale", 1.0) / self.world
        weights = [cell.recurrent_weight_values, cell.input_weight_values, cell.bkg_input_weights]
        positives = [cell.recurrent_weight_positive, cell.input_weight_positive,
                     cell.bkg_input_weight_positive]
        self.trainable = [True, bool(train_input), bool(train_noise)]
        self.grads = FlatGradients(cell.train_layout(), cell.device)
        self.train_mask = sum(1 << i for i, t in enumerate(self.trainable) if t)
        if order == "internal":
            self.m = torch.zeros_like(self.grads.flat)
            self.v = torch.zeros_like(self.grads.flat)
            self.iterations = 0
            self._losses = torch.zeros((4,), dtype=torch.float32, device=cell.device)
        sel = [i for i, t in enumerate(self.trainable) if t]
        self.opt = ExponentiatedAdam([weights[i] for i in sel], [positives[i] for i in sel],
                                     learning_rate=learning_rate)
        self._sel = sel

    def step(self, x, bkg_counts=None, state=None):
        """Forward rollout, BPTT, gradient all-reduce, Exp-Adam update.  Returns losses[4].

        Without ``bkg_counts`` the background noise is drawn on the device and the noise seed is
        advanced by one afterwards, as the reference's loop does once per rollout
        (``tf_utils.py:235-237``, ``multi_training.py:380``).  ``state`` is the carried state the
        rollout starts from (updated in place), e.g. the gray-screen state of
        ``multi_training.py:812-831``."""
        self.grads.zero_()
        self.cell.rollout(x, bkg_counts, state=state, return_z=False, return_v=False, save_for_bwd=True)
        if bkg_counts is None:
            self.cell.set_noise_seed(self.cell.noise_seed + 1)
        return self._finish_step()

    def step_rates(self, rates, lgn_seed, batch_size, state=None):
        """``step`` with both stochastic inputs drawn on the device: LGN spikes from the firing rates
        ``rates[T,n_lgn]`` / ``[B,T,n_lgn]`` with ``lgn_seed``, background counts from the cell's noise
        seed.  Nothing but the seeds comes from the host."""
        self.grads.zero_()
        self.cell.rollout_rates(rates, lgn_seed, batch_size, state=state, return_z=False, return_v=False,
                                save_for_bwd=True)
        self.cell.set_noise_seed(self.cell.noise_seed + 1)
        return self._finish_step()

    def _finish_step(self):
        if self.order == "internal":
            cell = self.cell
            losses = cell.backward_internal(self.loss, self.grads.flat, self._losses)
            # a rollout kernel whose bounded grid-barrier wait gave up leaves garbage behind: raise
            # here (V1GError, code ETIMEOUT) before the gradients reach the other replicas or the weights
            cell.synchronize()
            self.grads.all_reduce(self.group)
            if self.regularizers:
                w_int = C.c_void_p()
                cell._check(cell._lib.v1g_internal_weights(cell._libh, _lib.SRC_REC, C.byref(w_int)))
                n_rec = self.grads.sizes[0]
                w_view = _DevicePointer(w_int.value, n_rec)
                for reg in self.regularizers:
                    reg(w_view, self.grads.views[0], losses)
            self.iterations += 1
            cell._check(cell._lib.v1g_expadam_update_internal(
                cell._libh, self.grads.flat.data_ptr(), self.m.data_ptr(), self.v.data_ptr(),
                self.train_mask, self.lr, 0.9, 0.999, 1e-11, self.iterations, 1.0,
                C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            return losses
        _, _, _, losses = self.cell.backward(self.loss, accumulate_into=self.grads.views)
        self.cell.synchronize()                  # as above: no update from an aborted rollout
        self.grads.all_reduce(self.group)
        for reg in self.regularizers:
            reg(self.cell.recurrent_weight_values, self.grads.views[0], losses)
        self.opt.apply_gradients([self.grads.views[i] for i in self._sel])
        self.cell.refresh_weights()
        return losses

    def weights(self):
        """The three weight tensors in the caller's synapse order, up to date."""
        if self.order == "internal":
            self.cell.pull_weights()
        c = self.cell
        return c.recurrent_weight_values, c.input_weight_values, c.bkg_input_weights
