"""The Python half of the TensorFlow shim (``v1_glif_model_b200/tf_shim/v1g_tf.py``) run on the GPU.

TensorFlow is not installed here, so the glue is imported over the torch-backed stand-in of
``tests/golden/tf_standin.py`` and ``tf.load_op_library`` returns ops written in Python that do what the
``Compute`` methods of ``v1g_tf_ops.cc`` do: allocate the outputs and call the same C-ABI entry points
with the same arguments.  What this exercises is the glue itself: the reference's call signatures, the
``tf.custom_gradient`` contracts (nine gradient entries of ``calculate_synaptic_currents``,
``models.py:251-261``) and the routing of gradients to the weight variables, checked against the oracle.
"""
import ctypes as C
import importlib
import os
import sys

import numpy as np
import pytest
import torch

from util import TOL_GRAD, TOL_STATE, make_cells, make_inputs, rel_err

pytestmark = pytest.mark.gpu
KW = dict(dampening_factor=0.5, pseudo_width=0.5, recurrent_dampening_factor=0.4, voltage_gradient_dampening=0.3)


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class OpsInPython:
    """One method per REGISTER_OP of v1g_tf_ops.cc, same attribute and input names."""

    def __init__(self, lib):
        self.lib = lib

    def _ok(self, rc, handle=None):
        assert rc == 0, self.lib.v1g_last_error(C.c_void_p(handle) if handle else None).decode()

    def v1g_syn_currents(self, x, handle, source, n_neurons, n_receptors):
        x = x.contiguous()
        out = torch.empty((x.shape[0] * n_neurons, n_receptors), dtype=torch.float32, device=x.device)
        self._ok(self.lib.v1g_syn_currents_fwd(C.c_void_p(handle), source, _p(x), x.shape[0], _p(out), _stream()), handle)
        return out

    def v1g_syn_currents_grad(self, x, dy, handle, source, nnz):
        x, dy = x.contiguous(), dy.contiguous()
        d_x = torch.empty_like(x)
        d_w = torch.empty((nnz,), dtype=torch.float32, device=x.device)
        self._ok(self.lib.v1g_syn_currents_bwd(C.c_void_p(handle), source, _p(x), _p(dy), x.shape[0], _p(d_x), _p(d_w),
                                               _stream()), handle)
        return d_x, d_w

    def v1g_compact_spikes(self, x):
        x = x.contiguous()
        rows, cols = x.shape
        coords = torch.empty((rows * cols, 2), dtype=torch.int64, device=x.device)
        count = torch.empty((1,), dtype=torch.int32, device=x.device)
        self._ok(self.lib.v1g_compact_spikes_noalloc(_p(x), rows, cols, _p(coords), rows * cols, _p(count), _stream()))
        return coords, count

    def v1g_rollout(self, x, bkg_counts, handle, n_neurons, save_for_bwd):
        x, bkg_counts = x.contiguous(), bkg_counts.contiguous()
        b, t = x.shape[0], x.shape[1]
        z = torch.empty((b, t, n_neurons), dtype=torch.uint8, device=x.device)
        v = torch.empty((b, t, n_neurons), dtype=torch.float32, device=x.device)
        self._keep = (x, bkg_counts)          # the library reads the inputs again in the backward pass
        self._ok(self.lib.v1g_rollout_fwd(C.c_void_p(handle), b, t, _p(x), _p(bkg_counts) if bkg_counts.numel() else None,
                                          None, _p(z), _p(v), 1 if save_for_bwd else 0, _stream()), handle)
        return z, v

    def v1g_rollout_grad(self, g_z, g_v, handle, nnz_rec, nnz_lgn, nnz_bkg):
        g_z, g_v = g_z.contiguous(), g_v.contiguous()
        d = [torch.zeros((n,), dtype=torch.float32, device=g_z.device) for n in (nnz_rec, nnz_lgn, nnz_bkg)]
        self._ok(self.lib.v1g_rollout_bwd(C.c_void_p(handle), None, _p(g_z), _p(g_v), _p(d[0]), _p(d[1]), _p(d[2]), None,
                                          _stream()), handle)
        return d


    # state tensors in the reference's order: z_buf, v, r (int8), asc, psc_rise, psc
    def _state(self, t):
        from v1_glif_model_b200 import _lib
        return _lib.V1GState(*[x.data_ptr() for x in t], None)

    def v1g_step(self, z_buf, v, r, asc, psc_rise, psc, rec_inputs, handle):
        ins = [x.contiguous() for x in (z_buf, v, r, asc, psc_rise, psc)]
        outs = [torch.empty_like(x) for x in ins]
        z = torch.empty_like(ins[1])
        rec_inputs = rec_inputs.contiguous()
        s_in, s_out = self._state(ins), self._state(outs)
        self._ok(self.lib.v1g_step_fwd(C.c_void_p(handle), ins[1].shape[0], C.byref(s_in), _p(rec_inputs), C.byref(s_out),
                                       _p(z), _stream()), handle)
        return outs + [z]

    def v1g_step_grad(self, g_z_buf, g_v, g_r, g_asc, g_psc_rise, g_psc, g_z, g_v_out, new_v, new_r, handle):
        gs = [x.contiguous() for x in (g_z_buf, g_v, g_r, g_asc, g_psc_rise, g_psc)]
        outs = [torch.empty_like(x) for x in gs]
        d_rec = torch.empty_like(gs[5])
        keep = [x.contiguous() for x in (g_z, g_v_out, new_v, new_r)]
        s_out, s_in = self._state(gs), self._state(outs)
        self._ok(self.lib.v1g_step_bwd(C.c_void_p(handle), gs[1].shape[0], C.byref(s_out), _p(keep[0]), _p(keep[1]),
                                       _p(keep[2]), _p(keep[3]), C.byref(s_in), _p(d_rec), _stream()), handle)
        return outs + [d_rec]


@pytest.fixture()
def glue():
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, golden)
    import tf_standin
    from v1_glif_model_b200 import _lib
    saved = sys.modules.get("tensorflow")
    tf = tf_standin.install()
    tf.load_op_library = lambda path: OpsInPython(_lib.load())
    sys.modules.pop("v1_glif_model_b200.tf_shim.v1g_tf", None)
    mod = importlib.import_module("v1_glif_model_b200.tf_shim.v1g_tf")
    yield mod
    sys.modules.pop("v1_glif_model_b200.tf_shim.v1g_tf", None)
    for name in [m for m in sys.modules if m == "tensorflow" or m.startswith("tensorflow.")]:
        del sys.modules[name]
    if saved is not None:
        sys.modules["tensorflow"] = saved
    sys.path.remove(golden)


def _handle(cell):
    return C.cast(cell._libh, C.c_void_p).value


def test_calculate_synaptic_currents_keeps_the_reference_contract(glue):
    cfg, dicts, orc, cell = make_cells("small", **KW)
    n, d, r = cfg.n_neurons, orc.max_delay, orc._n_syn_basis
    g = torch.Generator().manual_seed(6)
    z_cpu = (torch.rand(2, n * d, generator=g) < 0.05).float().requires_grad_(True)
    dy = torch.randn(2 * n, r, generator=g)
    want = orc.calculate_i_rec_with_custom_grad(z_cpu)
    gz, gw = torch.autograd.grad(want, [z_cpu, orc.recurrent_weight_values], dy)

    fn = glue.calculate_synaptic_currents(_handle(cell), n)
    z_buf = z_cpu.detach().cuda().requires_grad_(True)
    weights = cell.recurrent_weight_values.clone().requires_grad_(True)
    out = fn(z_buf, cell.recurrent_indices, weights, weights, cell.recurrent_dense_shape,
             torch.from_numpy(np.asarray(dicts[0]["synaptic_basis_weights"])), None, None)
    assert out.shape == (2 * n, r) and rel_err(out, want.detach()) <= TOL_STATE
    out.backward(dy.cuda())
    assert rel_err(z_buf.grad, gz) <= TOL_GRAD and rel_err(weights.grad, gw) <= TOL_GRAD


def test_input_and_noise_currents_route_the_weight_gradient(glue):
    cfg, dicts, orc, cell = make_cells("small", **KW)
    n, r = cfg.n_neurons, orc._n_syn_basis
    g = torch.Generator().manual_seed(8)
    dy = torch.randn(2 * n, r, generator=g)
    x_t = (torch.rand(2, cfg.n_lgn, generator=g) < 0.1).float()
    counts = torch.poisson(torch.full((2, cfg.n_bkg), 0.4), generator=g)
    (gl,) = torch.autograd.grad(orc.calculate_input_current_from_spikes(x_t), [orc.input_weight_values], dy)
    (gb,) = torch.autograd.grad(orc.calculate_noise_current(2, counts.long()), [orc.bkg_input_weights], dy)
    for make, x, w0, want in ((glue.input_current, x_t, cell.input_weight_values, gl),
                              (glue.noise_current, counts, cell.bkg_input_weights, gb)):
        w = w0.clone().requires_grad_(True)
        out = make(_handle(cell), n, r, w.shape[0])(x.cuda(), w)
        out.backward(dy.cuda())
        assert rel_err(w.grad, want) <= TOL_GRAD


def test_compact_spikes_is_tf_where(glue):
    g = torch.Generator().manual_seed(3)
    x = (torch.rand(5, 777, generator=g) < 0.07).float()
    got = glue.compact_spikes(x.cuda())
    assert torch.equal(got.cpu(), torch.nonzero(x > 0))


def test_rollout_returns_float_spikes_and_weight_gradients(glue):
    cfg, dicts, orc, cell = make_cells("small", **KW)
    x, c = make_inputs(cfg, seq_len=30)
    xd, cd = torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda()
    ws = [w.clone().requires_grad_(True) for w in (cell.recurrent_weight_values, cell.input_weight_values,
                                                    cell.bkg_input_weights)]
    fn = glue.rollout(_handle(cell), cfg.n_neurons, [w.shape[0] for w in ws])
    z, v = fn(xd, cd, *ws)
    assert z.dtype == torch.float32                       # not cut by an integer output (models.py:1125)
    zo, vo, _ = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    assert torch.equal(z.cpu(), zo.detach()) and rel_err(v, vo.detach()) <= TOL_STATE
    g = torch.Generator().manual_seed(4)
    g_z, g_v = torch.randn(z.shape, generator=g) * 1e-3, torch.randn(v.shape, generator=g) * 1e-3
    ((z * g_z.cuda()).sum() + (v * g_v.cuda()).sum()).backward()
    for w in (orc.recurrent_weight_values, orc.input_weight_values, orc.bkg_input_weights):
        w.grad = None
    ((zo * g_z).sum() + (vo * g_v).sum()).backward()
    for got, want in zip(ws, (orc.recurrent_weight_values, orc.input_weight_values, orc.bkg_input_weights)):
        assert rel_err(got.grad, want.grad) <= TOL_GRAD


def test_dense_update_step_and_its_adjoint(glue):
    """``dense_update`` = ``_dense_update_impl`` + ``spike_function`` + the tail of ``call`` as one op with the
    adjoint of ``v1g_step_bwd``: new state and spikes against the oracle, gradients of a random cotangent
    against autograd through the oracle's step (stop-gradients of ``models.py:994, 1010-1018``)."""
    from oracle.cell_torch import SpikeFunction
    cfg, dicts, orc, cell = make_cells("small", dampening_factor=0.5, pseudo_width=0.5)
    n, d, r = cfg.n_neurons, orc.max_delay, orc._n_syn_basis
    g = torch.Generator().manual_seed(8)
    b = 2
    z_buf = (torch.rand(b, n * d, generator=g) < 0.1).float()
    leaves = [t.requires_grad_(True) for t in (torch.randn(b, n, generator=g) * 0.5 + 0.6,
                                               torch.randn(b, n * 2, generator=g), torch.randn(b, n * r, generator=g),
                                               torch.randn(b, n * r, generator=g), torch.randn(b, n * r, generator=g))]
    v, asc, psc_rise, psc, rec_inputs = leaves
    rr = torch.randint(0, 2, (b, n), generator=g)
    nv, nr, nasc, npr, npsc = orc._dense_update_impl(b, z_buf[:, :n], v, rr, asc, psc_rise, psc, rec_inputs)
    z = SpikeFunction.apply(nv - 1.0, 0.5, 0.5, None)
    z = torch.where(nr > 0, torch.zeros_like(z), z)
    cot = [torch.randn(t.shape, generator=g) for t in (nv, nasc, npr, npsc, z)]
    want = torch.autograd.grad(sum((t * c).sum() for t, c in zip((nv, nasc, npr, npsc, z), cot)), leaves)

    dv = [t.detach().cuda().requires_grad_(True) for t in leaves]
    fn = glue.dense_update(_handle(cell))
    out = fn(z_buf.cuda(), dv[0], rr.to(torch.int8).cuda(), dv[1], dv[2], dv[3], dv[4])
    new_z_buf, new_v, new_r, new_asc, new_pr, new_psc, z_dev = out
    assert torch.equal(new_v.detach().cpu(), nv.detach()) and torch.equal(new_r.cpu().long(), nr)
    assert torch.equal(z_dev.detach().cpu(), z.detach())
    assert torch.equal(new_z_buf.detach().cpu()[:, :n], z.detach()) and \
        torch.equal(new_z_buf.detach().cpu()[:, n:], z_buf[:, :-n])
    loss = sum((t * c.cuda()).sum() for t, c in zip((new_v, new_asc, new_pr, new_psc, z_dev), cot))
    loss.backward()
    for got, w in zip(dv, want):
        assert rel_err(got.grad, w) <= TOL_GRAD

