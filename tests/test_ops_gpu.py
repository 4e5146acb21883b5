"""GPU parity of the operator-level entry points (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from util import TOL_GRAD, TOL_STATE, make_case, make_inputs, rel_err

pytestmark = pytest.mark.gpu


def _cells(name, **kw):
    from v1_glif_model_b200.models import V1Column
    dense = kw.pop("dense_basis", False)
    nrec = kw.pop("n_receptors", None)
    cfg, dicts, orc = make_case(name, dense_basis=dense, n_receptors=nrec, **kw)
    return cfg, dicts, orc, V1Column(*dicts, **kw)


@pytest.mark.parametrize("shape,p", [((1, 1), 1.0), ((3, 7), 0.5), ((2, 4096), 0.01), ((5, 4097), 0.3),
                                     ((4, 12345), 0.0), ((2, 9000), 1.0), ((7, 33), 0.1)])
def test_compaction_is_bit_exact(shape, p):
    """tf.where order: row-major int64 coordinates; empty, full and ragged inputs."""
    cfg, dicts, orc, cell = _cells("tiny")
    g = torch.Generator().manual_seed(shape[1])
    x = (torch.rand(shape, generator=g) < p).float()
    x[x > 0] *= torch.rand(int(x.sum()), generator=g) + 0.1   # any positive value counts
    got = cell.compact_spikes(x.cuda())
    want = torch.nonzero(x > 0)
    assert got.dtype == torch.int64
    assert torch.equal(got.cpu(), want)


def test_pre_ind_table_inside_library_matches_oracle():
    cfg, dicts, orc, cell = _cells("small")
    for src, tab in ((0, orc.pre_ind_table), (1, orc.pre_input_ind_table), (2, orc.pre_bkg_ind_table)):
        order, splits = cell.pre_ind_table(src)
        assert np.array_equal(order, tab.order.numpy())
        assert np.array_equal(splits, tab.row_splits.numpy())


@pytest.mark.parametrize("dense_basis", [False, True])
def test_synaptic_currents_forward_three_sources(dense_basis):
    cfg, dicts, orc, cell = _cells("small", dense_basis=dense_basis)
    n, d = cfg.n_neurons, orc.max_delay
    g = torch.Generator().manual_seed(5)
    z_buf = (torch.rand(3, n * d, generator=g) < 0.05).float()
    x_t = (torch.rand(3, cfg.n_lgn, generator=g) < 0.1).float()
    counts = torch.poisson(torch.full((3, cfg.n_bkg), 0.4), generator=g)
    with torch.no_grad():
        want = [orc.calculate_i_rec_with_custom_grad(z_buf), orc.calculate_input_current_from_spikes(x_t),
                orc.calculate_noise_current(3, counts.long())]
    got = [cell.calculate_i_rec_with_custom_grad(z_buf.cuda()),
           cell.calculate_input_current_from_spikes(x_t.cuda()),
           cell.calculate_noise_current(3, counts=counts.cuda())]
    for a, b in zip(got, want):
        assert a.shape == b.shape
        assert rel_err(a, b) <= TOL_STATE
    # empty input -> exactly zero
    assert float(cell.calculate_i_rec_with_custom_grad(torch.zeros(3, n * d).cuda()).abs().max()) == 0.0


def test_synaptic_currents_linearity():
    """Size-independent property: currents of disjoint spike sets add up."""
    cfg, dicts, orc, cell = _cells("small")
    n, d = cfg.n_neurons, orc.max_delay
    g = torch.Generator().manual_seed(9)
    m = torch.rand(2, n * d, generator=g)
    a, b = (m < 0.03).float().cuda(), ((m > 0.5) & (m < 0.53)).float().cuda()
    ia, ib, iab = (cell.calculate_i_rec_with_custom_grad(t) for t in (a, b, a + b))
    assert rel_err(ia + ib, iab) <= TOL_STATE


@pytest.mark.parametrize("dense_basis", [False, True])
def test_synaptic_currents_gradient(dense_basis):
    cfg, dicts, orc, cell = _cells("small", dense_basis=dense_basis)
    n, d, r = cfg.n_neurons, orc.max_delay, orc._n_syn_basis
    g = torch.Generator().manual_seed(6)
    z_buf = (torch.rand(2, n * d, generator=g) < 0.05).float().requires_grad_(True)
    dy = torch.randn(2 * n, r, generator=g)
    out = orc.calculate_i_rec_with_custom_grad(z_buf)
    gz, gw = torch.autograd.grad(out, [z_buf, orc.recurrent_weight_values], dy)
    d_x, d_w = cell.syn_currents_grad(0, z_buf.detach().cuda(), dy.cuda())
    assert rel_err(d_x, gz) <= TOL_GRAD
    assert rel_err(d_w, gw) <= TOL_GRAD
    # LGN and background: autodiff of the forward ops in the reference
    x_t = (torch.rand(2, cfg.n_lgn, generator=g) < 0.1).float()
    counts = torch.poisson(torch.full((2, cfg.n_bkg), 0.4), generator=g)
    (gl,) = torch.autograd.grad(orc.calculate_input_current_from_spikes(x_t), [orc.input_weight_values], dy)
    (gb,) = torch.autograd.grad(orc.calculate_noise_current(2, counts.long()), [orc.bkg_input_weights], dy)
    _, d_wl = cell.syn_currents_grad(1, x_t.cuda(), dy.cuda(), want_dx=False)
    _, d_wb = cell.syn_currents_grad(2, counts.cuda(), dy.cuda(), want_dx=False)
    assert rel_err(d_wl, gl) <= TOL_GRAD
    assert rel_err(d_wb, gb) <= TOL_GRAD


@pytest.mark.parametrize("kw", [dict(), dict(hard_reset=True), dict(voltage_gradient_dampening=0.3)])
def test_dense_step_is_bit_exact(kw):
    """Given identical inputs the dense update reproduces the fp32 oracle bit for bit."""
    cfg, dicts, orc, cell = _cells("small", **kw)
    n, d, r = cfg.n_neurons, orc.max_delay, orc._n_syn_basis
    g = torch.Generator().manual_seed(7)
    b = 3
    state = ((torch.rand(b, n * d, generator=g) < 0.1).float(), torch.randn(b, n, generator=g) * 0.6 + 0.5,
             torch.randint(0, 3, (b, n), generator=g), torch.randn(b, n * 2, generator=g),
             torch.randn(b, n * r, generator=g), torch.randn(b, n * r, generator=g))
    rec_inputs = torch.randn(b, n * r, generator=g)
    with torch.no_grad():
        nv, nr, nasc, npr, npsc = orc._dense_update_impl(b, state[0][:, :n], state[1], state[2], state[3],
                                                         state[4], state[5], rec_inputs)
    gstate = (state[0].cuda(), state[1].cuda(), state[2].to(torch.int8).cuda(), state[3].cuda(),
              state[4].cuda(), state[5].cuda())
    gv, gr, gasc, gpr, gpsc = cell._dense_update_impl(b, gstate[0][:, :n], *gstate[1:], rec_inputs.cuda())
    assert torch.equal(gv.cpu(), nv) and torch.equal(gasc.cpu(), nasc)
    assert torch.equal(gpr.cpu(), npr) and torch.equal(gpsc.cpu(), npsc)
    assert torch.equal(gr.cpu().long(), nr)
    p2, pr2 = cell.update_psc(gstate[5], gstate[4], rec_inputs.cuda())
    assert torch.equal(p2.cpu(), npsc) and torch.equal(pr2.cpu(), npr)


def test_call_teacher_forced_rollout():
    """Step by step through the operator-level call with the oracle's state fed in each step."""
    cfg, dicts, orc, cell = _cells("small")
    x, c = make_inputs(cfg, seq_len=25)
    xo, co = torch.from_numpy(x).float(), torch.from_numpy(c).long()
    state = orc.zero_state(cfg.batch)
    for t in range(25):
        with torch.no_grad():
            (z, v), new_state = orc.call(xo[:, t], state, co[:, t])
        gstate = tuple(s.cuda() for s in state[:2]) + (state[2].to(torch.int8).cuda(),) + \
            tuple(s.cuda() for s in state[3:6]) + (state[6].cuda(),)
        (gz, gv), gnew = cell.call(xo[:, t].cuda(), gstate, bkg_counts=co[:, t].cuda())
        assert rel_err(cell.last_rec_inputs, orc.last_rec_inputs) <= TOL_STATE
        assert torch.equal(gz.cpu(), z)
        assert rel_err(gv, v) <= TOL_STATE
        for a, b in zip(gnew[:6], new_state[:6]):
            assert rel_err(a.float(), b.float()) <= TOL_STATE
        state = new_state


def test_step_backward_matches_autograd():
    cfg, dicts, orc, cell = _cells("small", dampening_factor=0.5, pseudo_width=0.5)
    import ctypes as C
    from v1_glif_model_b200 import _lib
    n, d, r = cfg.n_neurons, orc.max_delay, orc._n_syn_basis
    g = torch.Generator().manual_seed(8)
    b = 2
    z_buf = (torch.rand(b, n * d, generator=g) < 0.1).float()
    leaves = [t.requires_grad_(True) for t in (torch.randn(b, n, generator=g) * 0.5 + 0.6,
                                               torch.randn(b, n * 2, generator=g),
                                               torch.randn(b, n * r, generator=g),
                                               torch.randn(b, n * r, generator=g),
                                               torch.randn(b, n * r, generator=g))]
    v, asc, psc_rise, psc, rec_inputs = leaves
    rr = torch.randint(0, 2, (b, n), generator=g)
    nv, nr, nasc, npr, npsc = orc._dense_update_impl(b, z_buf[:, :n], v, rr, asc, psc_rise, psc, rec_inputs)
    from oracle.cell_torch import SpikeFunction
    z = SpikeFunction.apply(nv - 1.0, 0.5, 0.5, None)
    z = torch.where(nr > 0, torch.zeros_like(z), z)
    cot = [torch.randn_like(t, ) for t in (nv, nasc, npr, npsc, z, nv)]
    loss = (nv * cot[0]).sum() + (nasc * cot[1]).sum() + (npr * cot[2]).sum() + (npsc * cot[3]).sum() + \
        (z * cot[4]).sum() + (nv * cot[5]).sum()
    want = torch.autograd.grad(loss, leaves)
    dev = lambda t: t.detach().contiguous().cuda()
    g_out = _lib.V1GState(None, dev(cot[0]).data_ptr(), None, None, None, None)
    keep = [dev(cot[0]), dev(cot[1]), dev(cot[2]), dev(cot[3]), dev(cot[4]), dev(cot[5]), dev(nv),
            nr.to(torch.int8).cuda()]
    g_out = _lib.V1GState(None, keep[0].data_ptr(), None, keep[1].data_ptr(), keep[2].data_ptr(), keep[3].data_ptr())
    outs = [torch.empty(b, n).cuda(), torch.empty(b, 2 * n).cuda(), torch.empty(b, n * r).cuda(),
            torch.empty(b, n * r).cuda(), torch.empty(b, n * r).cuda()]
    g_in = _lib.V1GState(None, outs[0].data_ptr(), None, outs[1].data_ptr(), outs[2].data_ptr(), outs[3].data_ptr())
    rc = cell._lib.v1g_step_bwd(cell._libh, b, C.byref(g_out), keep[4].data_ptr(), keep[5].data_ptr(),
                                keep[6].data_ptr(), keep[7].data_ptr(), C.byref(g_in), outs[4].data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    for got, w in zip(outs, want):
        assert rel_err(got, w) <= TOL_GRAD


def test_invalid_connectivity_raises_value_error():
    from v1_glif_model_b200.models import V1Column
    cfg, dicts, orc = make_case("tiny")
    net, lgn, bkg = dicts
    bad = dict(lgn)
    bad["indices"] = lgn["indices"].copy()
    bad["indices"][0, 1] = cfg.n_lgn + 3
    with pytest.raises(ValueError, match="out of bounds"):
        V1Column(net, bad, bkg)


def test_expadam_kernel_matches_oracle():
    from oracle.expadam import expadam_step
    from v1_glif_model_b200.training import ExponentiatedAdam
    torch.manual_seed(2)
    w = torch.randn(10001)
    w[:7] = 0.0
    pos = w >= 0
    wg = w.clone().cuda()
    opt = ExponentiatedAdam([wg], [pos.cuda()], learning_rate=5e-3)
    m, v = torch.zeros_like(w), torch.zeros_like(w)
    for step in range(1, 4):
        g = torch.randn(10001)
        w, m, v = expadam_step(w, g, m, v, pos, 5e-3, 0.9, 0.999, 1e-11, step)
        opt.apply_gradients([g.cuda()])
    assert rel_err(wg, w) <= 1e-6
    assert rel_err(opt.m[0], m) <= 1e-6 and rel_err(opt.v[0], v) <= 1e-6
