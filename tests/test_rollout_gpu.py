"""GPU parity of the fused rollouts (forward and BPTT) against the CPU oracle and the fixtures."""
import os

import numpy as np
import pytest
import torch

from util import TOL_GRAD, TOL_STATE, assert_grad_close, first_spike_divergence, make_case, make_inputs, rel_err
from v1_glif_model_b200 import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KW = dict(dampening_factor=0.5, pseudo_width=0.5, recurrent_dampening_factor=0.5,
          voltage_gradient_dampening=0.5)
LOSS = dict(rate_cost=10.0, voltage_cost=1e-1, sync_cost=0.5, fano_target=1.0, sync_bin=10)


def _cells(name, options=(), **kw):
    from v1_glif_model_b200.models import V1Column
    dense = kw.pop("dense_basis", False)
    nrec = kw.pop("n_receptors", None)
    dtype = kw.pop("dtype", torch.float32)
    cfg, dicts, orc = make_case(name, dense_basis=dense, n_receptors=nrec, dtype=dtype, **kw)
    cell = V1Column(*dicts, **kw)
    for k, v in options:
        cell.set_option(k, v)
    return cfg, dicts, orc, cell


def _compare_rollout(cfg, orc, cell, x, c):
    with torch.no_grad():
        zo, vo, so = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    state = cell.zero_state(x.shape[0])
    z, v = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), state=state)
    cell.synchronize()
    # spikes are compared exactly; a divergence is accepted only as a proven threshold tie (the
    # oracle's voltage within a few float steps of 1 at the first differing entries), in which case
    # everything before that step is compared and the rest is not comparable
    t_tie = first_spike_divergence(z, zo, vo)
    if t_tie is not None:
        assert t_tie >= 1 and rel_err(v[:, :t_tie], vo[:, :t_tie]) <= TOL_STATE
        pytest.skip(f"threshold tie at step {t_tie}: compared up to it")
    assert rel_err(v, vo) <= TOL_STATE
    for got, want in zip(state[:6], so[:6]):
        assert rel_err(got.float(), want.float()) <= TOL_STATE
    assert torch.equal(state[0].cpu(), so[0])          # z_buf
    assert torch.equal(state[2].cpu().long(), so[2])   # refractory counters
    return z, v


@pytest.mark.parametrize("name,options,kw", [
    ("tiny", (), {}),
    ("small", (), {}),
    ("small", (("rollout_chunk", 32),), {}),
    ("small", (("rollout_chunk", 64), ("force_smem_kernel", 1)), {}),
    ("small", (("rollout_chunk", 96), ("state_in_global", 1)), {}),
    ("small", (("no_meta", 1),), {}),                      # plain post / sid / w arrays instead of packed records
    ("small", (), dict(hard_reset=True)),
    ("small", (), dict(dense_basis=True)),
    ("small", (("force_smem_kernel", 1),), dict(dense_basis=True, n_receptors=4)),
    ("small", (), dict(n_receptors=4)),
    ("small", (("force_smem_kernel", 1),), dict(n_receptors=3)),
])
def test_forward_rollout_matches_oracle(name, options, kw):
    cfg, dicts, orc, cell = _cells(name, options, **kw)
    x, c = make_inputs(cfg)
    _compare_rollout(cfg, orc, cell, x, c)
    cnt = cell.counters()
    assert cnt["spikes"] > 0 and cnt["rec_rows"] == cnt["spikes"] * orc.max_delay


def test_forward_rollout_c1_free_running():
    """Configuration 1 (5,000 neurons, batch 1): free-running spike trains agree with the oracle."""
    cfg, dicts, orc, cell = _cells("C1")
    x, c = make_inputs(cfg, seq_len=60)
    _compare_rollout(cfg, orc, cell, x, c)


def test_edge_cases_empty_input_and_single_step():
    cfg, dicts, orc, cell = _cells("tiny")
    x, c = make_inputs(cfg, seq_len=7)
    _compare_rollout(cfg, orc, cell, np.zeros_like(x), np.zeros_like(c))   # no events at all
    for t_len in (1, 2, 3):
        _compare_rollout(cfg, orc, cell, x[:, :t_len], c[:, :t_len])
    _compare_rollout(cfg, orc, cell, np.ones_like(x), c)                   # every LGN unit fires


@pytest.mark.parametrize("options", [(), (("force_smem_kernel", 1),)])
def test_chunked_rollout_carries_state(options):
    """Two chunks with the state carried over equal one rollout (osi_dsi_estimator.py:252-294)."""
    cfg, dicts, orc, cell = _cells("small", options)
    x, c = make_inputs(cfg, seq_len=50)
    xg, cg = torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda()
    s_one = cell.zero_state(cfg.batch)
    z1, v1 = cell.rollout(xg, cg, state=s_one)
    s_two = cell.zero_state(cfg.batch)
    za, va = cell.rollout(xg[:, :23].contiguous(), cg[:, :23].contiguous(), state=s_two)
    zb, vb = cell.rollout(xg[:, 23:].contiguous(), cg[:, 23:].contiguous(), state=s_two)
    cell.synchronize()
    assert torch.equal(torch.cat([za, zb], 1), z1)
    assert rel_err(torch.cat([va, vb], 1), v1) <= TOL_STATE
    for a, b in zip(s_two[:6], s_one[:6]):
        assert rel_err(a.float(), b.float()) <= TOL_STATE


def test_rollout_through_host_buffers():
    cfg, dicts, orc, cell = _cells("small")
    x, c = make_inputs(cfg)
    z_dev, v_dev = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda())
    z_host, v_host = cell.rollout_host(x, c, want_z=True, want_v=True)
    assert np.array_equal(z_host, z_dev.cpu().numpy())
    assert rel_err(v_host, v_dev) <= TOL_STATE


@pytest.mark.parametrize("pinned", [False, True])
def test_pipelined_rollout_through_host_buffers(pinned):
    """The chunked, copy-overlapped host entry point returns the spikes of the plain device rollout,
    as bytes and as one bit per neuron-step, for ragged chunk lengths and pageable or pinned inputs."""
    cfg, dicts, orc, cell = _cells("small")
    x, c = make_inputs(cfg, seq_len=60)
    z_dev, _ = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda())
    want = z_dev.cpu()
    xh, ch = (torch.from_numpy(x).pin_memory(), torch.from_numpy(c).pin_memory()) if pinned else (x, c)
    for chunk in (0, 17, 60, 1):
        got = cell.rollout_host_pipelined(xh, ch, z_format="uint8", chunk_steps=chunk)
        assert torch.equal(got, want), chunk
        bits = cell.rollout_host_pipelined(xh, ch, z_format="bits", chunk_steps=chunk).numpy().view(np.uint32)
        n = cfg.n_neurons
        unpacked = ((bits[..., :, None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(*bits.shape[:2], -1)[..., :n]
        assert np.array_equal(unpacked.astype(np.uint8), want.numpy()), chunk
        assert not np.any(((bits[..., -1] >> np.uint32(n % 32)) != 0) & (n % 32 != 0))   # padding bits are zero


def test_golden_fixture_forward_and_gradients():
    g = np.load(os.path.join(ROOT, "tests", "golden", "tiny_rollout.npz"))
    cfg, dicts, orc, cell = _cells("tiny", **KW)
    z, v = cell.rollout(torch.from_numpy(g["x"]).cuda(), torch.from_numpy(g["bkg_counts"]).cuda(),
                        save_for_bwd=True)
    assert np.array_equal(z.cpu().numpy(), g["z"])
    assert rel_err(v, g["v"]) <= TOL_STATE
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)).cuda() / 1000.0
    vlo = torch.from_numpy((-20.0 / cell.voltage_scale).astype(np.float32)).cuda()
    dwr, dwl, dwb, losses = cell.backward(dict(LOSS, rate_target=tgt, v_lo=vlo))
    cell.synchronize()
    assert abs(float(losses[0]) - float(g["loss"])) <= 1e-5 * abs(float(g["loss"]))
    assert rel_err(dwr, g["dw_rec"]) <= TOL_GRAD
    assert rel_err(dwl, g["dw_lgn"]) <= TOL_GRAD
    assert rel_err(dwb, g["dw_bkg"]) <= TOL_GRAD


def _oracle_grads(orc, cfg, x, c, vscale, dtype, g_z=None, g_v=None, loss=LOSS):
    z, v, _ = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    from oracle import losses as OL
    tgt = (torch.from_numpy(synth.make_rate_targets(cfg)).double() / 1000.0).to(dtype)
    vlo = torch.from_numpy(-20.0 / vscale).to(dtype)
    total = OL.rate_loss(z, tgt, loss["rate_cost"]) + OL.voltage_loss(v, vlo, loss["voltage_cost"]) + \
        OL.sync_loss(z, loss["sync_bin"], loss["sync_cost"], loss["fano_target"])
    if g_z is not None:
        total = total + (z * g_z).sum() + (v * g_v).sum()
    total.backward()
    return z.detach(), total.item(), [orc.recurrent_weight_values.grad, orc.input_weight_values.grad,
                                     orc.bkg_input_weights.grad]


@pytest.mark.parametrize("name,options,kw", [
    ("tiny", (), {}),
    ("small", (), {}),
    ("small", (("rollout_chunk", 32),), {}),
    ("small", (("rollout_chunk", 64), ("state_in_global", 1)), {}),
    ("small", (("no_meta", 1),), {}),                      # gather over plain arrays instead of packed records
    ("small", (), dict(dense_basis=True)),
    ("small", (), dict(n_receptors=4)),
    ("small", (), dict(pseudo_gauss=True, gauss_std=0.3)),
    ("small", (), dict(hard_reset=True)),
    ("tiny", (("pair_rows", 1),), {}),                     # two steps per 32-byte row in the backward ring
    ("small", (("pair_rows", 1),), {}),
    ("small", (("pair_rows", 1), ("rollout_chunk", 32)), dict(hard_reset=True)),
    ("small", (("pair_rows", 1),), dict(n_receptors=4)),
])
def test_bptt_gradients_match_oracle_autograd(name, options, kw):
    kw = dict(KW, **kw)
    cfg, dicts, orc, cell = _cells(name, options, **kw)
    x, c = make_inputs(cfg)
    zo, lo, go = _oracle_grads(orc, cfg, x, c, cell.voltage_scale, torch.float32)
    z, _ = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), save_for_bwd=True)
    assert torch.equal(z.cpu().float(), zo)
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)).cuda() / 1000.0
    vlo = torch.from_numpy((-20.0 / cell.voltage_scale).astype(np.float32)).cuda()
    grads = cell.backward(dict(LOSS, rate_target=tgt, v_lo=vlo))
    cell.synchronize()
    assert abs(float(grads[3][0]) - lo) <= 1e-4 * abs(lo)
    for got, want in zip(grads[:3], go):
        assert rel_err(got, want) <= TOL_GRAD


@pytest.mark.parametrize("pre,post", [(0, 0), (5, 3)])
def test_bptt_with_rate_distribution_target(pre, post):
    """The reference's firing-rate target (sorted rates per population against sorted target samples,
    quantile-Huber penalty, ``loss_functions.py:626-681, 873-889``) evaluated on the device from the
    saved spikes: loss value and weight gradients against autograd through the oracle's form of it,
    which is pinned to the reference's code by tests/golden/reference_rate_loss.npz."""
    from oracle import losses as OL
    cfg, dicts, orc, cell = _cells("small", **KW)
    x, c = make_inputs(cfg)
    groups = synth.make_rate_groups(cfg, dicts[0], 0)
    cost = 50.0
    z, v, _ = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    vlo = torch.from_numpy(-20.0 / cell.voltage_scale).float()
    total = OL.rate_distribution_loss(z, groups, cost, kappa=0.002, pre_delay=pre, post_delay=post) + \
        OL.voltage_loss(v, vlo, LOSS["voltage_cost"])
    total.backward()
    want = [orc.recurrent_weight_values.grad, orc.input_weight_values.grad, orc.bkg_input_weights.grad]
    zc, _ = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), save_for_bwd=True)
    assert torch.equal(zc.cpu().float(), z.detach())
    grads = cell.backward(dict(rate_cost=cost, rate_groups=groups, rate_kappa=0.002, rate_pre_delay=pre,
                               rate_post_delay=post, voltage_cost=LOSS["voltage_cost"], v_lo=vlo.cuda()))
    cell.synchronize()
    assert abs(float(grads[3][0]) - total.item()) <= 1e-4 * abs(total.item())
    for got, w in zip(grads[:3], want):
        assert rel_err(got, w) <= TOL_GRAD


@pytest.mark.parametrize("t_start,t_end", [(0, 0), (6, 54)])
def test_bptt_with_synchrony_samples_target(t_start, t_end):
    """The reference's synchrony target (population Fano factors of sampled groups of excitatory
    neurons over all bin sizes below half the window, ``loss_functions.py:964-1044``) on the
    device: loss value and weight gradients against autograd through the oracle's form, which is
    pinned to the reference's ``pop_fano_tf`` by tests/golden/reference_sync_loss.npz.  The 600-neuron
    net has fewer excitatory neurons than the samples ask for, so some neurons sit in two samples."""
    from oracle import losses as OL
    cfg, dicts, orc, cell = _cells("small", **KW)
    x, c = make_inputs(cfg)
    samples, bins, targets = synth.make_sync_samples(cfg, dicts[0], cfg.batch, n_samples=12, seed=1)
    cost = 0.05
    z, v, _ = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    vlo = torch.from_numpy(-20.0 / cell.voltage_scale).float()
    total = OL.synchronization_loss(z, samples, bins, targets, cost, t_start=t_start, t_end=t_end or None) + \
        OL.voltage_loss(v, vlo, LOSS["voltage_cost"])
    total.backward()
    want = [orc.recurrent_weight_values.grad, orc.input_weight_values.grad, orc.bkg_input_weights.grad]
    zc, _ = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), save_for_bwd=True)
    assert torch.equal(zc.cpu().float(), z.detach())
    grads = cell.backward(dict(sync_cost=cost, sync_samples=samples, sync_bin_sizes=bins, sync_bin_targets=targets,
                               sync_t_start=t_start, sync_t_end=t_end, voltage_cost=LOSS["voltage_cost"],
                               v_lo=vlo.cuda()))
    cell.synchronize()
    assert abs(float(grads[3][0]) - total.item()) <= 1e-4 * abs(total.item())
    for got, w in zip(grads[:3], want):
        assert rel_err(got, w) <= TOL_GRAD


def test_synchrony_samples_are_taken_from_every_call():
    """The reference redraws the synchrony samples in every call; two calls with freshly built lists
    (which CPython may well give the same address) must each use their own list."""
    cfg, dicts, orc, cell = _cells("small", **KW)
    x, c = make_inputs(cfg)
    cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), save_for_bwd=True)
    losses = []
    for seed in (1, 2, 1):
        samples, bins, targets = synth.make_sync_samples(cfg, dicts[0], cfg.batch, n_samples=12, seed=seed)
        spec = dict(sync_cost=0.05, sync_samples=list(samples), sync_bin_sizes=bins, sync_bin_targets=targets)
        losses.append(float(cell.backward(spec)[3][0]))
        del samples, spec
    cell.synchronize()
    # equal lists give equal losses up to the order of the atomic sums; different lists do not
    assert abs(losses[0] - losses[1]) > 1e-3 * abs(losses[0]) and abs(losses[0] - losses[2]) <= 1e-5 * abs(losses[0])


@pytest.mark.parametrize("batch", [1, 4, 6, 8])
def test_rollout_and_bptt_at_every_batch_width(batch):
    """Batch 1..4 uses 16-byte fp32 rows in the backward ring, 6..8 32-byte rows, 7 and 8 the general
    forward kernel; spikes must be exact and gradients inside the bar at each width, and a second
    backward pass over the same saved rollout must give the same recurrent gradient."""
    cfg, dicts, orc, cell = _cells("small", **KW)
    x, c = make_inputs(cfg, batch=batch, seq_len=30)
    zo, lo, go = _oracle_grads(orc, cfg, x, c, cell.voltage_scale, torch.float32)
    z, _ = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), save_for_bwd=True)
    assert torch.equal(z.cpu().float(), zo)
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)).cuda() / 1000.0
    vlo = torch.from_numpy((-20.0 / cell.voltage_scale).astype(np.float32)).cuda()
    grads = cell.backward(dict(LOSS, rate_target=tgt, v_lo=vlo))
    again = cell.backward(dict(LOSS, rate_target=tgt, v_lo=vlo))
    cell.synchronize()
    for got, want in zip(grads[:3], go):
        assert rel_err(got, want) <= TOL_GRAD
    assert torch.equal(grads[0], again[0])     # recurrent gradient: no atomics, same order


@pytest.mark.parametrize("mode", ["range", "threshold"])
def test_bptt_with_reference_voltage_penalties(mode):
    """The two penalties of the reference's ``VoltageRegularization`` (``loss_functions.py:1087-1119``):
    "range" = relu(|v - .5| - .5)^2 (lower bound 0, no ``v_lo``) and "threshold" = (v - 1)^2."""
    cfg, dicts, orc, cell = _cells("small", **KW)
    x, c = make_inputs(cfg)
    z, v, _ = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    cost = 1e-2
    if mode == "range":
        total = cost * torch.relu((v - 0.5).abs() - 0.5).pow(2).mean()
    else:
        total = cost * (v - 1.0).pow(2).mean()
    total.backward()
    want = [orc.recurrent_weight_values.grad, orc.input_weight_values.grad, orc.bkg_input_weights.grad]
    cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), save_for_bwd=True)
    grads = cell.backward(dict(voltage_cost=cost, voltage_mode=mode))
    cell.synchronize()
    assert abs(float(grads[3][0]) - total.item()) <= 1e-4 * abs(total.item())
    for got, w in zip(grads[:3], want):
        assert rel_err(got, w) <= TOL_GRAD


@pytest.mark.parametrize("with_normalizer", [False, True])
def test_bptt_with_osi_dsi_target(with_normalizer):
    """The reference's population OSI/DSI target (``OrientationSelectivityLoss``, crowd method,
    ``loss_functions.py:1340-1440``) on the device: loss value and weight gradients against autograd
    through the oracle's form, which is pinned to the reference's code by
    tests/golden/reference_osi_loss.npz."""
    from oracle import losses as OL
    cfg, dicts, orc, cell = _cells("small", **KW)
    x, c = make_inputs(cfg)
    rng = np.random.Generator(np.random.PCG64(5))
    n = cfg.n_neurons
    type_ids = np.asarray(dicts[0]["node_type_ids"], dtype=np.int32)
    n_types = int(type_ids.max()) + 1
    tuning = rng.uniform(0.0, 360.0, n).astype(np.float32)
    angle = rng.uniform(0.0, 360.0, cfg.batch).astype(np.float32)
    osi_t, dsi_t = rng.uniform(0.2, 0.6, n_types).astype(np.float32), rng.uniform(0.05, 0.3, n_types).astype(np.float32)
    counts = np.bincount(type_ids, minlength=n_types).astype(np.float32)
    norm = rng.lognormal(np.log(0.02), 0.6, n).astype(np.float32) if with_normalizer else None
    cost, pre, post = 5.0, 4, 6
    z, v, _ = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    vlo = torch.from_numpy(-20.0 / cell.voltage_scale).float()
    total = OL.orientation_selectivity_loss(z, angle, tuning, type_ids, osi_t, dsi_t, counts, cost, pre_delay=pre,
                                            post_delay=post, normalizer=norm) + \
        OL.voltage_loss(v, vlo, LOSS["voltage_cost"])
    total.backward()
    want = [orc.recurrent_weight_values.grad, orc.input_weight_values.grad, orc.bkg_input_weights.grad]
    zc, _ = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), save_for_bwd=True)
    assert torch.equal(zc.cpu().float(), z.detach())
    grads = cell.backward(dict(osi_cost=cost, osi_angle=angle, osi_tuning_angle=tuning, osi_type_ids=type_ids,
                               osi_targets=osi_t, dsi_targets=dsi_t, osi_type_counts=counts, osi_normalizer=norm,
                               osi_pre_delay=pre, osi_post_delay=post, voltage_cost=LOSS["voltage_cost"],
                               v_lo=vlo.cuda()))
    cell.synchronize()
    assert abs(float(grads[3][0]) - total.item()) <= 1e-4 * abs(total.item())
    for got, w in zip(grads[:3], want):
        assert rel_err(got, w) <= TOL_GRAD


@pytest.mark.parametrize("options", [(), (("no_q_pack", 1),), (("rollout_chunk", 64),), (("no_meta", 1),),
                                     (("pair_rows", 1),), (("pair_rows", 1), ("rollout_chunk", 64))])
def test_bptt_batch_of_five(options):
    """Batch 5 stores the backward Q rows as five 24-bit floats per 16-byte row (7.6e-6 relative
    rounding); the gradients must stay inside the 1e-4 bar, as they do with fp32 rows."""
    cfg, dicts, orc, cell = _cells("small", options, **KW)
    x, c = make_inputs(cfg, batch=5, seq_len=40)
    zo, lo, go = _oracle_grads(orc, cfg, x, c, cell.voltage_scale, torch.float32)
    z, _ = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), save_for_bwd=True)
    assert torch.equal(z.cpu().float(), zo)
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)).cuda() / 1000.0
    vlo = torch.from_numpy((-20.0 / cell.voltage_scale).astype(np.float32)).cuda()
    grads = cell.backward(dict(LOSS, rate_target=tgt, v_lo=vlo))
    cell.synchronize()
    for got, want in zip(grads[:3], go):
        assert rel_err(got, want) <= TOL_GRAD


def test_balanced_slices_do_not_change_the_results():
    """``v1g_balance_slices`` re-cuts the blocks' slices of the one-neuron-per-thread forward kernel by
    scatter work: with costs from the last saved rollout, with heavily skewed explicit costs (slices from
    a handful of neurons to the 512-neuron cap) and after a reset, spikes stay those of the oracle and
    the backward pass over the saved rollout gives the same gradients."""
    cfg, dicts, orc, cell = _cells("small", (("rollout_chunk", 32),), **KW)     # 19 blocks of 32 neurons
    x, c = make_inputs(cfg)
    zo, lo, go = _oracle_grads(orc, cfg, x, c, cell.voltage_scale, torch.float32)
    xd, cd = torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda()
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)).cuda() / 1000.0
    vlo = torch.from_numpy((-20.0 / cell.voltage_scale).astype(np.float32)).cuda()
    with pytest.raises(ValueError):
        cell.balance_slices()                                  # nothing saved yet
    skew = np.ones(cfg.n_neurons, dtype=np.float32)
    skew[:40] = 500.0
    for step, cost in enumerate(("saved", skew, skew[::-1].copy())):
        z, _ = cell.rollout(xd, cd, save_for_bwd=True)
        assert torch.equal(z.cpu().float(), zo)
        grads = cell.backward(dict(LOSS, rate_target=tgt, v_lo=vlo))
        cell.synchronize()
        for got, want in zip(grads[:3], go):
            assert rel_err(got, want) <= TOL_GRAD
        cell.balance_slices(None if isinstance(cost, str) else cost)
    z, _ = cell.rollout(xd, cd)
    assert torch.equal(z.cpu().float(), zo)
    with pytest.raises(ValueError):
        cell.balance_slices(-skew)
    cell.set_option("rollout_chunk", 64)                       # another slicing: the balanced cut is dropped
    z, _ = cell.rollout(xd, cd)
    assert torch.equal(z.cpu().float(), zo)


def test_forward_rollout_of_more_trials_than_one_launch_takes():
    """Ten trials (the reference's evaluation batch, ``osi_dsi_estimator.py:424``) run as groups of at most
    8: spikes equal the oracle's for every trial, the carried state is that of one wide rollout, counts
    drawn by the library follow the batch row, and a saved rollout of that width is refused."""
    cfg, dicts, orc, cell = _cells("small", **KW)
    x, c = make_inputs(cfg, batch=10, seq_len=30)
    zo, vo, so = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    xd, cd = torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda()
    state = cell.zero_state(10)
    z, v = cell.rollout(xd, cd, state=state)
    cell.synchronize()
    assert torch.equal(z.cpu().float(), zo.detach())
    assert rel_err(v, vo.detach()) <= TOL_STATE
    assert torch.equal(state[0].cpu(), so[0].detach()) and rel_err(state[5], so[5].detach()) <= TOL_STATE
    assert state[6].cpu().tolist() == [30] * 10
    # continuing from the carried state equals one rollout of both halves
    z2, _ = cell.rollout(xd, cd, state=state)
    x2, c2 = np.concatenate([x, x], 1), np.concatenate([c, c], 1)
    zo2, _, _ = orc.rollout(torch.from_numpy(x2), torch.from_numpy(c2).long())
    assert torch.equal(z2.cpu().float(), zo2.detach()[:, 30:])
    # counts drawn inside: the draw of a trial depends on its batch row, not on its place in a group
    cell.set_noise_seed(5)
    drawn = cell.sample_bkg_counts(10, 30)
    za, _ = cell.rollout(xd, drawn)
    zb, _ = cell.rollout(xd)
    cell.synchronize()
    assert torch.equal(za, zb) and not torch.equal(drawn[0], drawn[8])
    with pytest.raises(ValueError):
        cell.rollout(xd, cd, save_for_bwd=True)


@pytest.mark.parametrize("batch,nrec,options", [
    (3, 4, ()),                      # lane quads over fp32 16-byte rows
    (5, 4, ()),                      # lane quads over 24-bit rows
    (5, 4, (("no_q_pack", 1),)),     # 32-byte rows: the gather over plain arrays
    (5, 4, (("no_meta", 1),)),
    (8, 4, ()),
    (5, 5, ()),                      # five channels do not divide a warp: plain-array gather
    (5, 4, (("rollout_chunk", 64), ("state_in_global", 1))),
])
def test_bptt_with_more_synapse_types_than_ring_channels(batch, nrec, options):
    """More than 8 synapse types (the reference's basis table has 121 rows over 4 channels): the
    backward ring holds the raw per-channel adjoints and a synapse contracts them with its basis row.
    With 4 channels in 16-byte rows a quad of lanes shares a synapse (one lane per channel); every
    other shape walks plain arrays.  Long rows (several passes), rows that spike (weight gradient over
    the quad) and rows shorter than a pass are all in the 600-neuron net."""
    kw = dict(KW, dense_basis=True, n_receptors=nrec)
    cfg, dicts, orc, cell = _cells("small", options, **kw)
    assert dicts[0]["synaptic_basis_weights"].shape[0] > 8
    x, c = make_inputs(cfg, batch=batch, seq_len=40)
    zo, lo, go = _oracle_grads(orc, cfg, x, c, cell.voltage_scale, torch.float32)
    z, _ = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), save_for_bwd=True)
    assert torch.equal(z.cpu().float(), zo)
    assert int(z.sum()) > 100
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)).cuda() / 1000.0
    vlo = torch.from_numpy((-20.0 / cell.voltage_scale).astype(np.float32)).cuda()
    grads = cell.backward(dict(LOSS, rate_target=tgt, v_lo=vlo))
    cell.synchronize()
    assert abs(float(grads[3][0]) - lo) <= 1e-4 * abs(lo)
    for name, got, want in zip(("dW_rec", "dW_lgn", "dW_bkg"), grads[:3], go):
        assert_grad_close(got, want, name)


def test_bptt_from_carried_state_counts_pending_spikes():
    """Training from a carried state (the reference starts each step from its gray-screen state,
    multi_training.py:812-831): the state is a constant, but spikes still travelling in its z_buf
    reach their targets inside the rollout and belong in the recurrent weight gradient."""
    cfg, dicts, orc, cell = _cells("small", **KW)
    x, c = make_inputs(cfg, seq_len=50)
    xo, co = torch.from_numpy(x), torch.from_numpy(c).long()
    with torch.no_grad():
        _, _, mid = orc.rollout(xo[:, :20], co[:, :20])
    assert float(mid[0].sum()) > 0                                  # spikes are pending
    z2, v2, _ = orc.rollout(xo[:, 20:], co[:, 20:], state=tuple(t.detach() for t in mid))
    g = torch.Generator().manual_seed(5)
    g_z = torch.randn(z2.shape, generator=g) * 1e-2
    g_v = torch.randn(v2.shape, generator=g) * 1e-3
    ((z2 * g_z).sum() + (v2 * g_v).sum()).backward()
    want = [orc.recurrent_weight_values.grad, orc.input_weight_values.grad, orc.bkg_input_weights.grad]
    xg, cg = torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda()
    state = cell.zero_state(cfg.batch)
    cell.rollout(xg[:, :20].contiguous(), cg[:, :20].contiguous(), state=state, return_v=False)
    z, _ = cell.rollout(xg[:, 20:].contiguous(), cg[:, 20:].contiguous(), state=state, save_for_bwd=True)
    assert torch.equal(z.cpu().float(), z2.detach())
    grads = cell.backward(None, g_z=g_z.cuda(), g_v=g_v.cuda())
    cell.synchronize()
    for got, w in zip(grads[:3], want):
        assert rel_err(got, w) <= TOL_GRAD


def test_bptt_with_explicit_output_gradients():
    """dL/dz and dL/dv supplied as tensors (the general tape.gradient form), no in-kernel loss."""
    cfg, dicts, orc, cell = _cells("small", **KW)
    x, c = make_inputs(cfg)
    g = torch.Generator().manual_seed(11)
    shape = (cfg.batch, cfg.seq_len, cfg.n_neurons)
    g_z, g_v = torch.randn(shape, generator=g) * 1e-2, torch.randn(shape, generator=g) * 1e-3
    zero = dict(rate_cost=0.0, voltage_cost=0.0, sync_cost=0.0, fano_target=1.0, sync_bin=10)
    zo, lo, go = _oracle_grads(orc, cfg, x, c, cell.voltage_scale, torch.float32, g_z, g_v, loss=zero)
    cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), return_z=False, return_v=False,
                 save_for_bwd=True)
    grads = cell.backward(None, g_z=g_z.cuda(), g_v=g_v.cuda())
    cell.synchronize()
    for got, want in zip(grads[:3], go):
        assert rel_err(got, want) <= TOL_GRAD


def test_backward_without_saved_forward_is_an_error():
    from v1_glif_model_b200._lib import V1GError
    cfg, dicts, orc, cell = _cells("tiny")
    with pytest.raises(V1GError, match="save_for_bwd"):
        cell.backward(None)


def test_bounded_wait_reports_timeout_and_handle_survives():
    """A device-side wait that can never be satisfied gives up after its poll limit, the host sees
    V1G_ETIMEOUT, and the same handle then runs a rollout normally (no trap, no hang)."""
    import ctypes as C
    from v1_glif_model_b200._lib import ETIMEOUT, V1GError
    cfg, dicts, orc, cell = _cells("tiny")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert cell._lib.v1g_selftest_bounded_wait(cell._libh, 2000, stream) == 0
    with pytest.raises(V1GError) as err:
        cell.synchronize()
    assert err.value.code == ETIMEOUT
    cell.synchronize()                      # status was cleared
    x, c = make_inputs(cfg)
    _compare_rollout(cfg, orc, cell, x, c)  # the handle still works


def test_training_step_updates_weights_with_sign_constraint():
    from v1_glif_model_b200.training import Trainer
    cfg, dicts, orc, cell = _cells("small", **KW)
    x, c = make_inputs(cfg)
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)).cuda() / 1000.0
    vlo = torch.from_numpy((-20.0 / cell.voltage_scale).astype(np.float32)).cuda()
    tr = Trainer(cell, dict(LOSS, rate_target=tgt, v_lo=vlo), learning_rate=1e-2)
    w0 = cell.recurrent_weight_values.clone()
    l0 = tr.step(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda())
    cell.synchronize()
    w1 = tr.weights()[0]
    assert not torch.equal(w0, w1)
    assert torch.all((w1 >= 0) == cell.recurrent_weight_positive | (w1 == 0))
    assert torch.isfinite(l0).all()


def test_internal_order_training_equals_reference_order_training():
    """Two optimiser steps in the kernels' own synapse order give the weights that the same steps
    give through the caller's order (permute -> Exp-Adam -> permute back)."""
    from v1_glif_model_b200.training import Trainer
    results = []
    for order in ("reference", "internal"):
        cfg, dicts, orc, cell = _cells("small", **KW)
        x, c = make_inputs(cfg)
        tgt = torch.from_numpy(synth.make_rate_targets(cfg)).cuda() / 1000.0
        vlo = torch.from_numpy((-20.0 / cell.voltage_scale).astype(np.float32)).cuda()
        tr = Trainer(cell, dict(LOSS, rate_target=tgt, v_lo=vlo), learning_rate=5e-3,
                     train_input=True, train_noise=True, order=order)
        for _ in range(2):
            losses = tr.step(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda())
        cell.synchronize()
        results.append([w.clone() for w in tr.weights()] + [losses.clone()])
    for a, b in zip(results[0][:3], results[1][:3]):
        assert rel_err(b, a) <= 1e-5
    assert rel_err(results[1][3], results[0][3]) <= 1e-5


def test_training_with_weight_regularizers_in_both_orders():
    """Mean-stiff and EMD regularisers added to the reduced gradient: the step in the library's own
    synapse order gives the weights of the step in the caller's order."""
    from v1_glif_model_b200.training import Trainer, WeightRegularizer
    results = []
    for order in ("reference", "internal"):
        cfg, dicts, orc, cell = _cells("small", **KW)
        x, c = make_inputs(cfg)
        rng = np.random.Generator(np.random.PCG64(8))
        edge_types = rng.integers(0, 6, cell.recurrent_weight_values.numel())
        # the "initial" weights differ from the current ones (as after some training): at the very first
        # step of the reference's setting every deviation is exactly zero and its rounding noise alone
        # would set the sign of the sign-normalised Exp-Adam step of synapses without any other gradient
        w0 = cell.recurrent_weight_values.cpu().numpy() * rng.lognormal(0.0, 0.3, edge_types.size).astype(np.float32)
        regs = [WeightRegularizer(cell, "mean_stiff", edge_types, w0, 5.0, relative=True, order=order),
                WeightRegularizer(cell, "emd", edge_types, w0, 2.0, order=order)]
        tgt = torch.from_numpy(synth.make_rate_targets(cfg)).cuda() / 1000.0
        tr = Trainer(cell, dict(LOSS, rate_target=tgt), learning_rate=5e-3, order=order, regularizers=regs)
        for _ in range(3):
            losses = tr.step(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda())
        cell.synchronize()
        results.append([w.clone() for w in tr.weights()] + [losses.clone()])
    assert rel_err(results[1][0], results[0][0]) <= 1e-4
    assert rel_err(results[1][3], results[0][3]) <= 1e-4
    assert float(results[0][3][0]) > 0


def test_full_size_column_properties():
    """66,634-neuron column, batch 5: size-independent checks (no oracle at this size)."""
    from v1_glif_model_b200.models import V1Column
    cfg = synth.CONFIGS["C3"]
    dicts = synth.make_network(cfg, 0)
    cell = V1Column(*dicts)
    t_len = 60
    x = torch.from_numpy(synth.make_lgn_spikes(cfg, cfg.batch, t_len)).cuda()
    c = torch.from_numpy(synth.make_bkg_counts(cfg, cfg.batch, t_len)).cuda()
    z, v = cell.rollout(x, c)
    cell.synchronize()
    cnt = cell.counters()
    # event counters are exact integer identities of the spike trains and the connectivity
    order, splits = cell.pre_ind_table(0)
    n, d = cfg.n_neurons, cell.max_delay
    outdeg = torch.from_numpy(np.diff(splits).reshape(d, n).sum(0)).cuda()
    assert cnt["spikes"] == int(z.sum())
    assert cnt["rec_events"] == int((z.sum((0, 1)).long() * outdeg).sum())
    _, lsplits = cell.pre_ind_table(1)
    ldeg = torch.from_numpy(np.diff(lsplits)).cuda()
    assert cnt["lgn_rows"] == int(x.sum())
    assert cnt["lgn_events"] == int((x.sum((0, 1)).long() * ldeg).sum())
    assert torch.isfinite(v).all()
    # the two forward kernels agree (summation order of the ring atomics is the only difference)
    cell.set_option("force_smem_kernel", 1)
    z2, v2 = cell.rollout(x, c)
    cell.synchronize()
    mismatch = float((z2 != z).float().mean())
    assert mismatch <= 1e-6
    if mismatch == 0.0:
        assert rel_err(v2, v) <= TOL_STATE


def test_stress_column_runs_through_general_kernels():
    """230,924 neurons, batch 4: slices exceed one neuron per thread and the shared-memory budget,
    so the general forward kernel and the global state slabs are exercised at full size."""
    from v1_glif_model_b200.models import V1Column
    cfg = synth.CONFIGS["C5"]
    cell = V1Column(*synth.make_network(cfg, 0), **KW)
    t_len = 24
    x = torch.from_numpy(synth.make_lgn_spikes(cfg, cfg.batch, t_len)).cuda()
    c = torch.from_numpy(synth.make_bkg_counts(cfg, cfg.batch, t_len)).cuda()
    z, v = cell.rollout(x, c, save_for_bwd=True)
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)).cuda() / 1000.0
    vlo = torch.from_numpy((-20.0 / cell.voltage_scale).astype(np.float32)).cuda()
    grads = cell.backward(dict(LOSS, rate_target=tgt, v_lo=vlo))
    cell.synchronize()
    cnt = cell.counters()
    _, splits = cell.pre_ind_table(0)
    outdeg = torch.from_numpy(np.diff(splits).reshape(cell.max_delay, cfg.n_neurons).sum(0)).cuda()
    assert cnt["spikes"] == int(z.sum()) and cnt["spikes"] > 0
    assert cnt["rec_events"] == int((z.sum((0, 1)).long() * outdeg).sum())
    assert torch.isfinite(v).all()
    for g in grads[:3]:
        assert torch.isfinite(g).all() and float(g.abs().max()) > 0
    # chunked rollout with carried state reproduces the spikes of the single rollout
    state = cell.zero_state(cfg.batch)
    za, _ = cell.rollout(x[:, :10].contiguous(), c[:, :10].contiguous(), state=state)
    zb, _ = cell.rollout(x[:, 10:].contiguous(), c[:, 10:].contiguous(), state=state)
    cell.synchronize()
    assert float((torch.cat([za, zb], 1) != z).float().mean()) <= 1e-6
