"""Property tests of the fused rollouts on random small nets (at most 64 neurons): every drawn net is
run forward and backward on the GPU and on the oracle, spikes must agree exactly and state and
gradients within the parity bars.  The draws cover what the fixed configurations do not: delay
ranges of 1, 3, 5 and 8 steps (the generic-delay instantiation of the backward kernel, the smallest
and the largest ring), a ``max_delay`` argument below the largest delay in the data (the clip of
``models.py:633-636``), LGN delays above every recurrent delay (they widen ``max_delay`` although
LGN synapses are not delayed, ``models.py:531-535, 715-718``), refractory periods of a single step
(which block nothing, ``models.py:1018, 1113-1114``) and of many, source neurons without any
outgoing synapse, a step at which every neuron fires, hard reset, 4 and 5 receptor channels and a
dense basis with negative entries over 7 or 12 synapse types (projected and raw backward ring).
"""
import dataclasses

import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, event, given, settings
from hypothesis import strategies as st

from util import TOL_GRAD, TOL_STATE, first_spike_divergence, rel_err, rel_l2
from v1_glif_model_b200 import synth

pytestmark = pytest.mark.gpu
KW = dict(dampening_factor=0.5, pseudo_width=0.5, recurrent_dampening_factor=0.4,
          voltage_gradient_dampening=0.3)
LOSS = dict(rate_cost=10.0, voltage_cost=1e-1, sync_cost=0.5, fano_target=1.0, sync_bin=4)


@st.composite
def nets(draw):
    return dict(
        n=draw(st.integers(8, 64)), in_degree=draw(st.integers(1, 9)),
        delays=draw(st.sampled_from([1, 3, 5, 8])), receptors=draw(st.sampled_from([4, 5])),
        batch=draw(st.integers(1, 6)), steps=draw(st.integers(3, 26)), seed=draw(st.integers(0, 10_000)),
        clip=draw(st.booleans()), lgn_widens=draw(st.booleans()),
        t_ref=draw(st.sampled_from(["one_step", "mixed", "long"])),
        mute=draw(st.booleans()), burst=draw(st.booleans()), hard_reset=draw(st.booleans()),
        dense_basis=draw(st.booleans()), n_lgn=draw(st.integers(1, 20)), n_bkg=draw(st.integers(1, 8)),
        pair_rows=draw(st.booleans()), many_types=draw(st.booleans()))


def _build(p):
    cfg = synth.SynthConfig("prop", p["n"], 3, 0.75, p["in_degree"], p["n_lgn"], min(3, p["n_lgn"]),
                            n_bkg=p["n_bkg"], bkg_in_degree=2, max_delay=p["delays"],
                            n_receptors=p["receptors"], batch=p["batch"], seq_len=p["steps"],
                            bkg_weight_pa=60.0, lgn_weight_pa=40.0)
    net, lgn, bkg = synth.make_network(cfg, p["seed"])
    rng = np.random.default_rng(p["seed"] + 17)
    kw = dict(KW, hard_reset=p["hard_reset"])
    if p["clip"] and p["delays"] > 1:
        kw["max_delay"] = max(1, p["delays"] - 2)      # delays above it are clipped to it
    if p["lgn_widens"] and p["delays"] < 8 and not p["clip"]:
        lgn["delays"] = np.full_like(lgn["delays"], float(p["delays"] + 1))   # widens the ring only
    if p["t_ref"] == "one_step":
        net["node_params"]["t_ref"][:] = 0.5
    elif p["t_ref"] == "long":
        net["node_params"]["t_ref"][:] = 6.5
    if p["mute"]:
        # neuron 0 loses all its outgoing synapses: its rows of the presynaptic table are empty
        syn = net["synapses"]
        keep = syn["indices"][:, 1] != 0
        for k in ("indices", "weights", "delays", "syn_ids"):
            syn[k] = syn[k][keep]
        net["n_edges"] = int(keep.sum())
    if p["dense_basis"]:
        # 7 types: the backward ring holds one projected row per type; 12 types: it holds the raw channels
        # and the gather contracts them (lanes sharing a synapse with 4 channels, plain arrays with 5)
        s_types = 12 if p["many_types"] else 7
        net["synaptic_basis_weights"] = rng.normal(0.3, 0.6, (s_types, cfg.n_receptors)).astype(np.float32)
        for d in (net["synapses"], lgn, bkg):
            d["syn_ids"] = rng.integers(0, s_types, d["syn_ids"].shape[0]).astype(np.uint8)
    x = synth.make_lgn_spikes(cfg, p["batch"], p["steps"], p["seed"])
    c = synth.make_bkg_counts(cfg, p["batch"], p["steps"], p["seed"])
    if p["burst"] and p["steps"] >= 6:
        # a volley that drives every neuron over the threshold at the same step
        bkg["weights"] = np.abs(bkg["weights"]) * 40.0
        if p["dense_basis"]:
            net["synaptic_basis_weights"] = np.abs(net["synaptic_basis_weights"])
        c[:, 2, :] = 3
    return cfg, (net, lgn, bkg), kw, x, c


@settings(max_examples=40, deadline=None, derandomize=True, database=None,
          suppress_health_check=list(HealthCheck))
@given(nets())
def test_random_small_nets_forward_and_backward(p):
    from oracle.cell_torch import OracleV1Column
    from oracle import losses as OL
    from v1_glif_model_b200.models import V1Column
    cfg, dicts, kw, x, c = _build(p)
    if dicts[0]["synapses"]["indices"].shape[0] == 0:
        return
    orc = OracleV1Column(*dicts, **kw)
    cell = V1Column(*dicts, **kw)
    cell.set_option("pair_rows", int(p["pair_rows"]))     # both layouts of the backward ring
    assert cell.max_delay == orc.max_delay
    # forward
    z, v, so = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    state = cell.zero_state(p["batch"])
    zc, vc = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), state=state, save_for_bwd=True)
    cell.synchronize()
    if first_spike_divergence(zc, z.detach(), v.detach()) is not None:
        return                                  # a proven threshold tie: nothing further is comparable
    assert rel_err(vc, v.detach()) <= TOL_STATE
    assert torch.equal(state[0].cpu(), so[0].detach()) and torch.equal(state[2].cpu().long(), so[2])
    for got, want in zip(state[3:6], so[3:6]):
        assert rel_err(got, want.detach()) <= TOL_STATE
    if float(z.detach().sum(dim=2).max()) == p["n"]:
        event("a step at which every neuron of a trial fires")
    # backward: in-kernel losses against autograd of the oracle
    vscale = cell.voltage_scale
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)) / 1000.0
    vlo = torch.from_numpy((-20.0 / vscale).astype(np.float32))
    total = OL.rate_loss(z, tgt, LOSS["rate_cost"]) + OL.voltage_loss(v, vlo, LOSS["voltage_cost"]) + \
        OL.sync_loss(z, LOSS["sync_bin"], LOSS["sync_cost"], LOSS["fano_target"])
    total.backward()
    want = [orc.recurrent_weight_values.grad, orc.input_weight_values.grad, orc.bkg_input_weights.grad]
    grads = cell.backward(dict(LOSS, rate_target=tgt.cuda(), v_lo=vlo.cuda()))
    cell.synchronize()
    assert abs(float(grads[3][0]) - total.item()) <= 1e-4 * abs(total.item()) + 1e-9
    for name, got, w in zip(("dW_rec", "dW_lgn", "dW_bkg"), grads[:3], want):
        assert rel_err(got, w) <= TOL_GRAD, (name, p)
        assert rel_l2(got, w) <= TOL_GRAD, (name, p)


def test_delay_clip_and_widening_reach_the_library():
    """The two ``max_delay`` rules, checked directly: an explicit ``max_delay`` below the data's clips
    the delays (``models.py:633-636``), and LGN delays above all recurrent ones widen the ring
    (``models.py:531-535``) while the LGN synapses themselves stay undelayed."""
    from v1_glif_model_b200.models import V1Column
    cfg = dataclasses.replace(synth.CONFIGS["tiny"], max_delay=5)
    net, lgn, bkg = synth.make_network(cfg, 4)
    cell = V1Column(net, lgn, bkg, max_delay=2)
    assert cell.max_delay == 2 and cell.recurrent_dense_shape == (cfg.n_neurons, 2 * cfg.n_neurons)
    assert int(cell.recurrent_indices[:, 1].max()) < 2 * cfg.n_neurons
    lgn2 = dict(lgn, delays=np.full_like(lgn["delays"], 7.0))
    cell2 = V1Column(net, lgn2, bkg)
    assert cell2.max_delay == 7
    _, splits = cell2.pre_ind_table(0)
    per_delay = np.diff(splits).reshape(7, cfg.n_neurons).sum(1)
    assert per_delay[5:].sum() == 0 and per_delay[:5].sum() == net["synapses"]["indices"].shape[0]
