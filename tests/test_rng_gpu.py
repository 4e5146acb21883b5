"""The device-side samplers: background Poisson counts keyed like the reference's
``tf.random.stateless_poisson`` call (``models.py:865-887``) and LGN spikes
``uniform < 1 - exp(-rate/1000)`` (``stim_dataset.py:182-193``).

TensorFlow's random streams cannot be reproduced, so these tests pin what can be: the Philox
generator against its published known-answer vectors (CPU), the CUDA kernels bit for bit against
the NumPy restatement in ``oracle/rng.py``, the keying (seed, replica, step), the distributions, and
that chunked rollouts and the backward pass see the draws of the single forward rollout.
"""
import numpy as np
import pytest
import torch

from util import TOL_GRAD, make_cells, make_inputs, rel_err
from v1_glif_model_b200 import synth

KW = dict(dampening_factor=0.5, pseudo_width=0.5, recurrent_dampening_factor=0.5,
          voltage_gradient_dampening=0.5)


def test_philox_known_answers():
    """Philox-4x32-10 known-answer vectors of the Random123 distribution (counter, key -> output)."""
    from oracle import rng
    kat = [([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
           ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
           ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
            [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1])]
    for ctr, key, want in kat:
        got = rng.philox4x32(np.array(ctr, dtype=np.uint32), np.array(key, dtype=np.uint32))
        assert [int(v) for v in got] == want


def test_oracle_sampler_distributions():
    from oracle import rng
    c = rng.bkg_counts(5, 0, 0, 4, 1000, 100, 0.25)
    n = c.size
    assert abs(c.mean() - 0.25) < 5 * np.sqrt(0.25 / n) and abs(c.var() - 0.25) < 0.01
    # the key is (seed + replica * 1000003, step): replica r of seed s = replica 0 of seed s + r * 1000003
    assert np.array_equal(rng.bkg_counts(5, 2, 7, 2, 9, 100, 0.25), rng.bkg_counts(5 + 2 * 1000003, 0, 7, 2, 9, 100, 0.25))
    assert np.array_equal(rng.bkg_counts(5, 0, 0, 2, 30, 100, 0.25)[:, 10:], rng.bkg_counts(5, 0, 10, 2, 20, 100, 0.25))


def _chi2(observed, expected):
    return float(((observed - expected) ** 2 / expected).sum())


@pytest.mark.gpu
def test_background_counts_match_the_restatement_and_poisson():
    from math import exp, factorial
    from oracle import rng
    cfg, dicts, orc, cell = make_cells("small", **KW)
    cell.set_noise_seed(11, 3)
    got = cell.sample_bkg_counts(4, 500, first_step=17).cpu().numpy()
    want = rng.bkg_counts(11, 3, 17, 4, 500, cell.n_bkg, cell.bkg_firing_rate * 1e-3)
    assert np.array_equal(got, want)                         # bit for bit
    # same arguments -> same draws; another seed, replica or step -> other draws
    assert torch.equal(cell.sample_bkg_counts(4, 500, first_step=17), torch.from_numpy(got).cuda())
    cell.set_noise_seed(12, 3)
    assert not np.array_equal(cell.sample_bkg_counts(4, 500, first_step=17).cpu().numpy(), got)
    cell.set_noise_seed(11, 3)
    big = cell.sample_bkg_counts(8, 4000).cpu().numpy().ravel()
    lam = 0.25
    pmf = np.array([exp(-lam) * lam ** k / factorial(k) for k in range(4)])
    pmf = np.append(pmf, 1.0 - pmf.sum())
    obs = np.bincount(np.minimum(big, 4), minlength=5).astype(np.float64)
    assert _chi2(obs, pmf * big.size) < 35.0                 # 4 degrees of freedom, p ~ 5e-7
    assert abs(big.mean() - lam) < 5 * np.sqrt(lam / big.size)


@pytest.mark.gpu
def test_lgn_spikes_match_the_restatement_and_their_rates():
    from oracle import rng
    cfg, dicts, orc, cell = make_cells("small", **KW)
    t_len, n_lgn, b = 400, cell.input_dim, 3
    gen = np.random.Generator(np.random.PCG64(3))
    rates = gen.uniform(0.0, 60.0, (t_len, n_lgn)).astype(np.float32)
    rates[:, 0] = 0.0                                        # a silent unit never fires
    x = cell.sample_lgn_spikes(torch.from_numpy(rates).cuda(), b, seed=2**40 + 5).cpu().numpy()
    want = rng.lgn_spikes(rates, b, 2**40 + 5)
    # expm1 may differ in the last bit between the two implementations: a draw that lands exactly
    # there may flip
    assert (x != want).mean() <= 1e-5
    assert x[:, :, 0].sum() == 0
    p = rng.lgn_probability(rates).astype(np.float64)
    z = (x.sum(0).sum() - b * p.sum()) / np.sqrt(b * (p * (1 - p)).sum())
    assert abs(z) < 5.0
    per_trial = np.stack([rates, rates * 0.5, rates * 0.0]).astype(np.float32)   # one table per trial
    xt = cell.sample_lgn_spikes(torch.from_numpy(per_trial).cuda(), b, seed=9).cpu().numpy()
    assert xt[2].sum() == 0 and xt[0].sum() > xt[1].sum() > 0


@pytest.mark.gpu
def test_rate_driven_rollout_equals_rollout_over_sampled_spikes():
    cfg, dicts, orc, cell = make_cells("small", **KW)
    t_len, b = 50, cfg.batch
    gen = np.random.Generator(np.random.PCG64(4))
    rates = torch.from_numpy(gen.uniform(5.0, 120.0, (t_len, cell.input_dim)).astype(np.float32)).cuda()
    x = cell.sample_lgn_spikes(rates, b, seed=123)
    c = cell.sample_bkg_counts(b, t_len)
    z1, v1 = cell.rollout(x, c)
    z2, v2 = cell.rollout_rates(rates, 123, b, bkg_counts=c)
    z3, v3 = cell.rollout_rates(rates, 123, b)             # counts drawn inside: steps 0.. of the same seed
    cell.synchronize()
    assert int(z1.sum()) > 0
    assert torch.equal(z1, z2) and torch.equal(z1, z3)
    assert rel_err(v2, v1) <= 1e-6 and rel_err(v3, v1) <= 1e-6
    cnt = cell.counters()
    assert cnt["lgn_rows"] == int(x.sum())


@pytest.mark.gpu
def test_sampled_noise_is_the_same_in_chunks_and_in_the_backward_pass():
    cfg, dicts, orc, cell = make_cells("small", **KW)
    x, _ = make_inputs(cfg, seq_len=50)
    xg = torch.from_numpy(x).cuda()
    cell.set_noise_seed(21, 1)
    s_one = cell.zero_state(cfg.batch)
    z1, _ = cell.rollout(xg, None, state=s_one, save_for_bwd=True)
    loss = dict(rate_cost=10.0, voltage_cost=1e-1, sync_cost=0.5, fano_target=1.0, sync_bin=10,
                rate_target=torch.from_numpy(synth.make_rate_targets(cfg)).cuda() / 1000.0)
    g1 = cell.backward(loss)
    s_two = cell.zero_state(cfg.batch)
    za, _ = cell.rollout(xg[:, :23].contiguous(), None, state=s_two)
    assert s_two[6].tolist() == [23] * cfg.batch            # noise_step advanced (models.py:1133)
    zb, _ = cell.rollout(xg[:, 23:].contiguous(), None, state=s_two)
    cell.synchronize()
    assert torch.equal(torch.cat([za, zb], 1), z1) and s_two[6].tolist() == [50] * cfg.batch
    # the counts of that seed given explicitly: same spikes, same gradients
    c = cell.sample_bkg_counts(cfg.batch, 50, first_step=0)
    z2, _ = cell.rollout(xg, c, save_for_bwd=True)
    g2 = cell.backward(loss)
    cell.synchronize()
    assert torch.equal(z2, z1)
    for a, b in zip(g1[:3], g2[:3]):
        assert rel_err(a, b) <= 1e-6
    assert float(g1[2].abs().max()) > 0
    # the next rollout of a training loop uses the next seed (tf_utils.py:235-237): other noise
    cell.set_noise_seed(22, 1)
    z3, _ = cell.rollout(xg, None)
    assert not torch.equal(z3, z1)
