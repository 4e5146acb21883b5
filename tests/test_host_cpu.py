"""CPU tests: host logic, oracle self-checks, and that libv1g.so loads and exports the C ABI."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from v1_glif_model_b200 import _lib, synth
from v1_glif_model_b200.models import make_pre_ind_table

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(built_lib):
    header = open(os.path.join(ROOT, "include", "v1g.h")).read()
    declared = set(re.findall(r"\b(v1g_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 20
    lib = ctypes.CDLL(built_lib)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/v1g.h but not exported"
    # the Python binding covers the same set
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert _lib.load().v1g_version().startswith(b"v1g-sm100a")


def test_pre_ind_table_matches_oracle(built_lib):
    from oracle.cell_torch import make_pre_ind_table as oracle_table
    rng = np.random.default_rng(0)
    for n_src, nnz in [(7, 0), (5, 40), (1000, 5000), (33, 1)]:
        idx = np.stack([np.sort(rng.integers(0, 50, nnz)), rng.integers(0, n_src, nnz)], -1)
        order, splits = make_pre_ind_table(idx, n_src)
        o_order, o_splits = oracle_table(idx, n_src)
        assert np.array_equal(order, o_order)      # bit-exact, same stable order inside rows
        assert np.array_equal(splits, o_splits)    # empty rows kept
        assert splits.shape == (n_src + 1,)


def test_pre_ind_table_errors_like_reference(built_lib):
    with pytest.raises(ValueError, match="must be > 0"):
        make_pre_ind_table(np.zeros((0, 2), np.int64), 0)
    with pytest.raises(ValueError, match="must have shape"):
        make_pre_ind_table(np.zeros((4,), np.int64), 3)
    with pytest.raises(ValueError, match="Presynaptic index 9 is out of bounds"):
        make_pre_ind_table(np.array([[0, 1], [1, 9]]), 5)
    with pytest.raises(ValueError, match="Presynaptic index -1 is out of bounds"):
        make_pre_ind_table(np.array([[0, -1]]), 5)


def test_synthetic_network_schema_and_order():
    net, lgn, bkg = synth.make_network("small", seed=3)
    net2, _, _ = synth.make_network("small", seed=3)
    assert np.array_equal(net["synapses"]["indices"], net2["synapses"]["indices"])
    for d, n_src in ((net["synapses"], net["n_nodes"]), (lgn, lgn["n_inputs"]), (bkg, bkg["n_inputs"])):
        idx = d["indices"]
        key = idx[:, 0] * (idx.max() + 1) + idx[:, 1]
        assert np.all(np.diff(key) >= 0)           # post-major, as load_sparse.sort_indices
        assert idx[:, 1].max() < n_src and idx[:, 0].max() < net["n_nodes"]
        assert d["weights"].dtype == np.float32 and d["syn_ids"].dtype == np.uint8
    assert set(net["node_params"]) == {"C_m", "g", "E_L", "V_th", "V_reset", "t_ref", "k", "asc_amps"}
    x = synth.make_lgn_spikes("small", 2, 30)
    c = synth.make_bkg_counts("small", 2, 30)
    assert x.shape == (2, 30, lgn["n_inputs"]) and x.dtype == np.uint8
    assert c.shape == (2, 30, bkg["n_inputs"]) and c.dtype == np.int32


def test_oracle_custom_gradients_match_plain_autograd():
    """The oracle's hand-written gradient of the recurrent currents (the reference's
    tf.custom_gradient) equals autograd of a dense restatement of the same forward."""
    from util import make_case
    cfg, dicts, orc = make_case("tiny", dtype=torch.float64)
    n, d, r = cfg.n_neurons, orc.max_delay, orc._n_syn_basis
    torch.manual_seed(0)
    z_buf = (torch.rand(2, n * d, dtype=torch.float64) < 0.2).double().requires_grad_(True)
    dy = torch.randn(2 * n, r, dtype=torch.float64)
    out = orc.calculate_i_rec_with_custom_grad(z_buf)
    gz, gw = torch.autograd.grad(out, [z_buf, orc.recurrent_weight_values], dy)
    # dense restatement: I[b,post,r] = sum_syn z[b,pre_d] * w * basis[sid,r]
    w = orc.recurrent_weight_values.detach().clone().requires_grad_(True)
    z2 = z_buf.detach().clone().requires_grad_(True)
    idx = orc.recurrent_indices
    contrib = z2[:, idx[:, 1]][:, :, None] * (w[:, None] * orc.synaptic_basis_weights[orc.syn_ids])[None]
    dense = torch.zeros(2, n, r, dtype=torch.float64).index_add(1, idx[:, 0], contrib)
    gz2, gw2 = torch.autograd.grad(dense.reshape(2 * n, r), [z2, w], dy)
    assert torch.allclose(out, dense.reshape(2 * n, r).detach(), atol=1e-12)
    assert torch.allclose(gz, gz2, atol=1e-12)
    assert torch.allclose(gw, gw2, atol=1e-12)


def test_oracle_against_golden_vectors():
    """The committed fixture (written by tests/golden/make_golden.py) pins the oracle."""
    from util import make_case, make_inputs
    path = os.path.join(ROOT, "tests", "golden", "tiny_rollout.npz")
    g = np.load(path)
    cfg, dicts, orc = make_case("tiny", dtype=torch.float64, **_golden_kwargs())
    x, c = make_inputs(cfg)
    assert np.array_equal(x, g["x"]) and np.array_equal(c, g["bkg_counts"])
    with torch.no_grad():
        z, v, state = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    assert np.array_equal(z.numpy().astype(np.uint8), g["z"])
    assert np.allclose(v.numpy(), g["v"], rtol=0, atol=1e-12)
    assert np.allclose(state[5].numpy(), g["psc"], rtol=0, atol=1e-12)


def _golden_kwargs():
    return dict(dampening_factor=0.5, pseudo_width=0.5, recurrent_dampening_factor=0.5,
                voltage_gradient_dampening=0.5)


def test_flat_gradients_and_trainer_bookkeeping():
    from v1_glif_model_b200.training import FlatGradients
    fg = FlatGradients([3, 0, 5], "cpu")
    fg.views[0].fill_(1.0)
    fg.views[2].fill_(2.0)
    assert fg.flat.tolist() == [1, 1, 1, 2, 2, 2, 2, 2]
    assert fg.views[1].numel() == 0
    fg.all_reduce()  # no process group: unchanged
    assert fg.flat.sum().item() == 13.0
    fg.zero_()
    assert fg.flat.abs().sum().item() == 0.0


def test_expadam_oracle_properties():
    from oracle.expadam import expadam_step
    torch.manual_seed(1)
    w = torch.randn(100)
    w[:5] = 0.0
    pos = w >= 0
    g = torch.randn(100)
    w1, m1, v1 = expadam_step(w, g, torch.zeros(100), torch.zeros(100), pos, 1e-2, 0.9, 0.999, 1e-11, 1)
    assert torch.all((w1 >= 0) == pos | (w1 == 0))          # multiplicative update keeps the sign
    assert torch.all(w1[:5] == 0)                            # zeros stay zero
    up = (g < 0) & (w > 0)
    assert torch.all(w1[up] > w[up])                         # negative gradient grows |w|


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-13), (torch.float32, 2e-6)])
def test_oracle_scatter_transpose_equals_sparse_matmul(dtype, tol):
    """The oracle's optional scatter form of the spike-gradient product (used by the full-length
    parity runs at the benchmark shapes) gives the gradients of the reference-shaped form, which
    builds one sparse tensor per receptor channel and step (``models.py:187-202``)."""
    from util import make_case, make_inputs, rel_err
    kw = dict(dampening_factor=0.5, pseudo_width=0.5, recurrent_dampening_factor=0.3,
              voltage_gradient_dampening=0.4, dtype=dtype)
    grads = []
    for scatter in (False, True):
        cfg, dicts, orc = make_case("small", scatter_transpose=scatter, **kw)
        x, c = make_inputs(cfg, seq_len=25)
        z, v, _ = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
        g = torch.Generator().manual_seed(3)
        g_z = torch.randn(z.shape, generator=g, dtype=torch.float64).to(dtype) * 1e-2
        g_v = torch.randn(v.shape, generator=g, dtype=torch.float64).to(dtype) * 1e-3
        ((z * g_z).sum() + (v * g_v).sum()).backward()
        grads.append([w.grad.clone() for w in (orc.recurrent_weight_values, orc.input_weight_values,
                                               orc.bkg_input_weights)])
    for a, b in zip(*grads):
        assert float(b.abs().max()) > 0
        assert rel_err(a, b) <= tol
