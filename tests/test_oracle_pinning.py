"""Pins the oracle (and, on a GPU, the CUDA path) to the reference's own cell.

``tests/golden/reference_*.npz`` were produced by ``tests/golden/run_reference_models.py``, which
imports the reference's unmodified ``v1_model_utils/models.py`` over a torch-backed stand-in for
the TensorFlow calls it makes and steps its ``V1Column.call``.  The fixtures travel; the reference
tree and the stand-in are not needed to run these tests.
"""
import os

import numpy as np
import pytest
import torch

from util import TOL_GRAD, TOL_STATE, make_case, rel_err

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CASES = ["reference_tiny", "reference_tiny_hard_reset", "reference_small", "reference_small_gauss",
         "reference_small_real_basis"]


def _load(name):
    g = np.load(os.path.join(ROOT, "tests", "golden", name + ".npz"))
    kw = dict(dampening_factor=float(g["kw_dampening_factor"]),
              recurrent_dampening_factor=float(g["kw_recurrent_dampening_factor"]),
              voltage_gradient_dampening=float(g["kw_voltage_gradient_dampening"]),
              hard_reset=bool(g["hard_reset"]))
    if "pseudo_gauss" in g.files and bool(g["pseudo_gauss"]):
        kw.update(pseudo_gauss=True, gauss_std=float(g["gauss_std"]))
    return g, kw


def _case_kwargs(g):
    """Arguments of ``make_case`` that rebuild the fixture's network: for the fixture with the
    reference's own synaptic basis (4 time constants, 121 rows of basis weights) the tables and the
    synapse types stored in it replace the synthetic one-hot basis."""
    if "synaptic_basis_weights" not in g.files:
        return {}

    def mutate(net, lgn, bkg):
        net["tau_syn"] = g["tau_syn"]
        net["synaptic_basis_weights"] = g["synaptic_basis_weights"]
        net["synapses"]["syn_ids"], lgn["syn_ids"], bkg["syn_ids"] = g["syn_ids_rec"], g["syn_ids_lgn"], g["syn_ids_bkg"]
    return dict(n_receptors=int(g["tau_syn"].size), mutate=mutate)


def _cotangents(g):
    """Output cotangents of the fixture: stored, or regenerated from its seed (same generator
    calls as tests/golden/run_reference_models.py)."""
    if "g_z" in g.files:
        return torch.from_numpy(g["g_z"]), torch.from_numpy(g["g_v"])
    gen = torch.Generator().manual_seed(int(g["g_seed"]))
    shape = g["v"].shape
    g_z = torch.randn(shape, generator=gen, dtype=torch.float64) * 1e-2
    g_v = torch.randn(shape, generator=gen, dtype=torch.float64) * 1e-3
    return g_z, g_v


@pytest.mark.parametrize("name", CASES)
def test_oracle_equals_reference_cell(name):
    g, kw = _load(name)
    cfg, dicts, orc = make_case(str(g["config"]), seed=int(g["seed"]), dtype=torch.float64, **_case_kwargs(g), **kw)
    # the CSR table the reference built (make_pre_ind_table) is reproduced exactly
    assert np.array_equal(orc.pre_ind_table.order.numpy(), g["pre_ind_order"])
    assert np.array_equal(orc.pre_ind_table.row_splits.numpy(), g["pre_ind_row_splits"])
    z, v, state = orc.rollout(torch.from_numpy(g["x"]), torch.from_numpy(g["bkg_counts"]).long())
    assert np.array_equal(z.detach().numpy().astype(np.uint8), g["z"])
    assert np.abs(v.detach().numpy() - g["v"]).max() <= 1e-12
    for got, key in zip((state[0], state[3], state[4], state[5]), ("z_buf", "asc", "psc_rise", "psc")):
        assert np.abs(got.detach().numpy() - g[key]).max() <= 1e-12
    assert np.array_equal(state[2].numpy(), g["r"].astype(np.int64))
    g_z, g_v = _cotangents(g)
    ((z * g_z).sum() + (v * g_v).sum()).backward()
    for w, key in ((orc.recurrent_weight_values, "dw_rec"), (orc.input_weight_values, "dw_lgn"),
                   (orc.bkg_input_weights, "dw_bkg")):
        assert rel_err(w.grad, g[key]) <= 1e-10


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_cuda_path_equals_reference_cell(name):
    from v1_glif_model_b200.models import V1Column
    g, kw = _load(name)
    cfg, dicts, _ = make_case(str(g["config"]), seed=int(g["seed"]), **_case_kwargs(g), **kw)
    cell = V1Column(*dicts, **kw)
    order, splits = cell.pre_ind_table(0)
    assert np.array_equal(order, g["pre_ind_order"]) and np.array_equal(splits, g["pre_ind_row_splits"])
    state = cell.zero_state(g["x"].shape[0])
    z, v = cell.rollout(torch.from_numpy(g["x"]).cuda(), torch.from_numpy(g["bkg_counts"]).cuda(),
                        state=state)
    cell.synchronize()
    assert np.array_equal(z.cpu().numpy(), g["z"])
    assert rel_err(v, g["v"]) <= TOL_STATE
    for got, key in zip((state[0], state[3], state[4], state[5]), ("z_buf", "asc", "psc_rise", "psc")):
        assert rel_err(got, g[key]) <= TOL_STATE
    assert np.array_equal(state[2].cpu().numpy(), g["r"])
    cell.rollout(torch.from_numpy(g["x"]).cuda(), torch.from_numpy(g["bkg_counts"]).cuda(),
                 return_z=False, return_v=False, save_for_bwd=True)
    g_z, g_v = _cotangents(g)
    grads = cell.backward(None, g_z=g_z.float().cuda(), g_v=g_v.float().cuda())
    cell.synchronize()
    for got, key in zip(grads[:3], ("dw_rec", "dw_lgn", "dw_bkg")):
        assert rel_err(got, g[key]) <= TOL_GRAD


def _rate_fixture():
    f = np.load(os.path.join(ROOT, "tests", "golden", "reference_rate_loss.npz"))
    sizes = f["group_sizes"]
    offs = np.concatenate([[0], np.cumsum(sizes)])
    groups = [(f["group_neurons"][offs[i]:offs[i + 1]], f["group_targets"][offs[i]:offs[i + 1]])
              for i in range(len(sizes))]
    return f, groups


def test_oracle_rate_distribution_loss_equals_reference_loss_code():
    """``oracle/losses.py::rate_distribution_loss`` against the value and gradient the reference's
    ``compute_spike_rate_target_loss`` produced for the same spikes (fp64)."""
    from oracle import losses
    f, groups = _rate_fixture()
    z = torch.from_numpy(f["z"].astype(np.float64)).requires_grad_(True)
    loss = losses.rate_distribution_loss(z, groups, float(f["rate_cost"]), kappa=float(f["kappa"]),
                                         pre_delay=int(f["pre_delay"]), post_delay=int(f["post_delay"]))
    loss.backward()
    assert abs(loss.item() - float(f["loss"])) <= 1e-12 * abs(float(f["loss"]))
    assert rel_err(z.grad, torch.from_numpy(f["grad_z"])) <= 1e-12


def test_oracle_population_fano_loss_equals_reference_loss_code():
    """``oracle/losses.py::population_fano_loss`` against the Fano factors, loss and gradient that the
    reference's ``SynchronizationLoss.pop_fano_tf`` produced for the same population counts (fp64)."""
    from oracle import losses
    f = np.load(os.path.join(ROOT, "tests", "golden", "reference_sync_loss.npz"))
    pop = torch.from_numpy(f["counts"]).requires_grad_(True)
    loss = losses.population_fano_loss(pop, f["bin_sizes"], f["targets"], float(f["sync_cost"]))
    loss.backward()
    assert abs(loss.item() - float(f["loss"])) <= 1e-12 * abs(float(f["loss"]))
    assert rel_err(pop.grad, torch.from_numpy(f["grad_counts"])) <= 1e-12


@pytest.mark.parametrize("tag", ["plain", "normalized"])
def test_oracle_orientation_selectivity_loss_equals_reference_loss_code(tag):
    """``oracle/losses.py::orientation_selectivity_loss`` against the value and gradient of the
    reference's ``OrientationSelectivityLoss.__call__`` (crowd OSI/DSI) for the same spikes (fp64)."""
    from oracle import losses
    f = np.load(os.path.join(ROOT, "tests", "golden", "reference_osi_loss.npz"))
    z = torch.from_numpy(f["z"].astype(np.float64)).requires_grad_(True)
    loss = losses.orientation_selectivity_loss(
        z, f["angle"], f["tuning"], f["type_ids"], f["osi_targets"], f["dsi_targets"], f["type_counts"],
        float(f["osi_cost"]), pre_delay=int(f["pre_delay"]), post_delay=int(f["post_delay"]),
        normalizer=f["normalizer"] if tag == "normalized" else None)
    loss.backward()
    want = float(f["loss_" + tag])
    assert abs(loss.item() - want) <= 1e-12 * abs(want)
    assert rel_err(z.grad, torch.from_numpy(f["grad_z_" + tag])) <= 1e-11


def _expadam_fixture():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_expadam.npz"))


def test_oracle_expadam_equals_reference_optimizer_code():
    """``oracle/expadam.py`` against weights and moments that the reference's
    ``ExponentiatedAdam.update_step`` (dense branch) followed by its ``SignedConstraint`` produced over
    four steps in float32 (tests/golden/run_reference_optimizer.py)."""
    from oracle.expadam import expadam_step
    f = _expadam_fixture()
    w, pos = torch.from_numpy(f["w0"]), torch.from_numpy(f["positive"])
    m, v = torch.zeros_like(w), torch.zeros_like(w)
    for k in range(f["grads"].shape[0]):
        w, m, v = expadam_step(w, torch.from_numpy(f["grads"][k]), m, v, pos, float(f["lr"]),
                               float(f["beta_1"]), float(f["beta_2"]), float(f["epsilon"]), k + 1)
        assert rel_err(m, f["m"][k]) <= 1e-7 and rel_err(v, f["v"][k]) <= 1e-7
        assert rel_err(w, f["w"][k]) <= 1e-7
        assert np.array_equal(w.numpy() == 0, f["w"][k] == 0)       # zeros stay zeros, nothing else becomes one


@pytest.mark.gpu
def test_cuda_expadam_equals_reference_optimizer_code():
    """The Exp-Adam kernel against the same reference-generated fixture, through the C ABI."""
    import ctypes as C
    from v1_glif_model_b200 import _lib
    f = _expadam_fixture()
    lib = _lib.load()
    w = torch.from_numpy(f["w0"]).cuda()
    pos = torch.from_numpy(f["positive"].astype(np.uint8)).cuda()
    m, v = torch.zeros_like(w), torch.zeros_like(w)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for k in range(f["grads"].shape[0]):
        g = torch.from_numpy(f["grads"][k]).cuda()
        rc = lib.v1g_expadam_update(w.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), pos.data_ptr(),
                                    w.numel(), float(f["lr"]), float(f["beta_1"]), float(f["beta_2"]),
                                    float(f["epsilon"]), k + 1, 1.0, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert rel_err(m, f["m"][k]) <= 1e-6 and rel_err(v, f["v"][k]) <= 1e-6
        assert rel_err(w, f["w"][k]) <= 1e-6
        assert np.array_equal(w.cpu().numpy() == 0, f["w"][k] == 0)


def _regularizer_fixture():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_weight_regularizers.npz"))


@pytest.mark.parametrize("tag", ["mean_stiff", "mean_stiff_relative", "emd"])
def test_oracle_weight_regularizers_equal_reference_loss_code(tag):
    """``oracle/losses.py`` forms of the reference's weight regularisers against value and gradient that
    ``MeanStiffRegularizer`` / ``EarthMoversDistanceRegularizer`` produced for the same weights (fp64)."""
    from oracle import losses
    f = _regularizer_fixture()
    idx, n_groups, order, splits = losses.regularizer_groups(f["edge_type_ids"])
    w = torch.from_numpy(f["weights"]).requires_grad_(True)
    s = float(f["strength"])
    if tag == "emd":
        loss = losses.emd_regularizer(w, order, splits, f["initial_weights"].astype(np.float64), s)
    else:
        loss = losses.mean_stiff_regularizer(w, idx, n_groups, f["initial_weights"].astype(np.float64), s,
                                             relative=tag.endswith("relative"))
    loss.backward()
    want = float(f["loss_" + tag])
    assert abs(loss.item() - want) <= 1e-10 * abs(want)
    assert rel_err(w.grad, f["grad_" + tag]) <= 1e-9


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["mean_stiff", "mean_stiff_relative", "emd"])
def test_cuda_weight_regularizers_equal_reference_loss_code(tag):
    """The device kernels against the same reference-generated fixture (fp32 arithmetic: value within
    1e-5, gradient within 1e-4)."""
    from oracle import losses
    from v1_glif_model_b200.training import WeightRegularizer
    from util import make_cells
    f = _regularizer_fixture()
    cfg, dicts, orc, cell = make_cells("small", seed=4)
    kind = "emd" if tag == "emd" else "mean_stiff"
    reg = WeightRegularizer(cell, kind, f["edge_type_ids"], f["initial_weights"], float(f["strength"]),
                            relative=tag.endswith("relative"))
    w = torch.from_numpy(f["weights"].astype(np.float32)).cuda()
    grad = torch.zeros_like(w)
    loss = torch.zeros(1, device="cuda")
    reg(w, grad, loss)
    torch.cuda.synchronize()
    want = float(f["loss_" + tag])
    assert abs(float(loss) - want) <= 1e-5 * abs(want)
    assert rel_err(grad, f["grad_" + tag]) <= 1e-4
    # the gradient is accumulated, the value added
    reg(w, grad, loss)
    torch.cuda.synchronize()
    assert abs(float(loss) - 2 * want) <= 2e-5 * abs(want) and rel_err(grad, 2 * f["grad_" + tag]) <= 1e-4
