"""Golden vectors for the firing-rate target from the reference's OWN loss code (run from the repo
root, in a container that has the reference tree):

    python tests/golden/run_reference_losses.py /path/to/V1_GLIF_model

Imports ``v1_model_utils/loss_functions.py`` unmodified over ``tf_standin`` (its ``other_v1_utils``
import, which needs h5py, is satisfied by an empty module: none of the functions used here touch
it), and evaluates ``spike_trimming`` -> mean over batch and time ->
``compute_spike_rate_target_loss`` x ``rate_cost`` - the body of
``SpikeRateDistributionTarget.__call__`` - on seeded spikes of the 600-neuron synthetic net, with
one population per node type.  Writes ``tests/golden/reference_rate_loss.npz`` (spikes, populations,
loss, gradient with respect to the spikes' per-neuron rates).  ``tests/test_oracle_pinning.py``
checks ``oracle/losses.py::rate_distribution_loss`` against it.  A second fixture,
``reference_sync_loss.npz``, holds the population Fano factors of
``SynchronizationLoss.pop_fano_tf`` for seeded population counts and the loss built from them, for
``oracle/losses.py::synchronization_loss``; a third, ``reference_osi_loss.npz``, the population
OSI/DSI target (``OrientationSelectivityLoss`` with ``method="crowd_osi"``) with and without the
rate normalizer, for ``oracle/losses.py::orientation_selectivity_loss``.

The stand-in's ``tf.random.shuffle`` is the identity and its ``tf.sort`` is stable, so neurons with
equal rates keep the order of ``neuron_ids`` (the reference orders them at random).
"""
import importlib.util
import os
import sys
import tempfile
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import tf_standin  # noqa: E402
from v1_glif_model_b200 import synth  # noqa: E402

RATE_COST, PRE_DELAY, POST_DELAY = 100.0, 5, 3


def load_reference_losses(ref_root):
    os.environ.setdefault("NUMBA_CACHE_DIR", tempfile.mkdtemp(prefix="numba_cache_"))
    tf_standin.install()
    sys.modules.setdefault("other_v1_utils", types.ModuleType("other_v1_utils"))
    spec = importlib.util.spec_from_file_location(
        "reference_losses", os.path.join(ref_root, "v1_model_utils", "loss_functions.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("V1_GLIF_REFERENCE", "V1_GLIF_model")
    lf = load_reference_losses(ref_root)
    cfg = synth.CONFIGS["small"]
    net, _, _ = synth.make_network(cfg, 3)
    groups = synth.make_rate_groups(cfg, net, 3)
    rng = np.random.Generator(np.random.PCG64(99))
    b, t, n = 2, 40, cfg.n_neurons
    p = rng.lognormal(np.log(0.02), 1.0, n).clip(0.0, 0.5)           # per-neuron spike probability
    z = (rng.random((b, t, n)) < p[None, None, :]).astype(np.float64)
    zt = torch.from_numpy(z).requires_grad_(True)
    target_rates = {
        f"type{i}": dict(neuron_ids=torch.from_numpy(ids.astype(np.int64)),
                         sorted_target_rates=torch.from_numpy(tg.astype(np.float64)))
        for i, (ids, tg) in enumerate(groups)}
    trimmed = lf.spike_trimming(zt, pre_delay=PRE_DELAY, post_delay=POST_DELAY, trim=True)
    rates = trimmed.mean(dim=(0, 1))
    loss = lf.compute_spike_rate_target_loss(rates, target_rates, dtype=torch.float64) * RATE_COST
    loss.backward()
    out = os.path.join(HERE, "reference_rate_loss.npz")
    np.savez_compressed(
        out, z=z.astype(np.uint8), loss=loss.item(), grad_z=zt.grad.numpy(),
        rate_cost=RATE_COST, pre_delay=PRE_DELAY, post_delay=POST_DELAY, kappa=0.002,
        group_sizes=np.array([len(g[0]) for g in groups], dtype=np.int64),
        group_neurons=np.concatenate([g[0] for g in groups]).astype(np.int32),
        group_targets=np.concatenate([g[1] for g in groups]).astype(np.float32))
    ties = sum(int(len(np.unique(z[:, PRE_DELAY:t - POST_DELAY, g[0]].sum((0, 1)))) < len(g[0])) for g in groups)
    print(f"wrote {out}: loss {loss.item():.6e}, populations {len(groups)}, with ties {ties}")


def sync_fixture(ref_root):
    """Population Fano factors of the reference's ``SynchronizationLoss.pop_fano_tf`` and the mean
    squared error of ``__call__`` (``loss_functions.py:964-981, 1031-1044``) for seeded population
    counts; ``self`` is a stand-in object with the three attributes the method reads."""
    lf = load_reference_losses(ref_root)
    import tf_standin as _ts
    tf = sys.modules["tensorflow"]
    rng = np.random.Generator(np.random.PCG64(7))
    n_samples, width = 6, 120
    counts = rng.poisson(rng.uniform(0.2, 3.0, (n_samples, 1)), (n_samples, width)).astype(np.float64)
    counts[0] = 0.0                                     # a silent sample: mean clamped at 1e-7
    bin_sizes = (1, 2, 3, 5, 8, 13, 21, 34, 55, 89)     # the last two are not below half the window
    targets = rng.uniform(0.8, 2.5, len(bin_sizes))
    used = [b for b in bin_sizes if b < width // 2]
    stub = types.SimpleNamespace(_bin_sizes_ms=tuple(used), _dtype=torch.float64,
                                 _epsilon_tf=torch.tensor(1e-7, dtype=torch.float64))
    x = torch.from_numpy(counts).requires_grad_(True)
    fanos = lf.SynchronizationLoss.pop_fano_tf(stub, x)
    mse = tf.reduce_mean(tf.square(torch.from_numpy(targets[:len(used)]) - fanos))
    loss = 10.0 * mse
    loss.backward()
    out = os.path.join(HERE, "reference_sync_loss.npz")
    np.savez_compressed(out, counts=counts, bin_sizes=np.array(bin_sizes), targets=targets, sync_cost=10.0,
                        fanos=fanos.detach().numpy(), loss=loss.item(), grad_counts=x.grad.numpy())
    print(f"wrote {out}: loss {loss.item():.6e}, fanos {fanos.detach().numpy().round(3)}")


def osi_fixture(ref_root):
    """The population OSI/DSI target of the reference (``OrientationSelectivityLoss.__call__`` with
    ``method="crowd_osi"``, ``loss_functions.py:1340-1440``) on seeded spikes; the object is created
    without its constructor (which reads recorded data) and given the attributes the method reads."""
    lf = load_reference_losses(ref_root)
    rng = np.random.Generator(np.random.PCG64(11))
    b, t, n, n_types = 3, 50, 400, 4
    tuning = rng.uniform(0.0, 360.0, n)
    type_ids = rng.integers(0, n_types, n)
    angle = np.array([0.0, 45.0, 270.0])
    # orientation-tuned spike probabilities so that OSI and DSI are away from zero
    d = np.deg2rad(angle[:, None] - tuning[None, :])
    p = 0.02 * (1.0 + 0.6 * np.cos(2 * d) + 0.3 * np.cos(d)) * rng.lognormal(0.0, 0.5, n)[None, :]
    p[:, type_ids == 3] *= 0.002                       # a nearly silent type: denominator clamped
    z = (rng.random((b, t, n)) < p[:, None, :]).astype(np.float64)
    normalizer = rng.lognormal(np.log(0.01), 0.7, n)
    normalizer[::17] = 0.0                             # below the floor of 0.0005
    osi_t, dsi_t = rng.uniform(0.2, 0.6, n_types), rng.uniform(0.05, 0.3, n_types)
    counts = np.bincount(type_ids, minlength=n_types).astype(np.float64)
    out = {}
    for tag, norm in (("plain", None), ("normalized", normalizer)):
        obj = object.__new__(lf.OrientationSelectivityLoss)
        obj._pre_delay, obj._post_delay, obj._dtype, obj._method = 4, 6, torch.float64, "crowd_osi"
        obj._core_mask, obj._osi_cost = None, 20.0
        obj._tuning_angles = torch.from_numpy(tuning)
        obj._tf_pi = torch.tensor(np.pi, dtype=torch.float64)
        obj._min_rates_threshold = torch.tensor(0.0005, dtype=torch.float64)
        obj.node_type_ids = torch.from_numpy(type_ids.astype(np.int64))
        obj._n_node_types = n_types
        obj.osi_target_values, obj.dsi_target_values = torch.from_numpy(osi_t), torch.from_numpy(dsi_t)
        obj.cell_type_count = torch.from_numpy(counts)
        zt = torch.from_numpy(z).requires_grad_(True)
        loss = obj(zt, torch.from_numpy(angle), True,
                   normalizer=None if norm is None else torch.from_numpy(norm))
        loss.backward()
        out["loss_" + tag], out["grad_z_" + tag] = loss.item(), zt.grad.numpy()
        print(f"osi/dsi {tag}: loss {loss.item():.6e}")
    path = os.path.join(HERE, "reference_osi_loss.npz")
    np.savez_compressed(path, z=z.astype(np.uint8), angle=angle, tuning=tuning, type_ids=type_ids.astype(np.int32),
                        osi_targets=osi_t, dsi_targets=dsi_t, type_counts=counts, normalizer=normalizer,
                        osi_cost=20.0, pre_delay=4, post_delay=6, **out)
    print(f"wrote {path}")


def regularizer_fixture(ref_root):
    """The reference's weight regularisers (``MeanStiffRegularizer`` in both forms,
    ``loss_functions.py:171-220``, and ``EarthMoversDistanceRegularizer``, ``:536-601``) built from the
    600-neuron synthetic net with seeded edge types, evaluated on perturbed weights: value and gradient
    with respect to the weights (fp64)."""
    lf = load_reference_losses(ref_root)
    sys.modules["other_v1_utils"].connection_type_ids = lambda network: network["synapses"]["edge_type_ids"]
    tf_standin.set_policy_dtype(torch.float64)
    cfg = synth.CONFIGS["small"]
    net, _, _ = synth.make_network(cfg, 4)
    rng = np.random.Generator(np.random.PCG64(21))
    nnz = net["synapses"]["indices"].shape[0]
    # edge types with gaps in their ids and very different sizes, one with a single synapse
    edge_types = rng.choice(np.array([3, 4, 9, 17, 18, 40, 41, 77]), size=nnz,
                            p=np.array([30, 20, 15, 12, 10, 8, 4, 1]) / 100.0).astype(np.int64)
    edge_types[0] = 500
    net["synapses"]["edge_type_ids"] = edge_types
    vscale = (net["node_params"]["V_th"] - net["node_params"]["E_L"]).astype(np.float32)
    w0 = np.asarray(net["synapses"]["weights"], dtype=np.float32) / \
        vscale[np.asarray(net["node_type_ids"])[net["synapses"]["indices"][:, 0]]]
    w = (w0.astype(np.float64) * rng.lognormal(0.0, 0.3, nnz))          # the weights after some training
    out = dict(edge_type_ids=edge_types, initial_weights=w0, weights=w)
    for tag, make in (("mean_stiff", lambda: lf.MeanStiffRegularizer(0.7, net, penalize_relative_change=False, dtype=torch.float64)),
                      ("mean_stiff_relative", lambda: lf.MeanStiffRegularizer(0.7, net, penalize_relative_change=True, dtype=torch.float64)),
                      ("emd", lambda: lf.EarthMoversDistanceRegularizer(0.7, net, dtype=torch.float64))):
        reg = make()
        x = torch.from_numpy(w).requires_grad_(True)
        loss = reg(x)
        loss.backward()
        out["loss_" + tag], out["grad_" + tag] = loss.item(), x.grad.numpy()
        print(f"{tag}: loss {loss.item():.6e}")
    path = os.path.join(HERE, "reference_weight_regularizers.npz")
    np.savez_compressed(path, strength=0.7, **out)
    print(f"wrote {path}")


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("V1_GLIF_REFERENCE", "V1_GLIF_model")
    if len(sys.argv) > 2 and sys.argv[2] == "regularizers":
        regularizer_fixture(root)
        sys.exit(0)
    main()
    sync_fixture(root)
    osi_fixture(root)
    regularizer_fixture(root)
