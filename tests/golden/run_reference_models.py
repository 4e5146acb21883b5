"""Golden vectors from the reference's OWN cell (run from the repo root, in a container that has
the reference tree):

    python tests/golden/run_reference_models.py /path/to/V1_GLIF_model [fixture names]

Imports ``v1_model_utils/models.py`` unmodified from the reference tree over ``tf_standin`` (a
torch-backed stand-in for the TensorFlow calls it makes), builds its ``V1Column`` from the seeded
synthetic dictionaries, steps ``V1Column.call`` T times and back-propagates fixed random
cotangents of the outputs.  Writes ``tests/golden/reference_tiny.npz`` (inputs, spikes, voltages,
final state, the three weight gradients); ``tests/test_oracle_pinning.py`` checks ``oracle/``
against it.  The reference reads ``synaptic_data/tau_basis.npy`` and
``<data_dir>/tf_data/syn_id_to_syn_weights_dict.pkl`` relative to the working directory; both are
written to a temporary directory from the synthetic network.
"""
import importlib.util
import os
import pickle
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import tf_standin  # noqa: E402
from v1_glif_model_b200 import synth  # noqa: E402

KW = dict(dampening_factor=0.5, recurrent_dampening_factor=0.3, voltage_gradient_dampening=0.4,
          train_recurrent=True, train_recurrent_per_type=False, train_input=True, train_noise=True)
CASES = {"reference_tiny": dict(config="tiny", seed=0, hard_reset=False),
         "reference_tiny_hard_reset": dict(config="tiny", seed=1, hard_reset=True),
         # a busier net (hundreds of spikes, refractory periods, all delays in use); the output
         # cotangents are regenerated from g_seed by the test instead of being stored
         "reference_small": dict(config="small", seed=2, hard_reset=False, batch=2, seq_len=40,
                                 store_cotangents=False),
         # the Gaussian pseudo-derivative (spike_gauss / gauss_pseudo, models.py:17-21, 36-50, 1106-1107)
         "reference_small_gauss": dict(config="small", seed=5, hard_reset=False, batch=2, seq_len=30,
                                       store_cotangents=False, pseudo_gauss=True, gauss_std=0.3),
         # the reference's own synaptic basis: 4 time constants (synaptic_data/tau_basis.npy) and the 121
         # rows of basis weights with negative entries (synaptic_data/basis_function_weights.csv); the
         # fixture carries both tables, so the tests that use it need no reference tree
         "reference_small_real_basis": dict(config="small", seed=6, hard_reset=False, batch=3, seq_len=30,
                                            store_cotangents=False, real_basis=True)}


def load_reference_models(ref_root):
    # the reference's numba helper asks for an on-disk cache; keep it out of the reference tree
    os.environ.setdefault("NUMBA_CACHE_DIR", tempfile.mkdtemp(prefix="numba_cache_"))
    tf_standin.install()
    tf_standin.set_policy_dtype(torch.float64)
    spec = importlib.util.spec_from_file_location(
        "reference_models", os.path.join(ref_root, "v1_model_utils", "models.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod      # numba resolves the module of its jitted helper by name
    spec.loader.exec_module(mod)
    return mod


def run_case(models, name, config, seed, hard_reset, batch=None, seq_len=None, store_cotangents=True,
             pseudo_gauss=False, gauss_std=0.5, real_basis=False, ref_root=None):
    import dataclasses
    cfg = synth.CONFIGS[config]
    cfg = dataclasses.replace(cfg, batch=batch or cfg.batch, seq_len=seq_len or cfg.seq_len)
    extra = {}
    if real_basis:
        cfg = dataclasses.replace(cfg, n_receptors=4)
    net, lgn, bkg = synth.make_network(cfg, seed)
    if real_basis:
        from v1_glif_model_b200 import load_sparse
        load_sparse.load_basis(os.path.join(ref_root, "synaptic_data", "tau_basis.npy"),
                               os.path.join(ref_root, "synaptic_data", "basis_function_weights.csv"), network=net)
        rng = np.random.Generator(np.random.PCG64(seed + 5))
        n_types = net["synaptic_basis_weights"].shape[0]
        for d in (net["synapses"], lgn, bkg):
            d["syn_ids"] = rng.integers(0, n_types, d["syn_ids"].shape[0]).astype(np.uint8)
        extra = dict(tau_syn=net["tau_syn"], synaptic_basis_weights=net["synaptic_basis_weights"],
                     syn_ids_rec=net["synapses"]["syn_ids"], syn_ids_lgn=lgn["syn_ids"], syn_ids_bkg=bkg["syn_ids"])
    x = synth.make_lgn_spikes(cfg, cfg.batch, cfg.seq_len, seed)
    counts = synth.make_bkg_counts(cfg, cfg.batch, cfg.seq_len, seed)
    cwd = os.getcwd()
    with tempfile.TemporaryDirectory() as tmp:
        os.makedirs(os.path.join(tmp, "synaptic_data"))
        os.makedirs(os.path.join(tmp, "net", "tf_data"))
        np.save(os.path.join(tmp, "synaptic_data", "tau_basis.npy"), net["tau_syn"])
        with open(os.path.join(tmp, "net", "tf_data", "syn_id_to_syn_weights_dict.pkl"), "wb") as f:
            pickle.dump({i: row for i, row in enumerate(np.asarray(net["synaptic_basis_weights"]))}, f)
        net = dict(net, data_dir=os.path.join(tmp, "net"))
        os.chdir(tmp)
        try:
            cell = models.V1Column(net, lgn, bkg, hard_reset=hard_reset, pseudo_gauss=pseudo_gauss,
                                   gauss_std=gauss_std, **KW)
        finally:
            os.chdir(cwd)
    state = cell.zero_state(cfg.batch)
    xt = torch.from_numpy(x).to(torch.float64)
    zs, vs = [], []
    for t in range(cfg.seq_len):
        tf_standin.set_poisson_counts(torch.from_numpy(counts[:, t]))
        (z, v), state = cell.call(xt[:, t], state)
        zs.append(z)
        vs.append(v)
    z, v = torch.stack(zs, 1), torch.stack(vs, 1)
    g = torch.Generator().manual_seed(99 + seed)
    g_z = torch.randn(z.shape, generator=g, dtype=torch.float64) * 1e-2
    g_v = torch.randn(v.shape, generator=g, dtype=torch.float64) * 1e-3
    ((z * g_z).sum() + (v * g_v).sum()).backward()
    out = os.path.join(HERE, name + ".npz")
    np.savez_compressed(
        out, config=config, seed=seed, hard_reset=hard_reset, pseudo_gauss=pseudo_gauss, gauss_std=gauss_std,
        x=x, bkg_counts=counts,
        g_seed=99 + seed, **(dict(g_z=g_z.numpy(), g_v=g_v.numpy()) if store_cotangents else {}), z=z.detach().numpy().astype(np.uint8),
        v=v.detach().numpy(), z_buf=state[0].detach().numpy(), r=state[2].numpy(),
        asc=state[3].detach().numpy(), psc_rise=state[4].detach().numpy(),
        psc=state[5].detach().numpy(),
        dw_rec=cell.recurrent_weight_values.grad.numpy(),
        dw_lgn=cell.input_weight_values.grad.numpy(), dw_bkg=cell.bkg_input_weights.grad.numpy(),
        pre_ind_order=cell.pre_ind_table.flat_values.numpy(),
        pre_ind_row_splits=cell.pre_ind_table.row_splits.numpy(), **extra,
        **{"kw_" + k: v for k, v in KW.items() if isinstance(v, float)})
    print("wrote", out, os.path.getsize(out), "bytes; spikes:", int(z.sum()))


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("V1_GLIF_REFERENCE", "V1_GLIF_model")
    models = load_reference_models(ref_root)
    only = sys.argv[2:]
    for name, spec in CASES.items():
        if not only or name in only:
            run_case(models, name, ref_root=ref_root, **spec)


if __name__ == "__main__":
    main()
