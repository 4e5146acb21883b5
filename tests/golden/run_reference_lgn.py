"""Golden vectors for the LGN front end from the reference's OWN code (run from the repo root, in a
container that has the reference tree):

    python tests/golden/run_reference_lgn.py /path/to/V1_GLIF_model

Imports ``lgn_model/lgn.py`` unmodified over ``tf_standin`` (bmtk, h5py and matplotlib, which only the
table-building constructor and the plotting ``main`` use, are replaced by empty modules), makes an ``LGN``
object without running the constructor (it reads the network's csv/h5 files and caches), gives it
synthetic tables of the shapes the constructor stores (``lgn.py:458-472``), and calls the two methods of the
hot path, ``spatial_response`` (``lgn.py:481-517``, with and without the bmtk edge normalisation) and
``firing_rates_from_spatial`` (``lgn.py:519-528``), on a seeded movie.  Writes
``tests/golden/reference_lgn.npz``; ``tests/test_lgn.py`` checks ``oracle/lgn.py`` and the device front end
against it.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import tf_standin  # noqa: E402

H, W, T, U = 24, 40, 60, 50
FILTER_SIDES = (3, 5, 9)
LEN_DOM, LEN_NON_DOM = 20, 17


def synthetic_tables(seed=5):
    """Tables of the shapes the reference's constructor stores: three spatial-size classes, positions that
    include frame corners and edges, exact pixel centres and fractional offsets; a third of the units composite."""
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.uniform(0, W - 1, U).astype(np.float32)
    y = rng.uniform(0, H - 1, U).astype(np.float32)
    x[:6] = [0.0, W - 1, 0.0, W - 1, 7.0, 0.25]
    y[:6] = [0.0, 0.0, H - 1, H - 1, 5.0, H - 1]
    ndx = np.clip(x + rng.normal(0, 3, U), 0, W - 1).astype(np.float32)
    ndy = np.clip(y + rng.normal(0, 3, U), 0, H - 1).astype(np.float32)
    unit_class = rng.integers(0, len(FILTER_SIDES), U)
    unit_class[:6] = [2, 2, 2, 2, 0, 1]
    filters, indices = [], []
    for c, side in enumerate(FILTER_SIDES):
        r = np.arange(side) - side // 2
        sigma = side / 6.0 + 0.3
        g = np.exp(-(r[:, None] ** 2 + r[None, :] ** 2) / (2 * sigma * sigma))
        filters.append((g / g.sum()).astype(np.float32)[..., None, None])
        indices.append(np.where(unit_class == c)[0].astype(np.int32))
    composite = (rng.random(U) < 0.35).astype(np.float32)
    tt = np.arange(LEN_DOM)[::-1, None].astype(np.float64)
    kd = (np.exp(-tt / rng.uniform(2, 6, U)) * np.cos(tt / rng.uniform(1.5, 5, U))).astype(np.float32)
    tn = np.arange(LEN_NON_DOM)[::-1, None].astype(np.float64)
    kn = (np.exp(-tn / rng.uniform(2, 6, U)) * np.sin(tn / rng.uniform(1.5, 5, U))).astype(np.float32) * composite
    return dict(x=x, y=y, non_dominant_x=ndx, non_dominant_y=ndy, gaussian_filters=filters,
                spatial_range_indices=indices, dom_temporal_kernels=kd, non_dom_temporal_kernels=kn,
                amplitude=rng.uniform(-3, 3, U).astype(np.float32),
                non_dom_amplitude=(rng.uniform(-3, 3, U) * composite).astype(np.float32),
                is_composite=composite, spontaneous_firing_rates=rng.uniform(0.5, 6, U).astype(np.float32))


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("V1_GLIF_REFERENCE", "V1_GLIF_model")
    tf = tf_standin.install()
    tf_standin.set_policy_dtype(torch.float32)
    for name in ("h5py", "matplotlib", "matplotlib.pyplot", "bmtk", "bmtk.simulator", "bmtk.simulator.filternet",
                 "bmtk.simulator.filternet.lgnmodel", "bmtk.simulator.filternet.lgnmodel.fitfuns",
                 "bmtk.simulator.filternet.lgnmodel.spatialfilter",
                 "bmtk.simulator.filternet.lgnmodel.temporalfilter",
                 "bmtk.simulator.filternet.lgnmodel.util_fns", "bmtk.simulator.filternet.lgnmodel.cellmetrics"):
        mod = types.ModuleType(name)
        for attr in ("makeBasis_StimKernel", "GaussianSpatialFilter", "TemporalFilterCosineBump",
                     "get_tcross_from_temporal_kernel", "get_data_metrics_for_each_subclass"):
            setattr(mod, attr, None)
        sys.modules.setdefault(name, mod)
    import tempfile
    os.environ.setdefault("NUMBA_CACHE_DIR", tempfile.mkdtemp(prefix="numba_cache_"))
    spec = importlib.util.spec_from_file_location("reference_lgn", os.path.join(ref_root, "lgn_model", "lgn.py"))
    ref = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = ref
    spec.loader.exec_module(ref)

    tb = synthetic_tables()
    lgn = object.__new__(ref.LGN)
    lgn.dtype = torch.float32
    for key in ("x", "y", "non_dominant_x", "non_dominant_y", "amplitude", "non_dom_amplitude", "is_composite",
                "spontaneous_firing_rates", "dom_temporal_kernels", "non_dom_temporal_kernels"):
        setattr(lgn, key, tf.constant(tb[key], dtype=torch.float32))
    lgn.gaussian_filters = [tf.convert_to_tensor(g, dtype=torch.float32) for g in tb["gaussian_filters"]]
    lgn.spatial_range_indices = tb["spatial_range_indices"]
    ids = np.concatenate(tb["spatial_range_indices"])
    lgn.sorted_neuron_ids_indices = tf.convert_to_tensor(np.argsort(ids).astype(np.int32), dtype=torch.int32)

    rng = np.random.Generator(np.random.PCG64(17))
    movie = rng.normal(0, 0.4, (T, H, W)).astype(np.float32)
    movie[10:30] += np.sin(np.arange(W) * 0.5)[None, None, :].astype(np.float32)   # a grating part
    movie = np.clip(movie, -1, 1)
    frames = torch.from_numpy(movie)[..., None]
    out = dict(movie=movie)
    for compat in (True, False):
        dom, non_dom = lgn.spatial_response(frames, bmtk_compat=compat)
        rates = lgn.firing_rates_from_spatial(dom, non_dom)
        tag = "" if compat else "_plain"
        out.update({"dom" + tag: dom.numpy(), "non_dom" + tag: non_dom.numpy(), "rates" + tag: rates.numpy()})
    for key, val in tb.items():
        if key == "gaussian_filters":
            for c, g in enumerate(val):
                out[f"gaussian_filter_{c}"] = g
        elif key == "spatial_range_indices":
            for c, idx in enumerate(val):
                out[f"spatial_range_indices_{c}"] = idx
        else:
            out[key] = val
    np.savez_compressed(os.path.join(HERE, "reference_lgn.npz"), **out)
    print({k: (v.shape, float(np.abs(v).mean())) for k, v in out.items() if k.startswith(("dom", "rates"))})


if __name__ == "__main__":
    main()
