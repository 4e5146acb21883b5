"""The network reader (``v1_glif_model_b200/load_sparse.py``, mirror of the reference's
``v1_model_utils/load_sparse.py``) on a synthetic SONATA-like table: node selection, per-type
parameters, the post-major synapse order, the dictionary schema, the ``.npz`` round trip, and the way
back from trained weights to the edge file's order (``checkpoint_to_edges.py``)."""
import os

import numpy as np
import pytest

from v1_glif_model_b200 import load_sparse, synth


def _tables(seed=0, n=300, n_types=7, n_edge_types=23):
    """A network as the reference's pickle holds it: nodes grouped by type under BMTK ids that are a
    permutation of the positions, edges grouped by edge type in arbitrary order."""
    rng = np.random.Generator(np.random.PCG64(seed))
    type_of = rng.integers(0, n_types, n)
    params = [dict(V_th=-40.0 - i, g=4.0 + i, E_L=-70.0 - i, k=[0.003 * (i + 1), 0.03], C_m=60.0 + i,
                   V_reset=-70.0 - i, t_ref=1.0 + 0.3 * i, asc_amps=[-6.0 - i, 20.0 + i]) for i in range(n_types)]
    nodes = [dict(ids=np.nonzero(type_of == i)[0].astype(np.uint32), params=params[i]) for i in range(n_types)]
    m = 4000
    src, tgt = rng.integers(0, n, m), rng.integers(0, n, m)
    et = rng.integers(0, n_edge_types, m)
    edges = []
    for e in range(n_edge_types):
        sel = np.nonzero(et == e)[0]
        edges.append(dict(source=src[sel].astype(np.uint64), target=tgt[sel].astype(np.uint64), edge_type_id=100 + e,
                          params=dict(delay=1.0 + (e % 4) * 0.5, syn_id=e % 5, weight=rng.normal(0, 1, sel.size))))
    node_table = dict(x=rng.uniform(-800, 800, n), y=rng.uniform(0, 900, n), z=rng.uniform(-800, 800, n),
                      tuning_angle=rng.uniform(0, 360, n), node_type_id=(1000 + type_of))
    return dict(nodes=nodes, edges=edges), node_table, type_of, (src, tgt, et)


def test_sort_indices_is_the_reference_order():
    rng = np.random.default_rng(0)
    idx = rng.integers(0, 50, (500, 2)).astype(np.int32)
    w = rng.normal(size=500)
    si, sw = load_sparse.sort_indices(idx, w)
    key = si[:, 0].astype(np.int64) * (idx.max() + 1) + si[:, 1]
    assert np.all(np.diff(key) >= 0)
    assert sorted(map(tuple, np.c_[si, sw])) == sorted(map(tuple, np.c_[idx, w]))


def test_load_network_selection_schema_and_order(tmp_path):
    dat, node_table, type_of, (src, tgt, et) = _tables()
    net = load_sparse.load_network(dat, node_table, n_neurons=120, connected_selection=True)
    assert set(net) >= {"x", "y", "z", "tuning_angle", "node_type_id", "n_nodes", "n_edges", "node_params",
                        "node_type_ids", "synapses", "tf_id_to_bmtk_id", "bmtk_id_to_tf_id"}
    assert set(net["synapses"]) == {"indices", "weights", "delays", "syn_ids", "edge_type_ids", "dense_shape"}
    assert net["n_nodes"] == 120 and net["synapses"]["dense_shape"] == (120, 120)
    # the 120 nodes closest to the origin, in BMTK order
    r = np.sqrt(node_table["x"] ** 2 + node_table["z"] ** 2)
    chosen = np.sort(np.argsort(r, kind="stable")[:120])
    assert np.array_equal(net["tf_id_to_bmtk_id"], chosen)
    assert np.array_equal(net["node_type_ids"], type_of[chosen])
    assert np.allclose(net["node_params"]["C_m"][type_of[chosen]], 60.0 + type_of[chosen])
    # exactly the edges with both ends inside, post-major
    inside = np.isin(src, chosen) & np.isin(tgt, chosen)
    assert net["n_edges"] == int(inside.sum())
    idx = net["synapses"]["indices"]
    key = idx[:, 0].astype(np.int64) * (idx.max() + 1) + idx[:, 1]
    assert np.all(np.diff(key) >= 0)
    assert net["synapses"]["weights"].dtype == np.float32 and net["synapses"]["delays"].dtype == np.float16
    assert net["synapses"]["syn_ids"].dtype == np.uint8 and net["synapses"]["edge_type_ids"].dtype == np.uint16
    back = net["tf_id_to_bmtk_id"][idx]
    want = sorted(zip(tgt[inside].tolist(), src[inside].tolist(), (100 + et[inside]).tolist()))
    assert sorted(zip(back[:, 0].tolist(), back[:, 1].tolist(), net["synapses"]["edge_type_ids"].tolist())) == want
    with pytest.raises(ValueError, match="There are only 300 neurons"):
        load_sparse.load_network(dat, node_table, n_neurons=301)
    core = load_sparse.load_network(dat, node_table, n_neurons=20, connected_selection=False, core_only=True, seed=1)
    assert core["n_nodes"] == 20 and np.all(r[core["tf_id_to_bmtk_id"]] < 400)
    # the .npz form of the pickle gives the same network
    path = os.path.join(tmp_path, "network_dat.npz")
    load_sparse.save_network_dat(path, dat)
    again = load_sparse.load_network(load_sparse.load_network_dat(path), node_table, n_neurons=120)
    assert np.array_equal(again["synapses"]["indices"], idx)
    assert np.array_equal(again["synapses"]["weights"], net["synapses"]["weights"])


def test_load_input_keeps_edges_into_the_selection():
    dat, node_table, _, _ = _tables(seed=2)
    net = load_sparse.load_network(dat, node_table, n_neurons=100)
    rng = np.random.default_rng(3)
    edges = [dict(source=rng.integers(0, 40, 600), target=rng.integers(0, 300, 600),
                  params=dict(delay=1.0, syn_id=k, weight=rng.uniform(0, 2, 600))) for k in range(3)]
    lgn = load_sparse.load_input(dict(edges=edges), net["bmtk_id_to_tf_id"], n_input=40)
    assert set(lgn) == {"n_inputs", "indices", "weights", "delays", "syn_ids"} and lgn["n_inputs"] == 40
    assert lgn["indices"][:, 0].max() < 100 and lgn["indices"][:, 1].max() < 40
    n_in = sum(int((net["bmtk_id_to_tf_id"][e["target"]] >= 0).sum()) for e in edges)
    assert lgn["indices"].shape[0] == n_in
    key = lgn["indices"][:, 0].astype(np.int64) * (lgn["indices"].max() + 1) + lgn["indices"][:, 1]
    assert np.all(np.diff(key) >= 0)


def test_checkpoint_weights_return_to_edge_file_order():
    """``checkpoint_to_edges.py``: weights x voltage scale of the target, back in the edge file's order."""
    rng = np.random.default_rng(5)
    n, m = 80, 2000
    file_idx = np.stack([rng.integers(0, n, m), rng.integers(0, n, m)], 1).astype(np.int64)   # (target, source)
    file_w = rng.normal(0, 1, m)
    scale = rng.uniform(15, 30, n)
    sorted_idx, sorted_w = load_sparse.sort_indices(file_idx, file_w)
    cell_w = (sorted_w / scale[sorted_idx[:, 0]]).astype(np.float32)       # what V1Column holds
    out = load_sparse.checkpoint_weights_to_edges(cell_w, scale, sorted_idx, file_idx)
    assert out.dtype == np.float64 and np.allclose(out, file_w, rtol=1e-6, atol=1e-7)
    assert np.mean(out * file_w < 0) == 0.0                                # the reference's own sign check


def test_load_basis_forms(tmp_path):
    tau = np.array([1.0, 2.0, 4.0])
    rows = {2: [0.1, 0.2, 0.3], 0: [1.0, 0.0, -0.5], 1: [0.0, 1.0, 0.0]}
    t, b = load_sparse.load_basis(tau, rows)
    assert b.shape == (3, 3) and np.allclose(b[0], rows[0]) and np.allclose(b[2], rows[2])
    csv = os.path.join(tmp_path, "w.csv")
    with open(csv, "w") as f:
        f.write("connection_name,w0,w1,w2\na,1,0,-0.5\nb,0,1,0\n")
    net = {}
    load_sparse.load_basis(tau, csv, network=net)
    assert net["synaptic_basis_weights"].shape == (2, 3) and net["tau_syn"].tolist() == [1.0, 2.0, 4.0]
    with pytest.raises(ValueError):
        load_sparse.load_basis(tau, np.zeros((4, 2)))
