"""Host-side mirror of the reference's network loader: from the edge/node tables of a SONATA network
to the three dictionaries ``V1Column`` consumes, and back from trained weights to the edge file's
order.

=================================  ======================================================
here                               reference
=================================  ======================================================
``sort_indices``                   ``v1_model_utils/load_sparse.py:15-22``
``load_network``                   ``load_sparse.py:153-379`` (selection of the nodes, per-type
                                   parameters, edges -> post-major sorted arrays, dict schema ``:364-377``)
``load_input``                     ``load_sparse.py:382-471`` (schema ``:464-470``)
``load_basis``                     ``models.py:518-519, 617-622`` + ``load_sparse.py:77-97``
``checkpoint_weights_to_edges``    ``v1_model_utils/checkpoint_to_edges.py:47-117``
=================================  ======================================================

The reference reads its tables from ``network_dat.pkl`` (a pickle of ``{'nodes': [...], 'edges': [...]}``
that ``create_network_dat`` writes from the SONATA files with h5py/bmtk) and the node positions from
``v1_nodes.h5``.  Neither library is needed here: the functions take the same Python structures
directly, and ``save_network_dat`` / ``load_network_dat`` keep them in a plain ``.npz`` file, the
form in which a network leaves a machine that does have h5py.  Nothing here touches the GPU.
"""
from __future__ import annotations

import numpy as np

NODE_PARAM_KEYS = ("V_th", "g", "E_L", "k", "C_m", "V_reset", "t_ref", "asc_amps")


def sort_indices(indices, *arrays):
    """Post-major order: sort by ``post * max_ind + pre`` (``load_sparse.py:15-22``).  The sort is
    stable, so synapses with the same (post, pre) keep their listed order."""
    indices = np.asarray(indices)
    max_ind = int(np.max(indices)) + 1 if indices.size else 1
    if np.iinfo(indices.dtype).max < max_ind * (max_ind + 1):
        indices = indices.astype(np.int64)
    q = indices[:, 0] * max_ind + indices[:, 1]
    sorted_ind = np.argsort(q, kind="stable")
    return tuple(np.asarray(arr)[sorted_ind] for arr in (indices, *arrays))


def _select_nodes(node_table, n_nodes, n_neurons, core_only, connected_selection, seed):
    """Boolean selection of the network's nodes, the reference's four rules (``load_sparse.py:236-266``)."""
    rd = np.random.RandomState(seed=seed)
    x, z = np.asarray(node_table["x"], np.float32), np.asarray(node_table["z"], np.float32)
    r = np.sqrt(x ** 2 + z ** 2)
    if n_neurons > n_nodes:
        raise ValueError(f"There are only {n_nodes} neurons in the network")
    if connected_selection:      # the n_neurons nodes closest to the origin
        sorted_ind = np.argsort(r, kind="stable")
        sel = np.zeros(n_nodes, dtype=np.bool_)
        sel[sorted_ind[:n_neurons]] = True
    elif core_only:              # a random draw from the core (radius below 400 um)
        sel = r < 400
        n_core = int(np.sum(sel))
        if n_neurons > n_core:
            raise ValueError(f"There are only {n_core} neurons in the network core")
        if 0 < n_neurons <= n_core:
            (inds,) = np.where(sel)
            take = rd.choice(inds, size=n_neurons, replace=False)
            sel[:] = False
            sel[take] = True
    elif 0 < n_neurons <= n_nodes:
        take = rd.choice(np.arange(n_nodes), size=n_neurons, replace=False)
        sel = np.zeros(n_nodes, dtype=np.bool_)
        sel[take] = True
    else:
        sel = np.ones(n_nodes, dtype=np.bool_)
    return sel


def load_network(network_dat, node_table, core_only=True, n_neurons=296991, seed=3000,
                 connected_selection=True, random_weights=False, uniform_weights=False):
    """The ``network`` dictionary of ``load_sparse.load_network`` (``:153-379``).

    ``network_dat``: ``{'nodes': [{'ids', 'params'}...], 'edges': [{'source', 'target', 'edge_type_id',
    'params': {'delay', 'syn_id', 'weight'}}...]}`` as in the reference's pickle; ``node_table``: the
    arrays the reference reads from ``v1_nodes.h5`` (``x, y, z, tuning_angle, node_type_id``).
    """
    d = network_dat
    n_nodes = sum(len(a["ids"]) for a in d["nodes"])
    if n_neurons <= 0:
        n_neurons = n_nodes
    tf_id_to_bmtk_id = np.arange(n_nodes, dtype=np.int32)
    bmtk_id_to_tf_id = np.full(n_nodes, -1, dtype=np.int32)
    sel = _select_nodes(node_table, n_nodes, n_neurons, core_only, connected_selection, seed)
    n_nodes = int(np.sum(sel))
    tf_id_to_bmtk_id = tf_id_to_bmtk_id[sel]
    bmtk_id_to_tf_id[tf_id_to_bmtk_id] = np.arange(n_nodes, dtype=np.int32)

    n_node_types = len(d["nodes"])
    node_params = {k: np.empty((n_node_types, 2) if k in ("k", "asc_amps") else n_node_types, np.float32)
                   for k in NODE_PARAM_KEYS}
    node_type_ids = np.empty(n_nodes, np.int32)
    for i, node_type in enumerate(d["nodes"]):
        tf_ids = bmtk_id_to_tf_id[np.asarray(node_type["ids"], dtype=np.int32)]
        node_type_ids[tf_ids[tf_ids >= 0]] = i
        for k, v in node_params.items():
            v[i] = node_type["params"][k]

    indices, weights, delays, syn_ids, edge_type_ids = [], [], [], [], []
    for edge in d["edges"]:
        target = bmtk_id_to_tf_id[np.asarray(edge["target"], dtype=np.int64)]
        source = bmtk_id_to_tf_id[np.asarray(edge["source"], dtype=np.int64)]
        exists = np.logical_and(target != -1, source != -1)
        target, source = target[exists], source[exists]
        w = np.asarray(edge["params"]["weight"])[exists].astype(np.float32)
        if random_weights:
            np.random.shuffle(w)
        n_new = len(target)
        indices.append(np.array([target, source]).T.reshape(-1, 2))
        weights.append(w)
        delays.append(np.full(n_new, edge["params"]["delay"], dtype=np.float16))
        syn_ids.append(np.full(n_new, edge["params"]["syn_id"], dtype=np.uint8))
        edge_type_ids.append(np.full(n_new, edge["edge_type_id"], dtype=np.uint16))
    indices = np.concatenate(indices, axis=0).astype(np.int32) if indices else np.zeros((0, 2), np.int32)
    cat = lambda parts, dt: np.concatenate(parts, axis=0).astype(dt) if parts else np.zeros((0,), dt)
    weights, delays = cat(weights, np.float32), cat(delays, np.float16)
    syn_ids, edge_type_ids = cat(syn_ids, np.uint8), cat(edge_type_ids, np.uint16)
    if uniform_weights:
        weights[weights > 0] = np.mean(weights[weights > 0])
        weights[weights < 0] = np.mean(weights[weights < 0])
    n_edges = int(indices.shape[0])
    if n_edges:
        indices, weights, delays, syn_ids, edge_type_ids = sort_indices(indices, weights, delays, syn_ids,
                                                                        edge_type_ids)
    take = lambda key, dt: np.asarray(node_table[key], dtype=dt)[sel]
    return dict(
        x=take("x", np.float32), y=take("y", np.float32), z=take("z", np.float32),
        tuning_angle=take("tuning_angle", np.float32), node_type_id=take("node_type_id", np.int32),
        n_nodes=n_nodes, n_edges=n_edges, node_params=node_params, node_type_ids=node_type_ids,
        synapses=dict(indices=indices, weights=weights, delays=delays, syn_ids=syn_ids,
                      edge_type_ids=edge_type_ids, dense_shape=(n_nodes, n_nodes)),
        tf_id_to_bmtk_id=tf_id_to_bmtk_id, bmtk_id_to_tf_id=bmtk_id_to_tf_id)


def load_input(input_dat, bmtk_id_to_tf_id=None, n_input=17400):
    """An input population (LGN or background) as ``load_sparse.load_input`` returns it (``:382-471``):
    only edges whose target is in the selection are kept; the sources keep their own numbering."""
    post, pre, weights, delays, syn_ids = [], [], [], [], []
    for edge in input_dat["edges"]:
        target = np.asarray(edge["target"]).astype(np.int32)
        source = np.asarray(edge["source"]).astype(np.int32)
        w = np.asarray(edge["params"]["weight"]).astype(np.float32)
        n_new = len(target)
        d = np.full(n_new, edge["params"]["delay"], dtype=np.float16)
        s = np.full(n_new, edge["params"]["syn_id"], dtype=np.uint8)
        if bmtk_id_to_tf_id is not None:
            target = np.asarray(bmtk_id_to_tf_id)[target]
            exists = target != -1
            target, source, w, d, s = target[exists], source[exists], w[exists], d[exists], s[exists]
        post.append(target), pre.append(source), weights.append(w), delays.append(d), syn_ids.append(s)
    cat = lambda parts, dt: np.concatenate(parts, axis=0).astype(dt) if parts else np.zeros((0,), dt)
    indices = np.stack([cat(post, np.int32), cat(pre, np.int32)], -1)
    weights, delays, syn_ids = cat(weights, np.float32), cat(delays, np.float16), cat(syn_ids, np.uint8)
    if indices.shape[0]:
        indices, weights, delays, syn_ids = sort_indices(indices, weights, delays, syn_ids)
    return dict(n_inputs=n_input, indices=indices, weights=weights, delays=delays, syn_ids=syn_ids)


def load_basis(tau_basis, basis_weights, network=None):
    """The two synaptic-basis tables the reference's ``V1Column`` reads from files: the time constants
    of the receptor basis (``synaptic_data/tau_basis.npy``, ``models.py:518-519``) and one row of basis
    weights per synapse type (``syn_id_to_syn_weights_dict.pkl``, ``models.py:617-622``, whose rows come
    from ``synaptic_data/basis_function_weights.csv``, ``load_sparse.py:77-97``).  ``tau_basis``: array or
    ``.npy`` path; ``basis_weights``: ``[S, R]`` array, ``{syn_id: row}`` dictionary, or the ``.csv`` path
    (rows in file order).  With ``network`` given, both are stored in it under the keys
    ``v1_glif_model_b200.models.V1Column`` expects."""
    tau = np.load(tau_basis) if isinstance(tau_basis, str) else np.asarray(tau_basis)
    if isinstance(basis_weights, str):
        rows = [line.strip().split(",") for line in open(basis_weights) if line.strip()]
        basis = np.array([[float(v) for v in r[1:]] for r in rows[1:]], dtype=np.float32)
    elif isinstance(basis_weights, dict):
        basis = np.array([basis_weights[k] for k in sorted(basis_weights)], dtype=np.float32)
    else:
        basis = np.asarray(basis_weights, dtype=np.float32)
    if basis.ndim != 2 or basis.shape[1] != tau.size:
        raise ValueError(f"basis weights must be [S, {tau.size}], got {basis.shape}")
    if network is not None:
        network["tau_syn"] = np.asarray(tau, dtype=np.float64)
        network["synaptic_basis_weights"] = basis
    return np.asarray(tau, dtype=np.float64), basis


def save_network_dat(path, dat):
    """Flatten a ``{'nodes': [...], 'edges': [...]}`` structure (``network_dat.pkl`` / ``*_input_dat.pkl``)
    into one ``.npz`` file of plain arrays."""
    out = {"n_nodes": len(dat.get("nodes", [])), "n_edges": len(dat["edges"])}
    for i, node in enumerate(dat.get("nodes", [])):
        out[f"node{i}_ids"] = np.asarray(node["ids"])
        for k in NODE_PARAM_KEYS:
            out[f"node{i}_{k}"] = np.asarray(node["params"][k], dtype=np.float64)
    for i, edge in enumerate(dat["edges"]):
        out[f"edge{i}_source"] = np.asarray(edge["source"])
        out[f"edge{i}_target"] = np.asarray(edge["target"])
        out[f"edge{i}_weight"] = np.asarray(edge["params"]["weight"])
        out[f"edge{i}_meta"] = np.array([edge["params"]["delay"], edge["params"]["syn_id"],
                                         edge.get("edge_type_id", i)], dtype=np.float64)
    np.savez_compressed(path, **out)


def load_network_dat(path):
    f = np.load(path)
    nodes = [dict(ids=f[f"node{i}_ids"], params={k: f[f"node{i}_{k}"] for k in NODE_PARAM_KEYS})
             for i in range(int(f["n_nodes"]))]
    edges = []
    for i in range(int(f["n_edges"])):
        delay, syn_id, type_id = f[f"edge{i}_meta"]
        edges.append(dict(source=f[f"edge{i}_source"], target=f[f"edge{i}_target"], edge_type_id=int(type_id),
                          params=dict(delay=float(delay), syn_id=int(syn_id), weight=f[f"edge{i}_weight"])))
    return dict(nodes=nodes, edges=edges)


def checkpoint_weights_to_edges(recurrent_weights, voltage_scale, recurrent_indices, edge_file_indices):
    """Trained recurrent weights back in the order of the SONATA edge file
    (``checkpoint_to_edges.py:47-117``): multiply by the voltage scale of the target neuron, then undo
    the post-major sort that ``load_network`` applied to the file's ``(target, source)`` rows.

    ``recurrent_weights[nnz]``: the cell's weights in its own (sorted) order, e.g. after
    ``Trainer.weights()``; ``voltage_scale[N]`` per neuron; ``recurrent_indices[nnz, 2]`` the cell's
    ``(post, pre_delayed)`` rows (only the post column is used); ``edge_file_indices[nnz, 2]`` the edge
    file's ``(target, source)`` rows in file order.  Returns float64 weights in file order."""
    w = np.asarray(recurrent_weights, dtype=np.float32).reshape(-1)
    scale = np.asarray(voltage_scale)[np.asarray(recurrent_indices)[:, 0]]
    sorted_w = (w * scale).astype(np.float64)
    (sorted_ind,) = (np.argsort(_sort_key(np.asarray(edge_file_indices)), kind="stable"),)
    revert = np.argsort(sorted_ind, kind="stable")
    return sorted_w[revert]


def _sort_key(indices):
    max_ind = int(np.max(indices)) + 1
    if np.iinfo(indices.dtype).max < max_ind * (max_ind + 1):
        indices = indices.astype(np.int64)
    return indices[:, 0] * max_ind + indices[:, 1]
