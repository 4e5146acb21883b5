"""Shared helpers of the parity tests: build the oracle and the CUDA cell from the same dicts."""
import dataclasses

import numpy as np
import torch

from v1_glif_model_b200 import synth

# Tolerances of the parity contract: currents and state within 1e-5, gradients within 1e-4,
# relative to the largest magnitude of the reference tensor; indices and spikes bit-exact.
TOL_STATE = 1e-5
TOL_GRAD = 1e-4


def rel_err(a, b):
    a = torch.as_tensor(a, dtype=torch.float64).cpu()
    b = torch.as_tensor(b, dtype=torch.float64).cpu()
    denom = float(b.abs().max())
    if denom == 0.0:
        return float((a - b).abs().max())
    return float((a - b).abs().max()) / denom


def make_case(name, seed=0, dense_basis=False, n_receptors=None, **cell_kwargs):
    """(cfg, dicts, oracle cell, inputs) for a synthetic configuration."""
    from oracle.cell_torch import OracleV1Column
    cfg = synth.CONFIGS[name]
    if n_receptors is not None:
        cfg = dataclasses.replace(cfg, n_receptors=n_receptors)
    net, lgn, bkg = synth.make_network(cfg, seed)
    if dense_basis:
        # a dense [S, R] basis with negative entries, S > R, like the reference's fitted table
        rng = np.random.default_rng(seed + 1)
        s_types = 11
        net["synaptic_basis_weights"] = rng.normal(0.3, 0.6, (s_types, cfg.n_receptors)).astype(np.float32)
        for d in (net["synapses"], lgn, bkg):
            d["syn_ids"] = rng.integers(0, s_types, d["syn_ids"].shape[0]).astype(np.uint8)
    oracle = OracleV1Column(net, lgn, bkg, **cell_kwargs)
    return cfg, (net, lgn, bkg), oracle


def make_inputs(cfg, batch=None, seq_len=None, seed=0):
    b = batch or cfg.batch
    t = seq_len or cfg.seq_len
    x = synth.make_lgn_spikes(cfg, b, t, seed)
    c = synth.make_bkg_counts(cfg, b, t, seed)
    return x, c
