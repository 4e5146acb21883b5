"""Writes tests/golden/tiny_rollout.npz from the fp64 oracle (run from the repo root):

    python tests/golden/make_golden.py

The reference ships no golden vectors for this path and cannot run without TensorFlow, so these
fixtures pin the oracle against itself over time (any change to oracle/ or to the synthetic
generator that alters a number shows up as a failure of tests/test_host_cpu.py).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from util import make_case, make_inputs  # noqa: E402
from oracle import losses as OL  # noqa: E402
from v1_glif_model_b200 import synth  # noqa: E402

KW = dict(dampening_factor=0.5, pseudo_width=0.5, recurrent_dampening_factor=0.5,
          voltage_gradient_dampening=0.5)
LOSS = dict(rate_cost=10.0, voltage_cost=1e-1, sync_cost=0.5, fano_target=1.0, sync_bin=10)


def main():
    cfg, dicts, orc = make_case("tiny", dtype=torch.float64, **KW)
    x, c = make_inputs(cfg)
    z, v, state = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    vscale = (dicts[0]["node_params"]["V_th"] - dicts[0]["node_params"]["E_L"])[dicts[0]["node_type_ids"]]
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)).double() / 1000.0
    vlo = torch.from_numpy(-20.0 / vscale)
    loss = (OL.rate_loss(z, tgt, LOSS["rate_cost"]) + OL.voltage_loss(v, vlo, LOSS["voltage_cost"]) +
            OL.sync_loss(z, LOSS["sync_bin"], LOSS["sync_cost"]))
    loss.backward()
    out = os.path.join(ROOT, "tests", "golden", "tiny_rollout.npz")
    np.savez_compressed(
        out, x=x, bkg_counts=c, z=z.detach().numpy().astype(np.uint8), v=v.detach().numpy(),
        psc=state[5].detach().numpy(), psc_rise=state[4].detach().numpy(),
        asc=state[3].detach().numpy(), r=state[2].numpy(), z_buf=state[0].detach().numpy(),
        loss=np.float64(loss.item()),
        dw_rec=orc.recurrent_weight_values.grad.numpy(),
        dw_lgn=orc.input_weight_values.grad.numpy(), dw_bkg=orc.bkg_input_weights.grad.numpy())
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
