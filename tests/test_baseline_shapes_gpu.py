"""GPU parity at the shapes of the benchmark configurations themselves (not only on the small
test nets): configuration 1 for all 200 steps, configuration 2 in full (5,000 neurons, batch 2,
T=500, rate + voltage loss, pseudo-derivative width 0.5, dampening 0.5) with its gradients and an
fp64 arbitration, the same net at batch 5 / T=500 with 24-bit and fp32 rows in the backward ring,
and the full-size 66,634-neuron column for a truncated rollout from a warmed-up state.

The oracle runs with ``scatter_transpose=True`` (the spike-gradient product as one scatter per
channel instead of a sparse tensor per channel and step; same terms, see
``tests/test_host_cpu.py::test_oracle_scatter_transpose_equals_sparse_matmul``) so that the
full-length reverse sweeps take tens of seconds on the host instead of minutes.
"""
import numpy as np
import pytest
import torch

from util import (TOL_STATE, assert_grad_close, cuda_loss_spec, first_spike_divergence, grad_metrics,
                  make_cells, make_inputs, oracle_loss_and_grads, rel_err, rel_l2, state_to_oracle)
from v1_glif_model_b200 import synth

pytestmark = pytest.mark.gpu
KW = dict(dampening_factor=0.5, pseudo_width=0.5, recurrent_dampening_factor=0.5,
          voltage_gradient_dampening=0.5)
# configuration 2: mean-squared error of the per-neuron rate (per ms) against lognormal targets and
# 1e-3 x the voltage penalty
LOSS_C2 = dict(rate_cost=100.0, voltage_cost=1e-3, sync_cost=0.0, fano_target=1.0, sync_bin=50)
NAMES = ("dW_rec", "dW_lgn", "dW_bkg")


def _gpu_run(cell, cfg, x, c, loss, state=None):
    z, v = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), state=state,
                        save_for_bwd=True)
    grads = cell.backward(cuda_loss_spec(cfg, cell, loss))
    cell.synchronize()
    return z, v, grads


def _check_forward(z, v, zo, vo):
    """Spikes exactly, voltages within the state bar; a proven threshold tie shortens the window."""
    t_tie = first_spike_divergence(z, zo, vo)
    t_ok = z.shape[1] if t_tie is None else t_tie
    assert t_ok >= 1
    assert rel_err(v[:, :t_ok], vo[:, :t_ok]) <= TOL_STATE
    return t_tie


def test_configuration_1_all_200_steps():
    cfg, dicts, orc, cell = make_cells("C1")
    x, c = make_inputs(cfg)
    assert x.shape[1] == 200
    with torch.no_grad():
        zo, vo, so = orc.rollout(torch.from_numpy(x), torch.from_numpy(c).long())
    state = cell.zero_state(cfg.batch)
    z, v = cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), state=state)
    cell.synchronize()
    t_tie = _check_forward(z, v, zo, vo)
    assert int(zo.sum()) > 1000
    if t_tie is None:
        assert torch.equal(state[0].cpu(), so[0]) and torch.equal(state[2].cpu().long(), so[2])
        for got, want in zip(state[3:6], so[3:6]):
            assert rel_err(got, want) <= TOL_STATE


def test_configuration_2_in_full_with_fp64_arbitration():
    """5,000 neurons, batch 2, T=500: spikes exact, v within 1e-5, the three weight gradients within
    1e-4 of the fp32 oracle (max-norm and relative L2) and, entry by entry above 1e-3 of the largest,
    within 1e-2; against the fp64 oracle the CUDA path must be no further away than a small multiple
    of the fp32 oracle's own distance to fp64."""
    cfg, dicts, orc, cell = make_cells("C2", scatter_transpose=True, **KW)
    x, c = make_inputs(cfg)
    assert x.shape[:2] == (2, 500)
    zo, vo, lo, go = oracle_loss_and_grads(orc, cfg, x, c, cell.voltage_scale, LOSS_C2)
    z, v, grads = _gpu_run(cell, cfg, x, c, LOSS_C2)
    t_tie = _check_forward(z, v, zo, vo)
    if t_tie is not None:
        pytest.skip(f"threshold tie at step {t_tie}: spikes and voltages agree up to it; the gradients of "
                    "two different spike trains are not comparable")
    assert abs(float(grads[3][0]) - lo) <= 1e-4 * abs(lo)
    got32 = {}
    for name, got, want in zip(NAMES, grads[:3], go):
        got32[name] = assert_grad_close(got, want, f"C2 {name} vs fp32 oracle")
    # fp64 arbitration: same spikes (checked), gradients in double precision
    from util import make_case
    _, _, orc64 = make_case("C2", dtype=torch.float64, scatter_transpose=True, **KW)
    z64, _, _, g64 = oracle_loss_and_grads(orc64, cfg, x, c, cell.voltage_scale, LOSS_C2)
    if not torch.equal(z64.float(), zo):
        pytest.skip("the fp64 oracle's spike train differs from the fp32 one (a rounding tie): no arbitration")
    for name, got, o32, o64 in zip(NAMES, grads[:3], go, g64):
        e_gpu, e_o32 = rel_l2(got, o64), rel_l2(o32, o64)
        print(f"[parity] C2 {name}: relative L2 to the fp64 oracle: CUDA {e_gpu:.3e}, fp32 oracle {e_o32:.3e}")
        assert e_gpu <= 1e-4, f"C2 {name}: relative L2 to the fp64 oracle {e_gpu:.3e}"
        assert e_gpu <= 4.0 * e_o32 + 2e-6, (f"C2 {name}: CUDA path is {e_gpu:.3e} from fp64, the fp32 "
                                             f"oracle itself {e_o32:.3e}")


def test_batch_5_full_length_reverse_sweep_with_packed_and_fp32_rows():
    """The benchmarked storage formats over a full-length reverse sweep: the configuration-2 net at
    batch 5, T=500, once with the 24-bit rows of the backward ring (and the two flag bits inside the
    saved voltages) and once with fp32 rows; both must meet the gradient bars, and the difference
    between the two is reported."""
    cfg, dicts, orc, cell = make_cells("C2", scatter_transpose=True, **KW)
    x, c = make_inputs(cfg, batch=5, seq_len=500)
    zo, vo, lo, go = oracle_loss_and_grads(orc, cfg, x, c, cell.voltage_scale, LOSS_C2)
    z, v, packed = _gpu_run(cell, cfg, x, c, LOSS_C2)
    t_tie = _check_forward(z, v, zo, vo)
    if t_tie is not None:
        pytest.skip(f"threshold tie at step {t_tie}")
    cell.set_option("pair_rows", 1)               # two steps per 32-byte ring row (24-bit values)
    _, _, paired = _gpu_run(cell, cfg, x, c, LOSS_C2)
    for name, gp, want in zip(NAMES, paired[:3], go):
        assert_grad_close(gp, want, f"B=5 T=500 {name}, paired 24-bit rows")
    cell.set_option("pair_rows", 0)
    cell.set_option("no_q_pack", 1)
    _, _, plain = _gpu_run(cell, cfg, x, c, LOSS_C2)
    report = {}
    for name, gp, gf, want in zip(NAMES, packed[:3], plain[:3], go):
        report[name] = (assert_grad_close(gp, want, f"B=5 T=500 {name}, 24-bit rows"),
                        assert_grad_close(gf, want, f"B=5 T=500 {name}, fp32 rows"), rel_l2(gp, gf))
    print("[parity] B=5 T=500 packed vs fp32 rows, relative L2:", {k: v[2] for k, v in report.items()})
    # the packed rows may cost accuracy, but only at the level of their own rounding (7.6e-6 per entry)
    assert report["dW_rec"][2] <= 5e-5, report


def test_full_size_column_truncated_from_a_warmed_up_state():
    """66,634 neurons, batch 5 (configurations 3 and 4): 100 steps on the GPU bring the column to its
    working regime, then 20 steps forward and backward (rate + voltage + synchrony loss) are compared
    with the oracle started from that same state."""
    loss = dict(rate_cost=100.0, voltage_cost=1e-3, sync_cost=1.0, fano_target=1.0, sync_bin=5)
    cfg, dicts, orc, cell = make_cells("C4", scatter_transpose=True, **KW)
    warm, t_len = 100, 20
    x, c = make_inputs(cfg, batch=cfg.batch, seq_len=warm + t_len)
    xg, cg = torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda()
    state = cell.zero_state(cfg.batch)
    cell.rollout(xg[:, :warm].contiguous(), cg[:, :warm].contiguous(), state=state, return_z=False, return_v=False)
    cell.synchronize()
    start = state_to_oracle(state)
    assert float(start[0].sum()) > 0          # spikes are travelling in z_buf
    zo, vo, lo, go = oracle_loss_and_grads(orc, cfg, x[:, warm:], c[:, warm:], cell.voltage_scale, loss, state=start)
    z, v, grads = _gpu_run(cell, cfg, np.ascontiguousarray(x[:, warm:]), np.ascontiguousarray(c[:, warm:]), loss,
                           state=state)
    rate_hz = float(zo.mean()) * 1000.0
    print(f"[parity] C4-size window: mean rate {rate_hz:.2f} Hz, {int(zo.sum())} spikes")
    assert rate_hz > 1.0, rate_hz
    t_tie = _check_forward(z, v, zo, vo)
    if t_tie is not None:
        pytest.skip(f"threshold tie at step {t_tie}")
    assert abs(float(grads[3][0]) - lo) <= 1e-4 * abs(lo)
    for name, got, want in zip(NAMES, grads[:3], go):
        assert_grad_close(got, want, f"C4-size T=20 {name}, 24-bit rows")
    # the same saved rollout through fp32 rows in the backward ring
    cell.set_option("no_q_pack", 1)
    plain = cell.backward(cuda_loss_spec(cfg, cell, loss))
    cell.synchronize()
    for name, got, want in zip(NAMES, plain[:3], go):
        assert_grad_close(got, want, f"C4-size T=20 {name}, fp32 rows", tol_elem=1e-3)
