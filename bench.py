"""Benchmark of the V1 GLIF3 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A "step" is one data-parallel training step of the 66,634-neuron synthetic column
(benchmark configuration 4): forward rollout of T=500 ms at batch 5 per GPU, BPTT with the rate +
voltage + synchrony losses, one NCCL all-reduce of the flat fp32 weight-gradient buffer, an
Exp-Adam update of the recurrent and LGN weights.  ``value`` is simulated neuron-steps/s of that
whole step over all ranks with the inputs already on the device; ``e2e`` repeats it with the
step's inputs copied from pinned host memory and the loss read back every step.  At N=1 the line
also carries the forward-only number of configuration 3 (batch 5, T=2500) under ``fwd``.

``--impl reference`` times the CPU restatement of the reference's cell (oracle/, torch CPU ops on
all host threads; TensorFlow, which the reference itself needs, is not installable here) on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from v1_glif_model_b200 import synth  # noqa: E402

METRIC = "simulated neuron-steps/s, fwd+bwd training step at the 66k-neuron column"
UNIT = "neuron-steps/s"
LOSS = dict(rate_cost=100.0, voltage_cost=1e-3, sync_cost=1.0, fano_target=1.0, sync_bin=50)
CELL_KW = dict(dampening_factor=0.5, pseudo_width=0.5, recurrent_dampening_factor=0.5,
               voltage_gradient_dampening=0.5)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def fwd_bytes_per_launch(cnt, n, r, b, t):
    """Algorithmic bytes of one forward rollout: (31 + 24R + 25/B) per neuron-step for state,
    current accumulator and outputs, 9 B per delivered synapse event, 8 B per active source row."""
    dense = (31 + 24 * r + 25.0 / b) * n * b * t
    events = 9.0 * (cnt["rec_events"] + cnt["lgn_events"] + cnt["bkg_events"])
    rows = 8.0 * (cnt["rec_rows"] + cnt["lgn_rows"] + cnt["bkg_rows"])
    return dense + events + rows


def bwd_bytes_per_launch(cnt, n, r, b, t, nnz_rec):
    """Algorithmic bytes of one backward rollout: (37 + 24R + 25/B) per neuron-step, the
    recurrent synapse stream (9 B per synapse per step, shared by the batch) and 17 B per
    weight-gradient synapse event."""
    dense = (37 + 24 * r + 25.0 / b) * n * b * t
    return dense + 9.0 * nnz_rec * t + 17.0 * cnt["dw_events"]


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML, in-process, while the timed region
    runs (an `nvidia-smi` subprocess per sample stalls the driver for tens of ms and would itself
    perturb the measurement)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index, self.sm, self.bits, self.stop_flag, self.thread = index, [], 0, False, None
        self.max_mhz, self.handle, self.nv = None, None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = getattr(torch.cuda.get_device_properties(index), "uuid", None)
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nv = pynvml
        except Exception:
            self.nv = None

    def _sample(self):
        nv = self.nv
        self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
        try:
            self.bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
        except Exception:
            self.bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))

    def _run(self):
        while not self.stop_flag:
            try:
                self._sample()
            except Exception:
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nv is not None:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        reasons = sorted(name for bit, name in self.REASONS.items() if self.bits & bit)
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.sm), "source": "nvml" if self.nv else "unavailable"}


def loss_spec(cfg, cell_voltage_scale, device):
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)).to(device) / 1000.0
    vlo = torch.from_numpy((-20.0 / cell_voltage_scale).astype(np.float32)).to(device)
    return dict(LOSS, rate_target=tgt, v_lo=vlo)


# --------------------------------------------------------------------------------------
# CPU leg: the oracle restatement of the reference cell on the host cores
# --------------------------------------------------------------------------------------
def cpu_training_sample(cfg, dicts, t_sample, seed):
    """One fwd+bwd of `t_sample` steps at the configuration's batch on the CPU oracle."""
    from oracle.cell_torch import OracleV1Column
    from oracle import losses as OL
    torch.set_num_threads(os.cpu_count() or 1)
    orc = OracleV1Column(*dicts, **CELL_KW)
    x = torch.from_numpy(synth.make_lgn_spikes(cfg, cfg.batch, t_sample, seed))
    c = torch.from_numpy(synth.make_bkg_counts(cfg, cfg.batch, t_sample, seed)).long()
    vscale = orc.params["voltage_scale"][orc.params["node_type_ids"]]
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)) / 1000.0
    vlo = torch.from_numpy((-20.0 / vscale).astype(np.float32))

    def one():
        for w in (orc.recurrent_weight_values, orc.input_weight_values, orc.bkg_input_weights):
            w.grad = None
        t0 = time.perf_counter()
        z, v, _ = orc.rollout(x, c)
        total = OL.rate_loss(z, tgt, LOSS["rate_cost"]) + OL.voltage_loss(v, vlo, LOSS["voltage_cost"])
        if t_sample >= 2 * LOSS["sync_bin"]:
            total = total + OL.sync_loss(z, LOSS["sync_bin"], LOSS["sync_cost"])
        total.backward()
        return time.perf_counter() - t0
    return one


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = synth.CONFIGS[args.config]
    dicts = synth.make_network(cfg, 0)
    t_sample = args.cpu_sample_steps
    one = cpu_training_sample(cfg, dicts, t_sample, 0)
    for _ in range(args.warmup):
        one()
    times = [one() for _ in range(args.steps)]
    sec = float(np.mean(times))
    value = cfg.batch * cfg.n_neurons * t_sample / sec
    cores = torch.get_num_threads()
    sample = (f"fwd+bwd of {t_sample} of the {cfg.seq_len} simulated ms per step, batch {cfg.batch}, "
              f"N={cfg.n_neurons}; torch CPU restatement of the reference cell")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(cfg, args.gpus, t_sample),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "reference TensorFlow CPU path: unavailable on this box (TensorFlow not installed); "
                "the timed code is oracle/, the op-for-op restatement of v1_model_utils/models.py",
    }
    print(json.dumps(line))


def workload_config(cfg, n_gpus, t_len):
    return {"workload": f"{cfg.name}: {cfg.n_neurons:,}-neuron synthetic column, fwd+bwd training step "
                        "(rate+voltage+synchrony loss, Exp-Adam on recurrent+LGN weights)",
            "n_neurons": cfg.n_neurons, "batch_per_gpu": cfg.batch, "global_batch": cfg.batch * n_gpus,
            "seq_len": t_len, "n_receptors": cfg.n_receptors, "max_delay": cfg.max_delay,
            "parallelism": f"dp{n_gpus}",
            "l2": "inputs larger than L2 (saved rollout %.2f GB per step)" % (4e-9 * cfg.batch * cfg.n_neurons * t_len)}


# --------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist
    from v1_glif_model_b200.models import V1Column
    from v1_glif_model_b200.training import Trainer
    from v1_glif_model_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # stdout carries the JSON line only
        dist.init_process_group("nccl", device_id=dev)

    cfg = synth.CONFIGS[args.config]
    t_len = args.seq_len or cfg.seq_len
    b = cfg.batch
    dicts = synth.make_network(cfg, 0)
    cell = V1Column(*dicts, device=dev, **CELL_KW)
    lib = _lib.load()
    spec = loss_spec(cfg, cell.voltage_scale, dev)
    trainer = Trainer(cell, spec, learning_rate=1e-3, train_input=True, train_noise=False)
    # per-rank inputs (different seeds: the batch is sharded over ranks), pinned on the host
    x_host = torch.from_numpy(synth.make_lgn_spikes(cfg, b, t_len, seed=rank)).pin_memory()
    c_host = torch.from_numpy(synth.make_bkg_counts(cfg, b, t_len, seed=rank)).pin_memory()
    x_dev, c_dev = x_host.to(dev), c_host.to(dev)
    x_in, c_in = torch.empty_like(x_dev), torch.empty_like(c_dev)
    loss_host = torch.zeros(4).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def step_resident():
        trainer.step(x_dev, c_dev)

    def step_e2e():
        x_in.copy_(x_host, non_blocking=True)
        c_in.copy_(c_host, non_blocking=True)
        losses = trainer.step(x_in, c_in)
        loss_host.copy_(losses, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(max(args.warmup, 3)):
        step_resident()
    cell.synchronize()
    launches0 = lib.v1g_launch_count()
    fwd_ms, bwd_ms = [], []

    def step_probe():
        step_resident()
        fwd_ms.append(cell.last_kernel_ms(0))
        bwd_ms.append(cell.last_kernel_ms(1))

    with ClockSampler(local_rank) as clocks:
        total_ms = timed(step_probe if args.probe_kernels else step_resident, args.steps)
    launches = lib.v1g_launch_count() - launches0
    cell.synchronize()
    cnt = cell.counters()
    if not fwd_ms:  # kernel-only durations from one extra step outside the timed region
        step_resident()
        fwd_ms.append(cell.last_kernel_ms(0))
        bwd_ms.append(cell.last_kernel_ms(1))
        cnt = cell.counters()
    for _ in range(2):
        step_e2e()
    e2e_ms = timed(step_e2e, args.steps)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    n, r = cfg.n_neurons, cfg.n_receptors
    ns_per_step = world * b * n * t_len
    ms_per_step = total_ms / args.steps
    value = ns_per_step / (ms_per_step * 1e-3)
    peak, peak_kind = measured_peaks()
    nnz_rec = cell.recurrent_weight_values.numel()
    bb = bwd_bytes_per_launch(cnt, n, r, b, t_len, nnz_rec)
    fb = fwd_bytes_per_launch(cnt, n, r, b, t_len)
    bwd_s, fwd_s = float(np.mean(bwd_ms)) * 1e-3, float(np.mean(fwd_ms)) * 1e-3
    traffic = load_traffic(t_len)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, world, t_len),
        "e2e": {"value": ns_per_step / (e2e_ms / args.steps * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": int(x_host.numel() + c_host.numel() * 4),
                "d2h_bytes_per_step": 16},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "kernel": "rollout_bwd_kernel", "achieved": bb / bwd_s / 1e9,
                     "peak": peak, "peak_source": peak_kind, "unit": "GB/s",
                     "frac": bb / bwd_s / 1e9 / peak, "traffic": traffic.get("rollout_bwd_kernel"),
                     "algorithmic_bytes_per_launch": bb, "kernel_ms": bwd_s * 1e3},
        "roofline_fwd_kernel": {"bound": "hbm", "kernel": "rollout_fwd_reg_kernel",
                                "achieved": fb / fwd_s / 1e9, "peak": peak, "unit": "GB/s",
                                "frac": fb / fwd_s / 1e9 / peak,
                                "traffic": traffic.get("rollout_fwd_reg_kernel"),
                                "algorithmic_bytes_per_launch": fb, "kernel_ms": fwd_s * 1e3},
        "mean_rate_hz": cnt["spikes"] / (b * n * t_len) * 1000.0,
        "events_per_step": {k: cnt[k] / t_len for k in ("rec_events", "lgn_events", "bkg_events",
                                                        "dw_events", "bwd_events")},
    }
    if world == 1 and not args.no_fwd and args.config == "C4":
        line["fwd"] = forward_only(cell, lib, dev, args)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(cfg, dicts, args)
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def forward_only(cell, lib, dev, args):
    """Configuration 3: forward-only rollout, batch 5, T=2500, zero initial state."""
    cfg = synth.CONFIGS["C3"]
    t_len = args.fwd_seq_len or cfg.seq_len
    b, n, r = cfg.batch, cfg.n_neurons, cfg.n_receptors
    x_host = synth.make_lgn_spikes(cfg, b, t_len, seed=0)
    c_host = synth.make_bkg_counts(cfg, b, t_len, seed=0)
    x_dev, c_dev = torch.from_numpy(x_host).to(dev), torch.from_numpy(c_host).to(dev)
    z = torch.empty((b, t_len, n), dtype=torch.uint8, device=dev)
    v = torch.empty((b, t_len, n), dtype=torch.float32, device=dev)
    import ctypes as C
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def fwd():
        cell._check(lib.v1g_rollout_fwd(cell._libh, b, t_len, x_dev.data_ptr(), c_dev.data_ptr(), None,
                                        z.data_ptr(), v.data_ptr(), 0, stream))
    for _ in range(3):
        fwd()
    cell.synchronize()
    reps = max(3, args.steps)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kms = []
    e0.record()
    for _ in range(reps):
        fwd()
    e1.record()
    cell.synchronize()
    ms = e0.elapsed_time(e1) / reps
    kms.append(cell.last_kernel_ms(0))
    cnt = cell.counters()
    # end to end through the host-buffer entry point: spikes come back as uint8
    zh = np.empty((b, t_len, n), dtype=np.uint8)
    t0 = time.perf_counter()
    for _ in range(2):
        cell._check(lib.v1g_rollout_fwd_host(cell._libh, b, t_len, x_host.ctypes.data,
                                             c_host.ctypes.data, zh.ctypes.data, None, 0, stream))
    e2e_s = (time.perf_counter() - t0) / 2
    peak, _ = measured_peaks()
    fb = fwd_bytes_per_launch(cnt, n, r, b, t_len)
    ns = b * n * t_len
    return {"workload": "C3: forward only, batch 5, T=%d, z (uint8) and v (f32) written" % t_len,
            "value": ns / (ms * 1e-3), "unit": UNIT, "ms_per_rollout": ms,
            "us_per_simulated_ms": ms * 1e3 / t_len,
            "e2e": {"value": ns / e2e_s, "unit": UNIT, "h2d_bytes": int(x_host.nbytes + c_host.nbytes),
                    "d2h_bytes": int(zh.nbytes), "note": "pageable host buffers through v1g_rollout_fwd_host"},
            "roofline": {"bound": "hbm", "kernel": "rollout_fwd_reg_kernel",
                         "achieved": fb / (kms[0] * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": fb / (kms[0] * 1e-3) / 1e9 / peak, "kernel_ms": kms[0],
                         "algorithmic_bytes_per_launch": fb,
                         "traffic": load_traffic(t_len).get("rollout_fwd_reg_kernel")},
            "mean_rate_hz": cnt["spikes"] / ns * 1000.0}


def cpu_baseline(cfg, dicts, args):
    t_sample = args.cpu_sample_steps
    one = cpu_training_sample(cfg, dicts, t_sample, 0)
    one()
    sec = one()
    return {"value": cfg.batch * cfg.n_neurons * t_sample / sec, "unit": UNIT,
            "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"fwd+bwd of {t_sample} of the {cfg.seq_len} simulated ms, batch {cfg.batch}, "
                      f"N={cfg.n_neurons}, torch CPU restatement of the reference cell (oracle/)"}


def load_traffic(t_len=1):
    """DRAM bytes per launch from the committed ncu captures (measured per simulated step on a
    T=100 case; the kernels' traffic is proportional to T)."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if os.path.exists(path):
        with open(path) as f:
            per_step = json.load(f).get("per_step_bytes", {})
        return {k: v * t_len for k, v in per_step.items()}
    return {}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="C4", choices=["C4", "C5", "C2"],
                    help="C4 = the metric's configuration (default); C5 = 230,924-neuron stress; C2 = 5,000 neurons")
    ap.add_argument("--seq-len", type=int, default=0, help="override T of the training step")
    ap.add_argument("--fwd-seq-len", type=int, default=0, help="override T of the forward-only leg")
    ap.add_argument("--cpu-sample-steps", type=int, default=6)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fwd", action="store_true")
    ap.add_argument("--probe-kernels", action="store_true",
                    help="read per-kernel event times inside the timed loop (adds a sync per step)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
