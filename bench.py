"""Benchmark of the V1 GLIF3 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A "step" is one data-parallel training step of the 66,634-neuron synthetic column (benchmark
configuration 4): forward rollout of T=500 ms at batch 5 per GPU from a warmed-up carried state (the
reference starts every step from its gray-screen state, multi_training.py:812-831), BPTT with the
rate + voltage + synchrony losses, one NCCL all-reduce of the flat fp32 weight-gradient buffer, an
Exp-Adam update of the recurrent and LGN weights.  ``value`` is simulated neuron-steps/s of that whole
step over all ranks with the inputs already on the device; ``e2e`` repeats it with every step's LGN
spikes and background counts copied from pinned host memory (the copy of step k+1 runs on a second
stream while step k computes) and the losses read back every step; ``device_inputs`` repeats it with
both inputs drawn on the device from seeds.  At N=1 the line also carries the forward-only number of
configuration 3 (batch 5, T=2500) under ``fwd``; at N>=2 a ``stress`` record of configuration 5.

``--impl reference`` times the CPU restatement of the reference's cell (oracle/, torch CPU ops on all
host threads; TensorFlow, which the reference itself needs, is not installed here and its sources are
not present at run time) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
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
WARM_STEPS = 300          # simulated ms that bring the column from the zero state to its working regime
CPU_SECONDS_PER_STEP = 0.8  # oracle fwd+bwd per simulated ms at C4 on 16 threads, for sizing the CPU sample


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


def tensorflow_probe():
    """Whether the reference's own TensorFlow path could be driven here (it never can on a box
    without the reference's sources, but the probe says what was found)."""
    try:
        import tensorflow as tf  # noqa: F401
        return {"tensorflow_importable": True, "version": getattr(tf, "__version__", "?"),
                "note": "TensorFlow imports, but the reference's sources are not present at run time; "
                        "the timed code is oracle/, the op-for-op restatement of v1_model_utils/models.py"}
    except Exception as e:  # noqa: BLE001
        return {"tensorflow_importable": False, "error": type(e).__name__,
                "note": "reference TensorFlow CPU path: unavailable on this box (TensorFlow not installed); "
                        "the timed code is oracle/, the op-for-op restatement of v1_model_utils/models.py"}


# --------------------------------------------------------------------------------------
# CPU leg: the oracle restatement of the reference cell on the host cores
# --------------------------------------------------------------------------------------
def warmed_up_oracle_state(cfg, dicts, seed):
    """State of the column after WARM_STEPS ms of the stimulus.  On a box with a GPU the library's
    forward rollout produces it in milliseconds (it is an input of the timed CPU sample, not part of
    it); without one the oracle itself runs a shorter prefix."""
    x = synth.make_lgn_spikes(cfg, cfg.batch, WARM_STEPS, seed + 1000)
    c = synth.make_bkg_counts(cfg, cfg.batch, WARM_STEPS, seed + 1000)
    if torch.cuda.is_available():
        from v1_glif_model_b200.models import V1Column
        cell = V1Column(*dicts, **CELL_KW)
        state = cell.zero_state(cfg.batch)
        cell.rollout(torch.from_numpy(x).cuda(), torch.from_numpy(c).cuda(), state=state, return_z=False,
                     return_v=False)
        cell.synchronize()
        z_buf, v, r, asc, psc_rise, psc = [t.detach().cpu() for t in state[:6]]
        del cell
        torch.cuda.empty_cache()
        return (z_buf, v, r.to(torch.int64), asc, psc_rise, psc, torch.zeros((cfg.batch,), dtype=torch.int32)), "gpu"
    from oracle.cell_torch import OracleV1Column
    orc = OracleV1Column(*dicts, **CELL_KW)
    with torch.no_grad():
        _, _, state = orc.rollout(torch.from_numpy(x[:, :40]), torch.from_numpy(c[:, :40]).long())
    return tuple(t.detach() for t in state), "cpu prefix of 40 ms"


def cpu_training_sample(cfg, dicts, t_sample, seed):
    """One fwd+bwd of `t_sample` steps at the configuration's batch on the CPU oracle, from a
    warmed-up state, with the bench's three loss terms."""
    from oracle.cell_torch import OracleV1Column
    from oracle import losses as OL
    torch.set_num_threads(os.cpu_count() or 1)
    state0, how = warmed_up_oracle_state(cfg, dicts, seed)
    orc = OracleV1Column(*dicts, **CELL_KW)
    x = torch.from_numpy(synth.make_lgn_spikes(cfg, cfg.batch, t_sample, seed))
    c = torch.from_numpy(synth.make_bkg_counts(cfg, cfg.batch, t_sample, seed)).long()
    vscale = orc.params["voltage_scale"][orc.params["node_type_ids"]]
    tgt = torch.from_numpy(synth.make_rate_targets(cfg)) / 1000.0
    vlo = torch.from_numpy((-20.0 / vscale).astype(np.float32))
    # the synchrony term needs at least two bins; shorter samples use the largest bin that gives two
    sync_bin = min(LOSS["sync_bin"], max(t_sample // 2, 1))
    info = {"spikes": 0}

    def one():
        for w in (orc.recurrent_weight_values, orc.input_weight_values, orc.bkg_input_weights):
            w.grad = None
        t0 = time.perf_counter()
        z, v, _ = orc.rollout(x, c, state=state0)
        total = OL.rate_loss(z, tgt, LOSS["rate_cost"]) + OL.voltage_loss(v, vlo, LOSS["voltage_cost"]) + \
            OL.sync_loss(z, sync_bin, LOSS["sync_cost"], LOSS["fano_target"])
        total.backward()
        info["spikes"] = int(z.detach().sum())
        return time.perf_counter() - t0
    desc = (f"fwd+bwd (rate + voltage + synchrony over {sync_bin}-ms bins) of {t_sample} of the {cfg.seq_len} "
            f"simulated ms per step, extrapolated linearly in T; batch {cfg.batch}, N={cfg.n_neurons}, from a "
            f"state warmed up for {WARM_STEPS} ms ({how}); torch CPU restatement of the reference cell (oracle/)")
    return one, desc, info


def bounded_cpu_steps(requested, n_runs):
    """Simulated ms per CPU sample such that `n_runs` samples end within about four minutes."""
    budget = 240.0 / max(n_runs, 1)
    return int(max(6, min(requested, budget / CPU_SECONDS_PER_STEP)))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    cfg = synth.CONFIGS[args.config]
    dicts = synth.make_network(cfg, 0)
    t_sample = bounded_cpu_steps(args.cpu_sample_steps, args.steps + args.warmup)
    one, desc, info = cpu_training_sample(cfg, dicts, t_sample, 0)
    for _ in range(args.warmup):
        one()
    times = [one() for _ in range(args.steps)]
    sec = float(np.mean(times))
    value = cfg.batch * cfg.n_neurons * t_sample / sec
    cores = torch.get_num_threads()
    probe = tensorflow_probe()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(cfg, args.gpus, t_sample),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "mean_rate_hz": info["spikes"] / (cfg.batch * cfg.n_neurons * t_sample) * 1000.0,
        "reference_runtime": probe,
        "note": probe["note"] + ("; ONE CPU process ran (rank 0) whatever --gpus says: the value is not an "
                                 f"aggregate over {world} ranks" if world > 1 or args.gpus > 1 else ""),
    }
    print(json.dumps(line))


def workload_config(cfg, n_gpus, t_len):
    return {"workload": f"{cfg.name}: {cfg.n_neurons:,}-neuron synthetic column, fwd+bwd training step "
                        "(rate+voltage+synchrony loss, Exp-Adam on recurrent+LGN weights), every step from a "
                        f"carried state warmed up for {WARM_STEPS} ms",
            "n_neurons": cfg.n_neurons, "batch_per_gpu": cfg.batch, "global_batch": cfg.batch * n_gpus,
            "seq_len": t_len, "n_receptors": cfg.n_receptors, "max_delay": cfg.max_delay,
            "parallelism": f"dp{n_gpus}",
            "l2": "inputs larger than L2 (saved rollout %.2f GB per step)" % (4e-9 * cfg.batch * cfg.n_neurons * t_len)}


# --------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------
class Bench:
    """One rank: cell, trainer, inputs and timing helpers of a configuration."""

    def __init__(self, cfg, t_len, rank, world, dev, options=(), mutate=None):
        import torch.distributed as dist
        from v1_glif_model_b200.models import V1Column
        from v1_glif_model_b200.training import Trainer
        from v1_glif_model_b200 import _lib
        self.dist, self.cfg, self.t_len, self.rank, self.world, self.dev = dist, cfg, t_len, rank, world, dev
        self.b = b = cfg.batch
        self.dicts = synth.make_network(cfg, 0)
        if mutate is not None:
            mutate(*self.dicts)
        self.cell = cell = V1Column(*self.dicts, device=dev, **CELL_KW)
        self.options = tuple(options)
        for name, value in options:
            cell.set_option(name, value)
        self.lib = _lib.load()
        self.spec = loss_spec(cfg, cell.voltage_scale, dev)
        self.trainer = Trainer(cell, self.spec, learning_rate=1e-3, train_input=True, train_noise=False)
        # per-rank inputs (different seeds: the batch is sharded over ranks), pinned on the host
        self.x_host = torch.from_numpy(synth.make_lgn_spikes(cfg, b, t_len, seed=rank)).pin_memory()
        self.c_host = torch.from_numpy(synth.make_bkg_counts(cfg, b, t_len, seed=rank)).pin_memory()
        self.x_dev, self.c_dev = self.x_host.to(dev), self.c_host.to(dev)
        # carried state: WARM_STEPS ms of the same kind of input from the zero state, once
        xw = torch.from_numpy(synth.make_lgn_spikes(cfg, b, WARM_STEPS, seed=1000 + rank)).to(dev)
        cw = torch.from_numpy(synth.make_bkg_counts(cfg, b, WARM_STEPS, seed=1000 + rank)).to(dev)
        self.state0 = cell.zero_state(b)
        cell.rollout(xw, cw, state=self.state0, return_z=False, return_v=False)
        cell.synchronize()
        self.state = tuple(t.clone() for t in self.state0)
        # firing rates of the LGN units for the device-drawn inputs (the same drifting-grating formula)
        phi = torch.from_numpy(np.random.Generator(np.random.PCG64(7919 + rank)).uniform(0, 2 * np.pi, cfg.n_lgn))
        tt = torch.arange(t_len, dtype=torch.float64)[:, None] * 1e-3
        self.rates = (5.0 + 10.0 * torch.relu(torch.sin(2 * np.pi * 2.0 * tt + phi[None, :]))).float().to(dev)

    def reset_state(self):
        for dst, src in zip(self.state, self.state0):
            dst.copy_(src)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, steps):
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(steps):
            fn(k)
        e1.record()
        self.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return float(ms.item())

    def step_resident(self, k=0):
        self.reset_state()
        return self.trainer.step(self.x_dev, self.c_dev, state=self.state)

    def step_device_inputs(self, k=0):
        self.reset_state()
        return self.trainer.step_rates(self.rates, 1 + k + 100003 * self.rank, self.b, state=self.state)

    def make_e2e(self):
        """End-to-end step: inputs of step k+1 travel from pinned host memory on a second stream while
        step k computes; the losses are read back (and waited for) every step."""
        copy_stream = torch.cuda.Stream(device=self.dev)
        bufs = [(torch.empty_like(self.x_dev), torch.empty_like(self.c_dev)) for _ in range(2)]
        ready = [torch.cuda.Event() for _ in range(2)]
        free = [torch.cuda.Event() for _ in range(2)]
        loss_host = torch.zeros(4).pin_memory()
        main = torch.cuda.current_stream(self.dev)

        def prefetch(i):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(free[i])
                bufs[i][0].copy_(self.x_host, non_blocking=True)
                bufs[i][1].copy_(self.c_host, non_blocking=True)
                ready[i].record(copy_stream)
        for i in range(2):
            free[i].record(main)
        prefetch(0)

        def step(k):
            cur = k & 1
            prefetch(cur ^ 1)
            main.wait_event(ready[cur])
            self.reset_state()
            losses = self.trainer.step(bufs[cur][0], bufs[cur][1], state=self.state)
            free[cur].record(main)
            loss_host.copy_(losses, non_blocking=True)
            main.synchronize()
        return step


def run_ours(args):
    import torch.distributed as dist

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

    if args.only_lgn or args.only_real_basis:    # one side record alone (a small run for a profiler)
        if rank == 0:
            print(json.dumps({"lgn": lgn_record(args, dev)} if args.only_lgn else
                             {"real_basis": real_basis_record(args, rank, 1, dev)}))
        return
    options = [(o.split("=")[0], int(o.split("=")[1])) for o in args.lib_option]
    cfg = synth.CONFIGS[args.config]
    t_len = args.seq_len or cfg.seq_len
    bench = Bench(cfg, t_len, rank, world, dev, options)
    cell, lib, b = bench.cell, bench.lib, bench.b
    warm = max(args.warmup, 3)

    for k in range(warm):
        bench.step_resident(k)
    cell.synchronize()
    launches0 = lib.v1g_launch_count()
    with ClockSampler(local_rank) as clocks:
        total_ms = bench.timed(bench.step_resident, args.steps)
    launches = lib.v1g_launch_count() - launches0
    cell.synchronize()
    # kernel-only durations and event counters from one extra step outside the timed region
    bench.step_resident()
    fwd_ms, bwd_ms = cell.last_kernel_ms(0), cell.last_kernel_ms(1)
    cnt = cell.counters()

    step_e2e = bench.make_e2e()
    for k in range(2):
        step_e2e(k)
    e2e_ms = bench.timed(step_e2e, args.steps)
    for k in range(2):
        bench.step_device_inputs(k)
    dev_ms = bench.timed(bench.step_device_inputs, args.steps)
    cell.synchronize()
    cnt_dev = cell.counters()

    checks = gradient_checks(bench)
    if world > 1:
        checks["reduce_check"] = reduce_check(bench)
        # the two rollout kernels' durations on every rank (each rank has its own inputs; a step ends when
        # the slowest rank reaches the all-reduce)
        mine = torch.tensor([fwd_ms, bwd_ms], device=dev)
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        checks["kernel_ms_by_rank"] = [[round(float(v), 3) for v in t.tolist()] for t in every]

    stress = None
    if world > 1 and not args.no_stress and args.config == "C4":
        stress = stress_record(args, rank, world, dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    n, r = cfg.n_neurons, cfg.n_receptors
    ns_per_step = world * b * n * t_len
    ms_per_step = total_ms / args.steps
    value = ns_per_step / (ms_per_step * 1e-3)
    peak, peak_kind = measured_peaks()
    nnz_rec = bench.dicts[0]["synapses"]["indices"].shape[0]
    bb = bwd_bytes_per_launch(cnt, n, r, b, t_len, nnz_rec)
    fb = fwd_bytes_per_launch(cnt, n, r, b, t_len)
    bwd_s, fwd_s = bwd_ms * 1e-3, fwd_ms * 1e-3
    traffic = load_traffic(t_len)
    # the committed DRAM captures are of configuration 4; one thread per neuron (the register-resident
    # forward kernel) needs a slice of at most 512 neurons per block, a batch of at most 6 and 4 or 5 channels
    is_c4 = args.config == "C4" and not options
    slice_neurons = -(-n // torch.cuda.get_device_properties(dev).multi_processor_count)
    fwd_kernel_name = "rollout_fwd_reg_kernel" if slice_neurons <= 512 and b <= 6 and r in (4, 5) else "rollout_fwd_kernel"
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, world, t_len),
        "e2e": {"value": ns_per_step / (e2e_ms / args.steps * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": int(bench.x_host.numel() + bench.c_host.numel() * 4),
                "d2h_bytes_per_step": 16,
                "note": "inputs of step k+1 are copied from pinned host memory on a second stream while step k "
                        "computes; the losses are read back and waited for every step"},
        "device_inputs": {"value": ns_per_step / (dev_ms / args.steps * 1e-3), "unit": UNIT,
                          "h2d_bytes_per_step": 0,
                          "mean_rate_hz": cnt_dev["spikes"] / (b * n * t_len) * 1000.0,
                          "note": "LGN spikes drawn on the device from a resident firing-rate table and background "
                                  "counts from (noise seed, replica, step): the host sends seeds only"},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "kernel": "rollout_bwd_kernel", "achieved": bb / bwd_s / 1e9,
                     "peak": peak, "peak_source": peak_kind, "unit": "GB/s",
                     "frac": bb / bwd_s / 1e9 / peak,
                     "traffic": traffic.get("rollout_bwd_kernel") if is_c4 else None,
                     "traffic_source": "committed ncu capture of a T=100 case, scaled linearly in T" if is_c4
                                       else "no capture of this configuration",
                     "algorithmic_bytes_per_launch": bb, "kernel_ms": bwd_s * 1e3},
        "roofline_fwd_kernel": {"bound": "hbm", "kernel": fwd_kernel_name,
                                "achieved": fb / fwd_s / 1e9, "peak": peak, "unit": "GB/s",
                                "frac": fb / fwd_s / 1e9 / peak,
                                "traffic": traffic.get("rollout_fwd_reg_kernel") if is_c4 else None,
                                "algorithmic_bytes_per_launch": fb, "kernel_ms": fwd_s * 1e3},
        "roofline_step": {"achieved": (bb + fb) / (ms_per_step * 1e-3) / 1e9, "unit": "GB/s",
                          "frac": (bb + fb) / (ms_per_step * 1e-3) / 1e9 / peak,
                          "note": "algorithmic bytes of both rollout kernels over the whole step time"},
        "mean_rate_hz": cnt["spikes"] / (b * n * t_len) * 1000.0,
        "events_per_step": {k: cnt[k] / t_len for k in ("rec_events", "lgn_events", "bkg_events",
                                                        "dw_events", "bwd_events")},
        "storage": {"q_ring": "five 24-bit floats per 16-byte row (batch 5); fp32 rows with the library option "
                              "no_q_pack", "tape": "f32 voltage whose two lowest mantissa bits hold the spike and "
                                                   "refractory flags"},
        "lib_options": dict(options),
    }
    line.update(checks)
    if stress is not None:
        line["stress"] = stress
    if world == 1 and not args.no_fwd and args.config == "C4":
        line["fwd"] = forward_only(bench, args)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(cfg, bench.dicts, args)
    else:
        line["cpu_baseline"] = None
    if world == 1 and not args.no_real_basis and args.config == "C4":
        del bench
        torch.cuda.empty_cache()
        line["real_basis"] = real_basis_record(args, rank, world, dev)
    if world == 1 and not args.no_lgn and args.config == "C4":
        torch.cuda.empty_cache()
        line["lgn"] = lgn_record(args, dev)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def _raw_gradients(bench, options):
    """Flat weight gradients of one backward pass over the saved rollout with library options set."""
    cell = bench.cell
    for name, value in options:
        cell.set_option(name, value)
    flat = torch.zeros_like(bench.trainer.grads.flat)
    cell.backward_internal(bench.spec, flat)
    cell.synchronize()
    for name, _ in options:
        cell.set_option(name, dict(bench.options).get(name, 0))
    return flat


def gradient_checks(bench):
    """Outside the timed region: the same saved rollout differentiated with the benchmarked storage
    (24-bit rows) and with fp32 rows, and with the paired ring layout."""
    bench.reset_state()
    bench.cell.rollout(bench.x_dev, bench.c_dev, state=bench.state, return_z=False, return_v=False,
                       save_for_bwd=True)
    base = _raw_gradients(bench, ())
    n_rec = bench.trainer.grads.sizes[0]

    def rel_l2(a, ref):
        return float((a.double() - ref.double()).norm() / ref.double().norm())
    plain = _raw_gradients(bench, (("no_q_pack", 1),))
    paired = _raw_gradients(bench, (("pair_rows", 1),))
    return {"grad_check": {"dW_rec_rel_l2_24bit_vs_fp32_rows": rel_l2(base[:n_rec], plain[:n_rec]),
                           "dW_lgn_rel_l2_24bit_vs_fp32_rows": rel_l2(base[n_rec:], plain[n_rec:]),
                           "dW_rec_rel_l2_paired_vs_unpaired_ring": rel_l2(paired[:n_rec], base[:n_rec])}}


def reduce_check(bench):
    """N >= 2, outside the timed region: the all-reduced buffer against the ranks' own buffers, and the
    replicas' weights after the update against each other."""
    dist, tr, cell = bench.dist, bench.trainer, bench.cell
    bench.reset_state()
    tr.grads.zero_()
    cell.rollout(bench.x_dev, bench.c_dev, state=bench.state, return_z=False, return_v=False, save_for_bwd=True)
    cell.backward_internal(tr.loss, tr.grads.flat)
    cell.synchronize()
    flat = tr.grads.flat
    stride = max(flat.numel() // 65536, 1)
    local = torch.stack([flat.double().sum(), flat.double().abs().sum()])
    sample = flat[::stride].double().clone()
    sums = [torch.zeros_like(local) for _ in range(bench.world)]
    dist.all_gather(sums, local)
    samples = [torch.zeros_like(sample) for _ in range(bench.world)]
    dist.all_gather(samples, sample)
    tr.grads.all_reduce(tr.group)
    want_sum = sum(float(s[0]) for s in sums)
    scale = sum(float(s[1]) for s in sums)
    got_sum = float(flat.double().sum())
    want_sample = torch.stack(samples).sum(0)
    sample_err = float((flat[::stride].double() - want_sample).abs().max() / want_sample.abs().max().clamp_min(1e-30))
    # apply the update, then compare a checksum of the weights across replicas
    tr.iterations += 1
    cell._check(cell._lib.v1g_expadam_update_internal(
        cell._libh, flat.data_ptr(), tr.m.data_ptr(), tr.v.data_ptr(), tr.train_mask, tr.lr, 0.9, 0.999, 1e-11,
        tr.iterations, 1.0, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    w = tr.weights()
    wsum = torch.stack([w[0].double().sum(), w[1].double().sum(), (w[0].double() * w[0].double()).sum()])
    wsums = [torch.zeros_like(wsum) for _ in range(bench.world)]
    dist.all_gather(wsums, wsum)
    identical = all(torch.equal(wsums[0], o) for o in wsums[1:])
    return {"sum_rel_err": abs(got_sum - want_sum) / max(scale, 1e-30), "sampled_entries": int(sample.numel()),
            "sampled_entries_max_rel_err": sample_err, "replica_weight_checksums_identical": bool(identical)}


def stress_record(args, rank, world, dev):
    """Configuration 5 (230,924 neurons, batch 4 per GPU, ~12 Hz) at a reduced length, timed like the
    main step; attached to the line of multi-GPU runs."""
    cfg = synth.CONFIGS["C5"]
    t_len = args.stress_seq_len
    bench = Bench(cfg, t_len, rank, world, dev)
    cell = bench.cell
    for k in range(2):
        bench.step_resident(k)
    steps = max(3, min(args.steps, 5))
    ms = bench.timed(bench.step_resident, steps) / steps
    bench.step_resident()
    fwd_ms, bwd_ms = cell.last_kernel_ms(0), cell.last_kernel_ms(1)
    cnt = cell.counters()
    n, r, b = cfg.n_neurons, cfg.n_receptors, cfg.batch
    peak, _ = measured_peaks()
    nnz_rec = bench.dicts[0]["synapses"]["indices"].shape[0]
    bb, fb = bwd_bytes_per_launch(cnt, n, r, b, t_len, nnz_rec), fwd_bytes_per_launch(cnt, n, r, b, t_len)
    return {"workload": f"C5: {n:,} neurons, batch {b} per GPU, T={t_len} of {cfg.seq_len}, fwd+bwd training step",
            "value": world * b * n * t_len / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "n_gpus": world,
            "mean_rate_hz": cnt["spikes"] / (b * n * t_len) * 1000.0,
            "roofline": {"bound": "hbm", "kernel": "rollout_bwd_kernel", "achieved": bb / (bwd_ms * 1e-3) / 1e9,
                         "peak": peak, "unit": "GB/s", "frac": bb / (bwd_ms * 1e-3) / 1e9 / peak,
                         "kernel_ms": bwd_ms, "algorithmic_bytes_per_launch": bb, "traffic": None},
            "roofline_fwd_kernel": {"kernel": "rollout_fwd_kernel", "achieved": fb / (fwd_ms * 1e-3) / 1e9,
                                    "frac": fb / (fwd_ms * 1e-3) / 1e9 / peak, "kernel_ms": fwd_ms},
            "events_per_step": {k: cnt[k] / t_len for k in ("rec_events", "lgn_events", "bkg_events", "dw_events")}}


def real_basis_record(args, rank, world, dev):
    """The full-size column with the reference's own synaptic basis instead of the synthetic one-hot
    one: 4 time constants and 121 synapse types whose rows of basis weights are dense and partly
    negative (synaptic_data/tau_basis.npy and basis_function_weights.csv of the reference, carried by
    the committed fixture tests/golden/reference_small_real_basis.npz).  Up to 4 atomics per delivered
    synapse in the forward rollout; the backward ring holds the raw per-channel adjoints and a synapse
    reads 4 rows."""
    import dataclasses
    path = os.path.join(ROOT, "tests", "golden", "reference_small_real_basis.npz")
    if not os.path.exists(path):
        return {"unavailable": "fixture with the reference's basis tables not found"}
    g = np.load(path)
    tau, basis = g["tau_syn"], g["synaptic_basis_weights"]
    # background / LGN weight scales recalibrated for this basis (its rows sum to 1.2-2.7 over four
    # channels instead of one unit entry) so that the column settles near 4 Hz as in configuration 4
    cfg = dataclasses.replace(synth.CONFIGS["C4"], n_receptors=int(tau.size), bkg_weight_pa=17.3, lgn_weight_pa=3.05)

    def mutate(net, lgn, bkg):
        rng = np.random.Generator(np.random.PCG64(12))
        net["tau_syn"], net["synaptic_basis_weights"] = tau, basis
        for d in (net["synapses"], lgn, bkg):
            d["syn_ids"] = rng.integers(0, basis.shape[0], d["syn_ids"].shape[0]).astype(np.uint8)
    t_len = args.real_basis_seq_len
    bench = Bench(cfg, t_len, rank, world, dev, mutate=mutate)
    cell = bench.cell
    for k in range(2):
        bench.step_resident(k)
    steps = 3
    ms = bench.timed(bench.step_resident, steps) / steps
    bench.step_resident()
    fwd_ms, bwd_ms = cell.last_kernel_ms(0), cell.last_kernel_ms(1)
    cnt = cell.counters()
    n, r, b = cfg.n_neurons, cfg.n_receptors, cfg.batch
    peak, _ = measured_peaks()
    nnz_rec = bench.dicts[0]["synapses"]["indices"].shape[0]
    bb, fb = bwd_bytes_per_launch(cnt, n, r, b, t_len, nnz_rec), fwd_bytes_per_launch(cnt, n, r, b, t_len)
    return {"workload": f"C4 column with the reference's basis (R={r}, S={basis.shape[0]} dense rows), batch {b}, "
                        f"T={t_len}, fwd+bwd training step",
            "value": world * b * n * t_len / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms,
            "mean_rate_hz": cnt["spikes"] / (b * n * t_len) * 1000.0,
            "note": "synapse types drawn uniformly from the 121 rows; input weight scales calibrated for this basis",
            "roofline": {"bound": "hbm", "kernel": "rollout_bwd_kernel (raw rows)", "achieved": bb / (bwd_ms * 1e-3) / 1e9,
                         "peak": peak, "unit": "GB/s", "frac": bb / (bwd_ms * 1e-3) / 1e9 / peak, "kernel_ms": bwd_ms,
                         "algorithmic_bytes_per_launch": bb, "traffic": None},
            "roofline_fwd_kernel": {"achieved": fb / (fwd_ms * 1e-3) / 1e9, "frac": fb / (fwd_ms * 1e-3) / 1e9 / peak,
                                    "kernel_ms": fwd_ms}}


def lgn_record(args, dev):
    """The step upstream of the cell's input: movie -> LGN firing rates (lgn_model/lgn.py:481-528) at the
    reference's sizes: 120 x 240 frames, 17,400 units in 14 spatial size classes, temporal kernels of 250 ms."""
    from v1_glif_model_b200.lgn import LGN
    height, width, n_units, n_frames, taps = 120, 240, 17400, args.lgn_frames, 250
    sides = tuple(range(3, 31, 2))
    tb = synth.make_lgn_tables(n_units, height, width, sides, taps, taps, seed=4)
    lgn = LGN(**tb, row_size=height, col_size=width)
    movie = torch.rand((n_frames, height, width), device=dev) * 2 - 1
    for _ in range(3):
        lgn.firing_rates(movie)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    reps = 5
    torch.cuda.synchronize()
    ev[0].record()
    for _ in range(reps):
        lgn.spatial_response(movie)
    ev[1].record()
    for _ in range(reps):
        rates = lgn.firing_rates(movie)
    ev[2].record()
    torch.cuda.synchronize()
    spatial_ms, total_ms = ev[0].elapsed_time(ev[1]) / reps, ev[1].elapsed_time(ev[2]) / reps
    stencil_taps = 2 * sum(float(len(idx)) * (s + 1) ** 2 for idx, s in zip(tb["spatial_range_indices"], sides))
    flops = 2.0 * n_frames * (stencil_taps + n_units * 2 * taps)
    return {"workload": f"movie -> LGN firing rates: {n_frames} frames of {height} x {width}, {n_units} units, "
                        f"{len(sides)} filter sizes up to {sides[-1]} taps wide, {taps}-ms temporal kernels",
            "value": n_frames / (total_ms * 1e-3), "unit": "frames/s", "ms": total_ms, "spatial_kernel_ms": spatial_ms,
            "gflops": flops / (total_ms * 1e-3) / 1e9, "mean_rate_hz": float(rates.mean()),
            "note": "movie resident on the device; two kernels per call (stencils over frames held in shared "
                    "memory, temporal filter); inputs (115 MB per 1000 frames) exceed L2 together with the outputs"}


def forward_only(bench, args):
    """Configuration 3: forward-only rollout, batch 5, T=2500, from the warmed-up state."""
    cell, lib, dev = bench.cell, bench.lib, bench.dev
    cfg = synth.CONFIGS["C3"]
    t_len = args.fwd_seq_len or cfg.seq_len
    b, n, r = cfg.batch, cfg.n_neurons, cfg.n_receptors
    x_host = torch.from_numpy(synth.make_lgn_spikes(cfg, b, t_len, seed=0)).pin_memory()
    c_host = torch.from_numpy(synth.make_bkg_counts(cfg, b, t_len, seed=0)).pin_memory()
    x_dev, c_dev = x_host.to(dev), c_host.to(dev)
    z = torch.empty((b, t_len, n), dtype=torch.uint8, device=dev)
    v = torch.empty((b, t_len, n), dtype=torch.float32, device=dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def fwd():
        bench.reset_state()
        st = cell._state_struct(bench.state)
        cell._check(lib.v1g_rollout_fwd(cell._libh, b, t_len, x_dev.data_ptr(), c_dev.data_ptr(), C.byref(st),
                                        z.data_ptr(), v.data_ptr(), 0, stream))
    for _ in range(3):
        fwd()
    cell.synchronize()
    reps = max(3, args.steps)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fwd()
    e1.record()
    cell.synchronize()
    ms = e0.elapsed_time(e1) / reps
    kms = cell.last_kernel_ms(0)
    cnt = cell.counters()
    del v
    torch.cuda.empty_cache()
    peak, _ = measured_peaks()
    fb = fwd_bytes_per_launch(cnt, n, r, b, t_len)
    ns = b * n * t_len
    out = {"workload": "C3: forward only, batch 5, T=%d, z (uint8) and v (f32) written, from the warmed-up state" % t_len,
           "value": ns / (ms * 1e-3), "unit": UNIT, "ms_per_rollout": ms,
           "us_per_simulated_ms": ms * 1e3 / t_len,
           "roofline": {"bound": "hbm", "kernel": "rollout_fwd_reg_kernel",
                        "achieved": fb / (kms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                        "frac": fb / (kms * 1e-3) / 1e9 / peak, "kernel_ms": kms,
                        "algorithmic_bytes_per_launch": fb,
                        "traffic": load_traffic(t_len).get("rollout_fwd_reg_kernel"),
                        "traffic_source": "committed ncu capture of a T=100 case, scaled linearly in T"},
           "mean_rate_hz": cnt["spikes"] / ns * 1000.0}
    out["e2e"] = forward_e2e(bench, x_host, c_host, t_len, ns)
    return out


def forward_e2e(bench, x_host, c_host, t_len, ns):
    """End to end through the host-buffer entry points (pinned buffers in, spikes out)."""
    cell = bench.cell
    res = {}
    for fmt in ("bits", "uint8"):
        if not hasattr(cell, "rollout_host_pipelined"):
            break
        cell.rollout_host_pipelined(x_host, c_host, z_format=fmt)   # warm-up (allocations)
        t0 = time.perf_counter()
        for _ in range(2):
            zh = cell.rollout_host_pipelined(x_host, c_host, z_format=fmt)
        sec = (time.perf_counter() - t0) / 2
        res[fmt] = {"value": ns / sec, "unit": UNIT, "h2d_bytes": int(x_host.numel() + c_host.numel() * 4),
                    "d2h_bytes": int(zh.numel() * zh.element_size())}
    if not res:
        zh = np.empty((x_host.shape[0], t_len, cell._n_neurons), dtype=np.uint8)
        t0 = time.perf_counter()
        for _ in range(2):
            cell.rollout_host(x_host.numpy(), c_host.numpy(), want_z=True)
        sec = (time.perf_counter() - t0) / 2
        return {"value": ns / sec, "unit": UNIT, "h2d_bytes": int(x_host.numel() + c_host.numel() * 4),
                "d2h_bytes": int(zh.nbytes), "note": "v1g_rollout_fwd_host, one copy in, one rollout, one copy out"}
    best = res["bits"]
    return {"value": best["value"], "unit": UNIT, "h2d_bytes": best["h2d_bytes"], "d2h_bytes": best["d2h_bytes"],
            "note": "v1g_rollout_fwd_host_pipelined from the zero state: chunks of the rollout, input copies, "
                    "compute and result copies overlapped on three streams; spikes returned as 1 bit per "
                    "neuron-step", "uint8_spikes": res["uint8"]}


def cpu_baseline(cfg, dicts, args):
    t_sample = bounded_cpu_steps(args.cpu_sample_steps, 2)
    one, desc, info = cpu_training_sample(cfg, dicts, t_sample, 0)
    one()
    sec = one()
    return {"value": cfg.batch * cfg.n_neurons * t_sample / sec, "unit": UNIT,
            "cores": torch.get_num_threads(), "kind": "port", "sample": desc,
            "mean_rate_hz": info["spikes"] / (cfg.batch * cfg.n_neurons * t_sample) * 1000.0}


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
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default 10; 5 for the CPU arm)")
    ap.add_argument("--warmup", type=int, default=None, help="untimed steps before them (default 5; 3 for the CPU arm)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="C4", choices=["C4", "C5", "C2"],
                    help="C4 = the metric's configuration (default); C5 = 230,924-neuron stress; C2 = 5,000 neurons")
    ap.add_argument("--seq-len", type=int, default=0, help="override T of the training step")
    ap.add_argument("--fwd-seq-len", type=int, default=0, help="override T of the forward-only leg")
    ap.add_argument("--stress-seq-len", type=int, default=100, help="T of the configuration-5 record at N >= 2")
    ap.add_argument("--cpu-sample-steps", type=int, default=50,
                    help="simulated ms per CPU sample (reduced automatically so that the run ends within minutes)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fwd", action="store_true")
    ap.add_argument("--no-stress", action="store_true")
    ap.add_argument("--no-real-basis", action="store_true")
    ap.add_argument("--no-lgn", action="store_true")
    ap.add_argument("--only-lgn", action="store_true", help="run the LGN front-end record and nothing else")
    ap.add_argument("--only-real-basis", action="store_true", help="run the reference-basis record and nothing else")
    ap.add_argument("--lgn-frames", type=int, default=1000, help="frames of the movie of the LGN record")
    ap.add_argument("--real-basis-seq-len", type=int, default=200, help="T of the record with the reference's basis")
    ap.add_argument("--lib-option", action="append", default=[], metavar="NAME=VALUE",
                    help="library tuning option for the training cell, e.g. pair_rows=1 (repeatable)")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = 5 if args.impl == "reference" else 10
    if args.warmup is None:
        args.warmup = 3 if args.impl == "reference" else 5
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
