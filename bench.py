"""Benchmark of the NCN fused forward + backward (the one hot path of this repository).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One step = one fused forward + one fused backward (incl. the fixed-order dW reduction and, for
N > 1, the NCCL sum of dW) over one batch of synthetic rows.  With N > 1 (launched by torchrun,
one rank per GPU) every rank runs the same per-GPU workload on its own rows (weak scaling) and
`value` is the whole-job rows/s from the slowest rank's device time.

A default run (workload cfg2) then measures the other configurations for a few steps each and
attaches them under "workloads" (one GPU: configs 2-linear, 4, 3, 5, 1; several GPUs: config 5).

`--impl reference` times the CPU restatement of the reference's torch_ref path (oracle/) on the
host cores instead, rank 0 only, and beside it the reference's own literal torch_ref loops where
oracle/_ref/ holds them.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

# name -> per-GPU shape.  cfg2 is the configuration the headline metric is quoted on.
WORKLOADS = {
    "cfg1": dict(steps=100, warmup=20, B=1024, N=1024, n=2, L=10, w_var=0.5, dtype="f32", act="tanh", seed=0,
                 desc="CPU-sized NCN layer fp32 x[1024,1024] g=2 10 stages tanh"),
    "cfg2": dict(B=65536, N=4096, n=4, L=6, w_var=0.25, dtype="f32", act="tanh", seed=1,
                 desc="single-GPU NCN layer fp32 x[65536,4096] g=4 6 stages tanh"),
    "cfg2_linear": dict(B=65536, N=4096, n=4, L=6, w_var=0.25, dtype="f32", act="linear", seed=1,
                        desc="as cfg2 with linear activation"),
    "cfg4": dict(B=131072, N=4096, n=8, L=4, w_var=0.01, dtype="f32", act="tanh", seed=3, mode="invert",
                 desc="invertible variant fp32 x[131072,4096] g=8 4 stages"),
    "cfg3": dict(B=262144, N=8192, n=16, L=4, w_var=1 / 16, dtype="bf16", act="tanh", seed=2, mode="tape",
                 desc="bf16 storage x[262144,8192] g=16 4 stages"),
    "cfg5": dict(B=131072, N=2048, n=8, L=4, w_var=1 / 8, dtype="bf16", act="tanh", seed=4, layers=12, mode="tape",
                 desc="12 residual NCN layers D=2048 g=8 4 stages bf16, 131072 rows per GPU (1/8 of the 8-GPU global batch)"),
    "ref_e128": dict(B=4096, N=256, E=128, C=4, n=32, L=3, w_var=1 / 32, dtype="f32", act="tanh", seed=5, stage_keep="output",
                     desc="the reference's own bench shape scaled in rows: x[4096,256,128] 4 heads g=32 3 stages, one kernel per "
                          "stage, backward from each stage's output alone (the reference operator's contract)"),
    "ref_e128_mid": dict(B=4096, N=256, E=128, C=4, n=32, L=3, w_var=1 / 32, dtype="f32", act="tanh", seed=5,
                         stage_keep="mid",
                         desc="ref_e128 with the state after step 16 of every stage stored by the forward (inverse chains of 16 "
                              "steps: 1e-5 gradients; what the operator does by default)"),
    "ref_e128_input": dict(B=4096, N=256, E=128, C=4, n=32, L=3, w_var=1 / 32, dtype="f32", act="tanh", seed=5,
                           stage_keep="input",
                           desc="ref_e128 with the stage inputs kept for the backward (inverse chains of 16 steps: 1e-5 gradients)"),
    "ref_e128_small": dict(B=1024, N=256, E=128, C=4, n=32, L=3, w_var=1 / 32, dtype="f32", act="tanh", seed=5,
                           desc="ref_e128 with 1024 rows (profiling case)"),
    "small": dict(B=8192, N=4096, n=4, L=6, w_var=0.25, dtype="f32", act="tanh", seed=1,
                  desc="cfg2 with 8192 rows (profiling case)"),
    "cfg4_small": dict(B=8192, N=4096, n=8, L=4, w_var=0.01, dtype="f32", act="tanh", seed=3, mode="invert",
                       desc="cfg4 with 8192 rows (profiling case)"),
    "cfg5_small": dict(B=16384, N=2048, n=8, L=4, w_var=1 / 8, dtype="bf16", act="tanh", seed=4, layers=2, mode="tape",
                       desc="two residual layers of the cfg5 shape, 16384 rows (profiling case)"),
}

# Workloads measured for a few steps after the headline one in a default run (one GPU: all of them;
# several GPUs: the stack, which is the configuration quoted at 1/2/4/8 GPUs).
EXTRA_1GPU = ["cfg2_linear", "cfg4", "cfg3", "cfg5", "cfg1", "ref_e128", "ref_e128_mid"]
EXTRA_NGPU = ["cfg5"]

# DRAM bytes per element moved by the backward kernel in one launch (dram__bytes_read.sum +
# dram__bytes_write.sum over B*N) from an ncu capture of the 8192-row case of cfg2 (fp32, one stored
# state): 836.0 + 252.0 MB over 33.55 M elements.  Traffic grows in proportion to the rows, so the full
# launch is this figure times its elements.
BWD_TRAFFIC_BYTES_PER_ELEMENT = 32.43

# rows per step of the CPU arms (both the cpu_baseline leg and --impl reference use this one rule)
CPU_ROWS_PER_STEP = 1024
CPU_STEPS = 5


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--mode", default=None, help="backward mode override: auto|checkpoint|invert|recompute|tape")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the other workloads after the headline one")
    ap.add_argument("--extra-steps", type=int, default=5)
    return ap.parse_args()


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ------------------------------------------------------------------ CPU arms
def config_of(wl, mode=None, world=1):
    """The `config` object of a JSON line: the same keys in the GPU arm and in the reference arm."""
    w = 4 if wl["dtype"] == "f32" else 2
    return {"workload": wl["desc"], "rows_per_gpu": wl["B"], "D": wl["N"], "E": wl.get("E", 1), "heads": wl.get("C", 1),
            "g": wl["n"], "stages": wl["L"], "layers": wl.get("layers", 1), "activation": wl["act"],
            "backward_mode": mode or wl.get("mode", "auto"), "parallelism": f"dp{world}",
            "l2": ("inputs larger than L2 (%.2f GB per tensor)" if wl["B"] * wl["N"] * wl.get("E", 1) * w > 126e6 else
                   "inputs fit L2 (%.4f GB per tensor) and are not flushed between steps: a latency-bound case, not a "
                   "bandwidth figure") % (wl["B"] * wl["N"] * wl.get("E", 1) * w / 1e9)}


def cpu_port_rows_per_s(wl, steps=CPU_STEPS, warmup=1, rows=CPU_ROWS_PER_STEP, threads=None):
    """The oracle (vectorised torch-CPU restatement of the reference's torch_ref path), forward +
    autograd backward, on `rows` rows of the workload per step; median over `steps` timed steps.
    One sampling rule for every CPU figure this file prints."""
    from oracle import ncn_oracle as O

    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    rows = min(rows, wl["B"])
    E, C = wl.get("E", 1), wl.get("C", 1)
    x, xa, ws, dy, dya = O.make_inputs(wl["seed"], rows, wl["N"], E, wl["L"], wl["w_var"])
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.net_fwd_bwd(x, xa, ws, dy, dya, 0.9, wl["act"], wl["n"], C)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    med = sorted(times)[len(times) // 2]
    ws_mb = 5 * rows * wl["N"] * E * 4 / 1e6
    sample = (f"{rows} of {wl['B']} rows of the workload per step ({ws_mb:.0f} MB of fp32 tensors), median of {len(times)} steps "
              f"after {warmup} warm-up, vectorised torch-CPU restatement of torch_ref, forward + autograd backward")
    return {"value": rows / med, "unit": "rows/s", "cores": threads, "kind": "port", "sample": sample}, med, times


def cpu_literal_rows_per_s(rows=2):
    """The reference's OWN torch_ref loops (RefTorchNaive, torch_ref/ncn_pytorch.py:103-124; one Python
    iteration per batch row, head, group and step), forward + autograd backward on `rows` rows of
    config 1.  Present only where oracle/build_ref_python.py has put the reference's files under
    oracle/_ref/; returns None otherwise."""
    from oracle import build_ref_python
    from oracle import ncn_oracle as O

    mod = build_ref_python.load("torch_ref.ncn_pytorch")
    if mod is None:
        return None
    wl = WORKLOADS["cfg1"]
    x, xa, ws, dy, dya = O.make_inputs(wl["seed"], rows, wl["N"], 1, wl["L"], wl["w_var"])
    x.requires_grad_(True)
    xa.requires_grad_(True)
    ws = [w.requires_grad_(True) for w in ws]
    net = mod.RefTorchNaive(0.9, "tanh", wl["L"], wl["n"], 1, ws)
    t0 = time.perf_counter()
    y, ya = net(x, xa)
    y.backward(dy)
    dt = time.perf_counter() - t0
    return {"value": rows / dt, "unit": "rows/s", "cores": 1, "kind": "reference",
            "sample": f"{rows} rows of config 1 (x[1024,1024], g=2, 10 stages), the reference's literal RefTorchNaive loops "
                      f"(interpreter-bound, one thread), forward + autograd backward, {dt:.1f} s, not extrapolated"}


def run_reference(args, wl, rank):
    if rank != 0:
        return
    base, med, times = cpu_port_rows_per_s(wl, steps=max(1, args.steps), warmup=max(1, args.warmup))
    value = base["value"]
    line = {
        "impl": "reference", "metric": "ncn_fwd_bwd_rows_per_s", "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * med,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": config_of(wl, args.mode, args.gpus),
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    lit = cpu_literal_rows_per_s()
    if lit is not None:
        line["cpu_reference_literal"] = lit
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
def kernel_names(wl, mode):
    """The kernels the library picks for this workload (for the roofline label)."""
    if wl.get("E", 1) > 1:
        return "feat_fwd_kernel (ncn_feat.cuh)", "feat_bwd_kernel (ncn_feat.cuh)"
    n = wl["n"]
    if n == 16 or mode == "recompute":
        return "pair_fwd_dual_kernel (ncn_pairs.cuh)", "rows_bwd_kernel / pair_bwd_wide_kernel"
    if n == 4 and wl["L"] <= 6:
        return "lane_fwd_kernel (ncn_lanes.cuh)", "lanep_bwd_kernel (ncn_lanes_pipe.cuh)"
    return "lane_fwd_kernel (ncn_lanes.cuh)", "lane_bwd_kernel (ncn_lanes.cuh)"


def measure(ncn, name, wl, mode_override, dev, rank, world, steps, warmup, clocks_index=None):
    """Device-resident timing of `steps` forward + backward steps of one workload.  Returns
    (summary dict, objects needed by the e2e leg)."""
    import torch.distributed as dist

    dtype = torch.float32 if wl["dtype"] == "f32" else torch.bfloat16
    w = 4 if wl["dtype"] == "f32" else 2
    B, N, n, L = wl["B"], wl["N"], wl["n"], wl["L"]
    E, C = wl.get("E", 1), wl.get("C", 1)
    mode = mode_override or wl.get("mode", "auto")
    g = torch.Generator(device=dev).manual_seed(wl["seed"] + 1000 * rank)
    x = torch.randn(B, N, E, generator=g, device=dev, dtype=torch.float32).to(dtype).requires_grad_(True)
    xa = torch.zeros(B, N, E, device=dev, dtype=dtype).requires_grad_(True)
    dy = torch.randn(B, N, E, generator=g, device=dev, dtype=torch.float32).to(dtype)
    dya = torch.zeros(B, N, E, device=dev, dtype=dtype)
    gw = torch.Generator().manual_seed(wl["seed"])
    layers = wl.get("layers", 0)
    if layers:
        net = ncn.NCNResidualStack(layers, 0.9, wl["act"], n, 1, L, 1, w_std=wl["w_var"] ** 0.5,
                                   backward_mode="tape" if mode == "auto" else mode).to(dev)
        ws = [net.weight]
    else:
        ws = [(torch.randn(2 * E, generator=gw) * wl["w_var"] ** 0.5).to(dev).requires_grad_(True) for _ in range(L)]
        net = ncn.NCNNetTestCuda(0.9, wl["act"], n, C, L, ws, backward_mode=mode)

    if wl.get("stage_keep"):
        ncn.set_stage_backward(wl["stage_keep"])  # per-stage operator: what it keeps for its backward

    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]

    def step(i=None):
        x.grad = None; xa.grad = None
        for p in ws:
            p.grad = None
        if i is not None:
            ev[i][0].record()
        y, ya = net(x, xa)
        if i is not None:
            ev[i][1].record()
        torch.autograd.backward([y, ya], [dy, dya])
        ncn.allreduce_weight_grads(ws)
        if i is not None:
            ev[i][2].record()

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(clocks_index if clocks_index is not None else dev.index) as clocks:
        t_start = torch.cuda.Event(enable_timing=True); t_end = torch.cuda.Event(enable_timing=True)
        t_start.record()
        for i in range(steps):
            step(i)
        t_end.record()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ncn.ops.device_status()
    ncn.set_stage_backward("auto")
    ms = t_start.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / steps
    fwd_ms = sorted(e[0].elapsed_time(e[1]) for e in ev)[len(ev) // 2]
    bwd_ms = sorted(e[1].elapsed_time(e[2]) for e in ev)[len(ev) // 2]
    value = world * B / (ms_step * 1e-3)

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    # every layer of a stack moves the same bytes; with several features per position every STAGE is
    # its own forward and backward kernel and moves them again
    per_stage = E > 1
    launches = max(1, layers) * (L if per_stage else 1)  # backward launches per step
    elems = B * N * E * launches
    bwd_bytes = 6 * w * elems  # reads y, ya, dy, dya; writes dx, dxa
    bwd_gbs = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    step_gbs = 10 * w * elems / ((fwd_ms + bwd_ms) * 1e-3) / 1e9
    fk, bk = kernel_names(wl, mode)
    roofline = {
        "bound": "hbm", "kernel": bk + (", %d launches per step" % launches if launches > 1 else ""),
        "forward_kernel": fk, "achieved": bwd_gbs, "peak": peak, "peak_source": peak_src,
        "unit": "GB/s", "frac": bwd_gbs / peak, "ms_per_launch": bwd_ms / launches,
        # measured on the 8192-row case of the cfg2 shape (fp32, one stored state), scaled by the elements
        "traffic": (BWD_TRAFFIC_BYTES_PER_ELEMENT * elems if name in ("cfg2", "small") and mode == "auto" else None),
        "algorithmic_bytes": bwd_bytes // launches,
        "fwd_plus_bwd": {"achieved": step_gbs, "frac": step_gbs / peak, "frac_of_8TBs_nominal": step_gbs / 8000.0,
                         "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "algorithmic_bytes": 10 * w * elems},
        "note": "bound by the FMA and special-function pipes (n*L dependent tanh steps per element), not by HBM; "
                "the HBM fraction is reported because the metric asks for it",
    }
    summary = {
        "value": value, "unit": "rows/s", "ms_per_step": ms_step, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "mode": mode,
        "dtype": wl["dtype"], "rows_per_s_per_gpu": value / world, "roofline": roofline,
        "gpu_launches": (3 * L if per_stage else 3) * steps * max(1, layers), "clocks": clocks.summary(),
        "steps": steps, "warmup": warmup, "config": config_of(wl, mode, world),
    }
    return summary, (dtype, ws, mode, layers, per_stage)


def run_b200(args, wl, rank, world, local_rank):
    import torch.distributed as dist

    import ncn_cuda_b200 as ncn

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    m, (dtype, ws, mode, layers, per_stage) = measure(ncn, args.workload, wl, args.mode, dev, rank, world, args.steps,
                                                      args.warmup, local_rank)
    line = {
        "metric": "ncn_fwd_bwd_rows_per_s", "value": m["value"], "unit": "rows/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": m["config"], "roofline": m["roofline"], "gpu_launches": m["gpu_launches"], "clocks": m["clocks"],
        "rows_per_s_per_gpu": m["rows_per_s_per_gpu"],
    }

    if not args.no_e2e and not layers and not per_stage:
        e2e = run_e2e(ncn, wl, dev, dtype, ws, mode, world, rank)  # every rank: its rows through its own host buffers
        if rank == 0:
            line["e2e"] = e2e
    del ws
    torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()

    # the other configurations, a few steps each (device-resident figures; same timing rules)
    if not args.no_extra and args.workload == "cfg2":
        extra = {}
        for name in (EXTRA_1GPU if world == 1 else EXTRA_NGPU):
            try:
                # a sub-millisecond step (config 1) is timed over more steps: a handful of them is over before the clocks settle
                ew = WORKLOADS[name]
                em, keep = measure(ncn, name, ew, None, dev, rank, world, ew.get("steps", args.extra_steps),
                                   ew.get("warmup", 3), local_rank)
                del keep
                extra[name] = {k: em[k] for k in ("value", "unit", "ms_per_step", "fwd_ms", "bwd_ms", "mode", "dtype",
                                                  "rows_per_s_per_gpu", "steps", "warmup")}
                extra[name]["l2"] = em["config"]["l2"]
                extra[name]["workload"] = WORKLOADS[name]["desc"]
                extra[name]["roofline_frac_bwd"] = em["roofline"]["frac"]
                extra[name]["roofline_frac_fwd_plus_bwd"] = em["roofline"]["fwd_plus_bwd"]["frac"]
                extra[name]["kernels"] = [em["roofline"]["forward_kernel"], em["roofline"]["kernel"]]
                extra[name]["clocks"] = em["clocks"]
            except RuntimeError as e:  # e.g. a device too small for the largest configuration
                extra[name] = {"error": str(e).splitlines()[0][:200]}
            torch.cuda.empty_cache()
            if world > 1:
                dist.barrier()
        line["workloads"] = extra

    if rank == 0 and world == 1 and not args.no_cpu and not layers:
        base, _, _ = cpu_port_rows_per_s(wl)
        line["cpu_baseline"] = base
        lit = cpu_literal_rows_per_s()
        if lit is not None:
            line["cpu_reference_literal"] = lit
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_e2e(ncn, wl, dev, dtype, ws, mode, world, rank):
    """Same metric through the host-buffer entry: inputs in pinned host memory, results back in
    pinned host memory, all copies inside the timed region.  Every rank pushes its own rows through
    its own GPU at the same time; the time is the slowest rank's, the weight gradients are summed
    over the ranks once per step as in the device-resident run."""
    import torch.distributed as dist

    from ncn_cuda_b200.host import net_fwd_bwd_host

    B, N = wl["B"], wl["N"]
    g = torch.Generator().manual_seed(wl["seed"] + 1000 * rank)
    ok, err = 1, ""
    try:  # eight pinned tensors of the full batch per rank; a host that cannot pin them has no e2e number
        hx = torch.empty(B, N, 1, dtype=dtype).pin_memory()
        hx.copy_(torch.randn(B, N, 1, generator=g).to(dtype))
        hxa = torch.zeros(B, N, 1, dtype=dtype).pin_memory()
        hdy = torch.empty(B, N, 1, dtype=dtype).pin_memory()
        hdy.copy_(torch.randn(B, N, 1, generator=g).to(dtype))
        hdya = torch.zeros(B, N, 1, dtype=dtype).pin_memory()
        out = tuple(torch.empty(B, N, 1, dtype=dtype).pin_memory() for _ in range(4))
    except RuntimeError as e:
        ok, err = 0, str(e).splitlines()[0][:200]
    if world > 1:  # all ranks run it or none does (the repetitions contain a collective)
        flag = torch.tensor([ok], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = int(flag.item())
    if not ok:
        return {"value": None, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "not measured: pinned host buffers could not be allocated on every rank" + (": " + err if err else "")}
    W = torch.stack([p.detach() for p in ws])
    reps = 5

    def one():
        res = net_fwd_bwd_host(hx, hxa, W, hdy, hdya, 0.9, wl["act"], wl["n"], 1, out=out, backward_mode=mode, device=dev)
        if world > 1:  # the data-parallel exchange: one sum of the flat weight gradient
            dwd = res[4].to(dev)
            dist.all_reduce(dwd, op=dist.ReduceOp.SUM)
            res[4].copy_(dwd)

    one()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    # each repetition timed on its own, the median reported: the host side of this path (pinned
    # memory, PCIe root) is shared with other jobs and single repetitions can be disturbed
    times, walls = [], []
    for _ in range(reps):
        t0 = time.perf_counter()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        one()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        walls.append((time.perf_counter() - t0) * 1e3)
    ms = sorted(times)[len(times) // 2]
    wall = sorted(walls)[len(walls) // 2] * 1e-3
    if world > 1:
        t = torch.tensor([ms, wall], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, wall = float(t[0].item()), float(t[1].item())
    el = hx.element_size() * B * N
    return {"value": world * B / (ms * 1e-3), "unit": "rows/s", "h2d_bytes_per_step": world * 4 * el,
            "d2h_bytes_per_step": world * (4 * el + W.numel() * 4), "rows": world * B, "ms_per_step": ms,
            "wall_ms_per_step": wall * 1e3, "ms_each_repetition": [round(t, 2) for t in times],
            "ms_best_repetition": round(min(times), 2),
            "note": "host-buffer call (ncn_cuda_b200.host.net_fwd_bwd_host), chunked 3-stream pipeline on every GPU, median of 5 repetitions after one warm-up pass, max over ranks"}


def main():
    args = parse()
    wl = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, wl, rank)
        return
    if not torch.cuda.is_available():
        sys.exit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    if world != args.gpus and world > 1:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)
    run_b200(args, wl, rank, world, local_rank)


if __name__ == "__main__":
    main()
