"""Benchmark of the NCN fused forward + backward (the one hot path of this repository).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One step = one fused forward + one fused backward (incl. the fixed-order dW reduction and, for
N > 1, the NCCL sum of dW) over one batch of synthetic rows.  With N > 1 (launched by torchrun,
one rank per GPU) every rank runs the same per-GPU workload on its own rows (weak scaling) and
`value` is the whole-job rows/s from the slowest rank's device time.

`--impl reference` times the CPU restatement of the reference's torch_ref path (oracle/) on the
host cores instead; rank 0 only.
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
    "ref_e128": dict(B=4096, N=256, E=128, C=4, n=32, L=3, w_var=1 / 32, dtype="f32", act="tanh", seed=5,
                     desc="the reference's own bench shape scaled in rows: x[4096,256,128] 4 heads g=32 3 stages, one kernel per stage"),
    "ref_e128_small": dict(B=1024, N=256, E=128, C=4, n=32, L=3, w_var=1 / 32, dtype="f32", act="tanh", seed=5,
                           desc="ref_e128 with 1024 rows (profiling case)"),
    "small": dict(B=8192, N=4096, n=4, L=6, w_var=0.25, dtype="f32", act="tanh", seed=1,
                  desc="cfg2 with 8192 rows (profiling case)"),
}

# DRAM bytes per element moved by the backward kernel in one launch, from the ncu capture
# summarised in profiles/ (dram__bytes_read.sum + dram__bytes_write.sum over B*N); None until measured.
BWD_TRAFFIC_BYTES_PER_ELEMENT = 31.39  # profiles/pair_kernels_cfg2_small_ncu_full.md: 1053.2 MB over 33.55 M elements


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
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
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


# ------------------------------------------------------------------ CPU arm (oracle)
def cpu_rows_per_s(wl, seconds, threads=None, rows=None):
    """Vectorised torch-CPU restatement of the reference's torch_ref path, forward + autograd
    backward, on a bounded sample of the workload's rows."""
    from oracle import ncn_oracle as O

    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    fixed = rows is not None
    if not fixed:  # first call: spin up the thread pool and autograd before anything is timed
        xw, xaw, wsw, dyw, dyaw = O.make_inputs(wl["seed"], 4, wl["N"], wl.get("E", 1), wl["L"], wl["w_var"])
        O.net_fwd_bwd(xw, xaw, wsw, dyw, dyaw, 0.9, wl["act"], wl["n"], wl.get("C", 1))
    rows = rows or 8
    dt_run = 0.0
    while True:
        x, xa, ws, dy, dya = O.make_inputs(wl["seed"], rows, wl["N"], wl.get("E", 1), wl["L"], wl["w_var"])
        t0 = time.perf_counter()
        O.net_fwd_bwd(x, xa, ws, dy, dya, 0.9, wl["act"], wl["n"], wl.get("C", 1))
        dt_run = time.perf_counter() - t0
        if fixed or dt_run >= seconds / 3 or rows >= wl["B"] or rows >= 4096:
            break
        rows = min(wl["B"], max(rows * 2, int(rows * (seconds / 2) / max(dt_run, 1e-3))))
    return rows / dt_run, threads, rows, dt_run


def run_reference(args, wl, rank):
    if rank != 0:
        return
    per_step = []
    rows = None
    for i in range(args.warmup + args.steps):
        v, threads, rows, dt = cpu_rows_per_s(wl, args.cpu_seconds / max(1, args.steps), rows=rows)
        if i >= args.warmup:
            per_step.append((rows, dt))
    tot_rows = sum(r for r, _ in per_step)
    tot_t = sum(t for _, t in per_step)
    value = tot_rows / tot_t
    sample = f"{rows} of {wl['B']} rows of the workload per step, vectorised torch-CPU restatement of torch_ref, forward + autograd backward"
    line = {
        "impl": "reference", "metric": "ncn_fwd_bwd_rows_per_s", "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * tot_t / max(1, len(per_step)),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": {"workload": wl["desc"], "rows": wl["B"], "D": wl["N"], "g": wl["n"], "stages": wl["L"],
                   "activation": wl["act"]},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
def run_b200(args, wl, rank, world, local_rank):
    import torch.distributed as dist

    import ncn_cuda_b200 as ncn
    from oracle import ncn_oracle as O  # used by the cpu_baseline leg only

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    dtype = torch.float32 if wl["dtype"] == "f32" else torch.bfloat16
    w = 4 if wl["dtype"] == "f32" else 2
    B, N, n, L = wl["B"], wl["N"], wl["n"], wl["L"]
    E, C = wl.get("E", 1), wl.get("C", 1)
    mode = args.mode or wl.get("mode", "auto")
    g = torch.Generator(device=dev).manual_seed(wl["seed"] + 1000 * rank)
    x = torch.randn(B, N, E, generator=g, device=dev, dtype=torch.float32).to(dtype).requires_grad_(True)
    xa = torch.zeros(B, N, E, device=dev, dtype=dtype).requires_grad_(True)
    dy = torch.randn(B, N, E, generator=g, device=dev, dtype=torch.float32).to(dtype)
    dya = torch.zeros(B, N, E, device=dev, dtype=dtype)
    gw = torch.Generator().manual_seed(wl["seed"])
    layers = wl.get("layers", 0)
    if layers:
        net = ncn.NCNResidualStack(layers, 0.9, wl["act"], n, 1, L, 1, w_std=wl["w_var"] ** 0.5,
                                   backward_mode="recompute" if mode == "auto" else mode).to(dev)
        ws = [net.weight]
    else:
        ws = [(torch.randn(2 * E, generator=gw) * wl["w_var"] ** 0.5).to(dev).requires_grad_(True) for _ in range(L)]
        net = ncn.NCNNetTestCuda(0.9, wl["act"], n, C, L, ws, backward_mode=mode)

    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]

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

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local_rank) as clocks:
        t_start = torch.cuda.Event(enable_timing=True); t_end = torch.cuda.Event(enable_timing=True)
        t_start.record()
        for i in range(args.steps):
            step(i)
        t_end.record()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ncn.ops.device_status()
    ms = t_start.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
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
    elems = B * N * E * max(1, layers) * (L if per_stage else 1)
    bwd_bytes = 6 * w * elems  # reads y, ya, dy, dya; writes dx, dxa
    bwd_gbs = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    step_gbs = 10 * w * elems / ((fwd_ms + bwd_ms) * 1e-3) / 1e9
    roofline = {
        "bound": "hbm", "kernel": ("feat_bwd_kernel (ncn_feat.cuh), %d launches per step" % L if per_stage
                                   else "pair_bwd_dual_kernel (ncn_pairs.cuh)" if n <= 8 and mode != "recompute" and not (dtype != torch.float32 and mode == "auto")
                                   else "rows_bwd_kernel / pair_bwd_wide_kernel"), "achieved": bwd_gbs, "peak": peak, "peak_source": peak_src,
        "unit": "GB/s", "frac": bwd_gbs / peak, "ms_per_launch": bwd_ms / (L if per_stage else 1),
        # measured on the cfg2 shape (fp32, one checkpoint); traffic grows in proportion to the rows
        "traffic": (BWD_TRAFFIC_BYTES_PER_ELEMENT * elems if args.workload in ("cfg2", "small") and mode == "auto" else None),
        "algorithmic_bytes": bwd_bytes // (L if per_stage else 1),
        "fwd_plus_bwd": {"achieved": step_gbs, "frac": step_gbs / peak, "frac_of_8TBs_nominal": step_gbs / 8000.0,
                         "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "algorithmic_bytes": 10 * w * elems},
        "note": "issue-bound kernel (n*L dependent tanh steps per element); HBM fraction reported as the metric asks",
    }

    line = {
        "metric": "ncn_fwd_bwd_rows_per_s", "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": {"workload": wl["desc"], "rows_per_gpu": B, "D": N, "E": E, "heads": C, "g": n, "stages": L, "activation": wl["act"],
                   "backward_mode": mode, "parallelism": f"dp{world}", "l2": "inputs larger than L2 (%.2f GB per tensor)" % (B * N * E * w / 1e9)},
        "roofline": roofline, "gpu_launches": (3 * L if per_stage else 3) * args.steps * max(1, layers), "clocks": clocks.summary(),
        "rows_per_s_per_gpu": value / world,
    }

    if not args.no_e2e and not layers and not per_stage:
        e2e = run_e2e(ncn, wl, dev, dtype, ws, mode, world, rank)  # every rank: its rows through its own host buffers
        if rank == 0:
            line["e2e"] = e2e
    if world > 1:
        dist.barrier()
    if rank == 0 and world == 1 and not args.no_cpu and not layers:
        v, threads, rows, dt = cpu_rows_per_s(wl, args.cpu_seconds)
        line["cpu_baseline"] = {
            "value": v, "unit": "rows/s", "cores": threads, "kind": "port",
            "sample": f"{rows} of {B} rows, vectorised torch-CPU restatement of torch_ref, forward + autograd backward, {dt:.1f} s",
        }
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
    reps = 3

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
            "note": "host-buffer call (ncn_cuda_b200.host.net_fwd_bwd_host), chunked 3-stream pipeline on every GPU, median of 3 repetitions, max over ranks"}


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
