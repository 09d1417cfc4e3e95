"""CPU-only checks: the C-ABI library loads and exports what include/ncn_b200.h declares, host-side
logic (backward planning, row sharding, index map), and the data-parallel gradient sum on gloo ranks."""
import ctypes
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "ncn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ncn_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from ncn_cuda_b200 import _lib

    names = header_functions()
    assert len(names) >= 11
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_lib.SIGNATURES) == names  # the ctypes table binds exactly the header's functions
    loaded = _lib.load()
    assert loaded.ncn_version() >= 100
    assert loaded.ncn_status_string(1).decode().startswith("bad shape")
    # pure host arithmetic, no device needed
    assert loaded.ncn_ckpt_bytes(8, 64, 1, 6, 4, 0) == 1 * 2 * 8 * 64 * 4
    assert loaded.ncn_ckpt_bytes(8, 64, 1, 4, 4, 0) == 0
    assert loaded.ncn_ckpt_bytes(8, 64, 1, 4, 4, 8) == 1 * 2 * 8 * 64 * 4      # tape: the last state
    assert loaded.ncn_ckpt_bytes(8, 64, 1, 6, 4, 8) == 2 * 2 * 8 * 64 * 4
    # states the per-stage forward stores: one per 16 steps short of the last; with bf16 storage (dtype 1) the end state too
    one = 2 * 3 * 64 * 128 * 4
    assert loaded.ncn_stage_mid_bytes(3, 64, 128, 32, 0) == one
    assert loaded.ncn_stage_mid_bytes(3, 64, 128, 16, 0) == 0
    assert loaded.ncn_stage_mid_bytes(3, 64, 128, 64, 0) == 3 * one
    assert loaded.ncn_stage_mid_bytes(3, 64, 128, 16, 1) == one
    assert loaded.ncn_stage_mid_bytes(3, 64, 128, 32, 1) == 2 * one


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from ncn_cuda_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or eager fallback"):
        _lib.load()


def test_cpu_tensors_are_rejected():
    import ncn_cuda_b200 as ncn

    x = torch.randn(2, 8, 1)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ncn.ops.stage_fwd(x, x, torch.randn(2), 0.9, 0, 4, 1, 0)


def test_plan_backward():
    from ncn_cuda_b200.ncn_pytorch_wrapper_v2 import plan_backward

    f32, bf16 = torch.float32, torch.bfloat16
    assert plan_backward(f32, 4, 6, False, "auto") == (False, 4, False)      # 24 steps -> checkpoint every 4 stages
    assert plan_backward(f32, 8, 4, False, "auto") == (False, 2, False)
    assert plan_backward(f32, 2, 10, False, "auto") == (False, 8, False)
    assert plan_backward(f32, 4, 3, False, "auto") == (False, 0, False)      # 12 steps: nothing to store
    assert plan_backward(f32, 16, 4, False, "checkpoint") == (False, 1, False)
    assert plan_backward(f32, 4, 6, False, "invert") == (False, 0, False)
    assert plan_backward(bf16, 16, 4, False, "auto") == (False, 0, True)    # bf16 storage: the stored end state
    assert plan_backward(f32, 8, 4, True, "auto") == (False, 2, True)       # residual layer: stored states, no replay
    assert plan_backward(bf16, 16, 4, False, "recompute") == (True, 0, False)
    assert plan_backward(bf16, 16, 4, False, "tape") == (False, 0, True)   # 64 steps from the fp32 end state
    assert plan_backward(bf16, 16, 8, False, "tape") == (False, 4, True)
    assert plan_backward(f32, 8, 4, True, "tape") == (False, 2, True)
    assert plan_backward(f32, 4, 3, True, "tape") == (False, 0, True)
    with pytest.raises(ValueError):
        plan_backward(f32, 8, 4, True, "invert")
    with pytest.raises(ValueError):
        plan_backward(f32, 8, 4, False, "bogus")


def test_shard_rows_partition():
    from ncn_cuda_b200 import shard_rows

    for B in (1, 7, 64, 1_048_576):
        for world in (1, 2, 3, 8):
            spans = [shard_rows(B, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def test_index_map_matches_oracle():
    from ncn_cuda_b200 import group_pos_to_index_v2
    from oracle import ncn_oracle as O

    for N, n in [(64, 2), (48, 4), (36, 3), (256, 32)]:
        for stage in range(0, 9):
            ref = O.stage_index(N, n, stage)
            for g in range(N // n):
                got = group_pos_to_index_v2(N, n, stage, g, torch.arange(n))
                assert torch.equal(got, ref[g])
            assert group_pos_to_index_v2(N, n, stage, 1, 1, one_based=True) == int(ref[0, 0]) + 1
    with pytest.raises(AssertionError):
        group_pos_to_index_v2(30, 4, 0, 0, 0)


def test_activation_vocabulary():
    from ncn_cuda_b200 import ops

    assert ops.ACTIVATION_CODES == {"tanh": 0, "relu": 1, "sigmoid": 2, "linear": -1, "leaky-relu": 3}
    assert ops.activation_code("linear") == -1 and ops.activation_code(2) == 2
    from ncn_cuda_b200.ncn_pytorch_invertible import _activation_nr

    assert _activation_nr("tanh") == 0 and _activation_nr("anything") == -1
    assert _activation_nr("leaky-relu") == 3


WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from oracle import ncn_oracle as O
from ncn_cuda_b200 import allreduce_weight_grads, shard_rows
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
B, N, n, L = 12, 64, 4, 3
x, xa, ws, dy, dya = O.make_inputs(5, B, N, 1, L, 0.25, dya_zero=False)
b, e = shard_rows(B, rank, world)
_, _, dx, dxa, dWs = O.net_fwd_bwd(x[b:e], xa[b:e], ws, dy[b:e], dya[b:e], 0.9, "tanh", n, 1)
for deterministic in (False, True):
    params = [w.clone().requires_grad_() for w in ws]
    for p_, g in zip(params, dWs):
        p_.grad = g.clone()
    allreduce_weight_grads(params, deterministic=deterministic)
    _, _, fdx, _, fdW = O.net_fwd_bwd(x, xa, ws, dy, dya, 0.9, "tanh", n, 1)
    for p_, g in zip(params, fdW):
        assert O.rel_err(p_.grad, g) < 1e-5, (rank, deterministic)
    assert O.rel_err(dx, fdx[b:e]) < 1e-6          # rows are independent: dX needs no exchange
dist.destroy_process_group()
print("ok", rank)
"""


def test_gradient_sum_over_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29731", str(script), ROOT]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("ok") == 2


def test_bench_reference_arm_prints_contract_line():
    import json

    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] == "port" and line["value"] > 0
    assert "rows_per_gpu" in line["config"] and "backward_mode" in line["config"]  # the GPU arm's config keys
    if "cpu_reference_literal" in line:  # present where oracle/_ref/ holds the reference's torch_ref files
        assert line["cpu_reference_literal"]["kind"] == "reference" and line["cpu_reference_literal"]["value"] > 0


def test_host_pipeline_chunk_bounds():
    from ncn_cuda_b200.host import chunk_bounds

    for B, rows in [(65536, 4096), (100, 4096), (30000, 4096), (24576, 4096), (7, 2), (1, 1), (4097, 4096)]:
        b = chunk_bounds(B, rows)
        assert b[0][0] == 0 and b[-1][1] == B
        assert all(x[1] == y[0] for x, y in zip(b, b[1:]))          # contiguous, in order
        assert all(0 < e - s <= rows for s, e in b)                  # fit the device slots
    long = chunk_bounds(65536, 4096)
    assert long[0] == (0, 1024) and long[-1] == (64512, 65536)       # short chunks at both ends
