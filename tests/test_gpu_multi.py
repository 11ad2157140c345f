"""Expert-parallel parity on 2+ GPUs: every rank's routing and layer output against the CPU
oracle evaluated on the global problem.  Skipped on boxes with fewer GPUs.

Every case runs several forwards with DIFFERENT activations per forward (same weights) and
checks the last one, so a kernel that consumed a dispatched cell, a returned row, a count or a
flag left over from the forward before cannot pass; one case also lets a rank sleep on the host
between forwards so that the ranks enter their forwards skewed in time."""
import json
import os
import subprocess
import sys
from dataclasses import asdict

import numpy as np
import pytest

from aristos_b200 import synth
from aristos_b200.config import KleosConfig, baseline_config
from oracle import c_oracle, moe_oracle
from tests import moe_harness as hz

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ACT_SEEDS = [3000, 1000, 2000]  # one per forward; the last one is checked
# the two arrangements of the 16-bit routed layer: separate launches (default) and KLEOS_FLOW=1
ARR = {"launches": {}, "persistent": {"KLEOS_FLOW": "1"}}


def _run_world(tmp_path, cfg, world, bias=None, act_seeds=ACT_SEEDS, port=29611, extra_env=None,
               rows=None, sleep=None, mode="device", timeout=900):
    spec = dict(cfg=asdict(cfg), seed=0, act_seeds=list(act_seeds), mode=mode, sleep=sleep,
                rows=None if rows is None else [int(r) for r in rows],
                bias=None if bias is None else [float(b) for b in bias])
    sp = tmp_path / "spec.json"
    sp.write_text(json.dumps(spec))
    env = dict(os.environ, KLEOS_WAIT_MS="3000", NCCL_NVLS_ENABLE="0")
    env.pop("KLEOS_FLOW", None)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "multirank_worker.py"), str(sp), str(tmp_path)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]


def _views(cfg, world, act_seed):
    """Every rank's packed sections with the weights of seed 0 and the activations of act_seed."""
    views = []
    for r in range(world):
        v = synth.split_packed(cfg, synth.packed_input(cfg, r, world), world)
        v["A"] = synth.round_to_dtype(synth.activations(cfg, r, act_seed), cfg.torch_dtype)
        views.append(v)
    return views


def _check_rank(cfg, ref, got, r, rows=None):
    assert got["status"][0] == 0, f"rank {r} device status {got['status']}"
    routing = {k: got[k] for k in ("topk", "slots", "counts", "mcw")}
    out = got["out"]
    if rows is not None:  # the worker saved only the sampled rows: put them where the checker looks
        full = np.zeros((cfg.S, cfg.H), dtype=np.float32)
        full[rows] = out
        out = full
    return hz.check_against_oracle(cfg, ref, got["probs"], out, routing, rows=rows)


@pytest.mark.parametrize("arr", ["launches", "persistent"])
@pytest.mark.parametrize("dtype,world", [(2, 2), (0, 2), (2, 4), (2, 8)])
def test_expert_parallel_parity(tmp_path, gpu_count, dtype, world, arr):
    if gpu_count < world:
        pytest.skip(f"needs {world} GPUs")
    if arr == "persistent" and dtype == 0:
        pytest.skip("float layers never run the persistent kernel")
    cfg = KleosConfig(sequence_len=256, hidden_size=512, intermediate_size=1024, num_experts=8,
                      torch_dtype=dtype)
    ref = moe_oracle.moe_forward(cfg, world, _views(cfg, world, ACT_SEEDS[-1]))
    got = _run_world(tmp_path, cfg, world, port=29611 + world + dtype, extra_env=ARR[arr])
    for r in range(world):
        _check_rank(cfg, ref[r], got[r], r)


@pytest.mark.parametrize("arr", ["launches", "persistent"])
def test_expert_parallel_skewed_routing(tmp_path, gpu_count, arr):
    """Hot experts, drops and experts that receive nothing from some rank."""
    world = 2
    if gpu_count < world:
        pytest.skip("needs 2 GPUs")
    cfg = KleosConfig(sequence_len=512, hidden_size=256, intermediate_size=256, num_experts=16,
                      torch_dtype=2, capacity_factor=1.25)
    bias = synth.zipf_gate_bias(cfg, 1.2) * 2.0
    ref = moe_oracle.moe_forward(cfg, world, _views(cfg, world, ACT_SEEDS[-1]), gate_bias=bias)
    got = _run_world(tmp_path, cfg, world, bias=bias, port=29631, extra_env=ARR[arr])
    for r in range(world):
        _check_rank(cfg, ref[r], got[r], r)


@pytest.mark.parametrize("arr", ["launches", "persistent"])
@pytest.mark.parametrize("mode", ["device", "host"])
def test_ranks_skewed_in_time_with_new_tokens_every_forward(tmp_path, gpu_count, mode, arr):
    """Six forwards, new tokens each time, rank 1 sleeping 5 ms on the host before each of its
    forwards: rank 0 finishes dispatching forward n+1 while rank 1 has not yet entered it."""
    world = 2
    if gpu_count < world:
        pytest.skip("needs 2 GPUs")
    cfg = KleosConfig(sequence_len=1024, hidden_size=512, intermediate_size=512, num_experts=16,
                      torch_dtype=2)
    seeds = [100, 200, 300, 400, 500, 600]
    ref = moe_oracle.moe_forward(cfg, world, _views(cfg, world, seeds[-1]))
    got = _run_world(tmp_path, cfg, world, act_seeds=seeds, port=29641 + (mode == "host"),
                     sleep=dict(rank=1, ms=5), mode=mode, extra_env=ARR[arr])
    for r in range(world):
        _check_rank(cfg, ref[r], got[r], r)


BASELINE_CASES = [("C3", 2, "launches"), ("C3", 2, "persistent"), ("C5", 2, "persistent"),
                  ("C3", 4, "launches"), ("C3", 4, "persistent"), ("C5", 4, "persistent"),
                  ("C3", 8, "launches"), ("C3", 8, "persistent"), ("C4", 8, "persistent"),
                  ("C5", 8, "launches")]


@pytest.mark.parametrize("name,world,arr", BASELINE_CASES, ids=[f"{n}-w{w}-{a}" for n, w, a in BASELINE_CASES])
def test_benchmark_layers_expert_parallel(tmp_path, gpu_count, name, world, arr):
    """The benchmark layers at the world sizes they are quoted on: routing of every token of
    every rank bit-exact, layer output of a seeded sample of 64 tokens per rank within the bf16
    tolerance (the oracle's FFN is evaluated only for the sampled tokens)."""
    if gpu_count < world:
        pytest.skip(f"needs {world} GPUs")
    cfg, extra = baseline_config(name)
    bias = synth.zipf_gate_bias(cfg, extra["zipf"]) if extra["zipf"] else None
    rng = np.random.default_rng(7)
    rows = np.sort(rng.choice(cfg.S, size=64, replace=False)).astype(np.int32)
    seeds = ACT_SEEDS[1:]  # two forwards with different tokens
    got = _run_world(tmp_path, cfg, world, bias=bias, act_seeds=seeds, rows=rows,
                     port=29700 + 10 * world + int(name[1]), timeout=1500, extra_env=ARR[arr])
    views = _views(cfg, world, seeds[-1])
    c_oracle.use_all_cores()
    worst = 0.0
    for r in range(world):
        ref = c_oracle.moe_forward_rank(cfg, world, r, views, gate_bias=bias, tokens=rows)
        worst = max(worst, _check_rank(cfg, ref, got[r], r, rows=rows))
    print(f"{name} on {world} GPUs ({arr}): routing bit-exact on {world * cfg.S} tokens, "
          f"worst sampled output error {worst:.3e}")
