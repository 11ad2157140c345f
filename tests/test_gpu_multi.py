"""Expert-parallel parity on 2+ GPUs: every rank's routing and layer output against the CPU
oracle evaluated on the global problem.  Skipped on boxes with fewer GPUs."""
import json
import os
import subprocess
import sys
from dataclasses import asdict

import numpy as np
import pytest

from aristos_b200 import synth
from aristos_b200.config import KleosConfig
from oracle import moe_oracle
from tests import moe_harness as hz

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_world(tmp_path, cfg, world, bias=None, forwards=2, port=29611, extra_env=None):
    spec = dict(cfg=asdict(cfg), forwards=forwards, seed=0,
                bias=None if bias is None else [float(b) for b in bias])
    sp = tmp_path / "spec.json"
    sp.write_text(json.dumps(spec))
    env = dict(os.environ, KLEOS_WAIT_MS="2000", NCCL_NVLS_ENABLE="0", **(extra_env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "multirank_worker.py"), str(sp), str(tmp_path)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]


@pytest.mark.parametrize("dtype,world", [(2, 2), (0, 2), (2, 4), (2, 8)])
def test_expert_parallel_parity(tmp_path, gpu_count, dtype, world):
    if gpu_count < world:
        pytest.skip(f"needs {world} GPUs")
    cfg = KleosConfig(sequence_len=256, hidden_size=512, intermediate_size=1024, num_experts=8,
                      torch_dtype=dtype)
    views = [synth.split_packed(cfg, synth.packed_input(cfg, r, world), world) for r in range(world)]
    ref = moe_oracle.moe_forward(cfg, world, views)
    got = _run_world(tmp_path, cfg, world, port=29611 + world + dtype)
    for r in range(world):
        assert got[r]["status"][0] == 0, f"rank {r} device status {got[r]['status']}"
        routing = {k: got[r][k] for k in ("topk", "slots", "counts", "mcw")}
        hz.check_against_oracle(cfg, ref[r], got[r]["probs"], got[r]["out"], routing)


def test_expert_parallel_skewed_routing(tmp_path, gpu_count):
    """Hot experts, drops and experts that receive nothing from some rank."""
    world = 2
    if gpu_count < world:
        pytest.skip("needs 2 GPUs")
    cfg = KleosConfig(sequence_len=512, hidden_size=256, intermediate_size=256, num_experts=16,
                      torch_dtype=2, capacity_factor=1.25)
    bias = synth.zipf_gate_bias(cfg, 1.2) * 2.0
    views = [synth.split_packed(cfg, synth.packed_input(cfg, r, world), world) for r in range(world)]
    ref = moe_oracle.moe_forward(cfg, world, views, gate_bias=bias)
    got = _run_world(tmp_path, cfg, world, bias=bias, forwards=3, port=29631)
    for r in range(world):
        assert got[r]["status"][0] == 0
        routing = {k: got[r][k] for k in ("topk", "slots", "counts", "mcw")}
        hz.check_against_oracle(cfg, ref[r], got[r]["probs"], got[r]["out"], routing)


EXPERIMENTAL = pytest.mark.skipif(os.environ.get("KLEOS_TEST_EXPERIMENTAL") != "1",
                                  reason="opt-in code paths: set KLEOS_TEST_EXPERIMENTAL=1")


@EXPERIMENTAL
@pytest.mark.parametrize("world", [2, 8])
def test_overlapped_dispatch_mode(tmp_path, gpu_count, world):
    """KLEOS_OVERLAP=1: per-cell flagged dispatch on the copy stream beside a GEMM1 that plans in
    its prologue and waits per cell.  Same results as the default path are required."""
    if gpu_count < world:
        pytest.skip(f"needs {world} GPUs")
    cfg = KleosConfig(sequence_len=512, hidden_size=512, intermediate_size=1024, num_experts=16,
                      torch_dtype=2)
    views = [synth.split_packed(cfg, synth.packed_input(cfg, r, world), world) for r in range(world)]
    ref = moe_oracle.moe_forward(cfg, world, views)
    got = _run_world(tmp_path, cfg, world, forwards=3, port=29651 + world,
                     extra_env=dict(KLEOS_OVERLAP="1"))
    for r in range(world):
        assert got[r]["status"][0] == 0, f"rank {r} device status {got[r]['status']}"
        routing = {k: got[r][k] for k in ("topk", "slots", "counts", "mcw")}
        hz.check_against_oracle(cfg, ref[r], got[r]["probs"], got[r]["out"], routing)
