"""Generates the committed golden fixtures from the NumPy oracle.

    python tests/golden/make_golden.py

Each fixture holds the packed, dtype-rounded inputs of every rank of a tiny layer and the
oracle's outputs for them, so that the tests do not depend on the random generator of the NumPy
version that happens to be installed.  The reference project has no golden vectors of its own
(no test suite, no expected outputs anywhere in its tree), so these pin the two oracle
implementations and the CUDA path against each other, not against the reference.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from aristos_b200 import synth  # noqa: E402
from aristos_b200.config import KleosConfig  # noqa: E402
from oracle import moe_oracle  # noqa: E402

CASES = {
    "fp32_w1": (dict(sequence_len=128, hidden_size=64, intermediate_size=128, num_experts=8,
                     torch_dtype=0), 1, None),
    "bf16_w1": (dict(sequence_len=128, hidden_size=64, intermediate_size=128, num_experts=8,
                     torch_dtype=2), 1, None),
    "bf16_w2_zipf": (dict(sequence_len=128, hidden_size=64, intermediate_size=64, num_experts=8,
                          torch_dtype=2, capacity_factor=1.25), 2, 1.2),
    "fp32_top1": (dict(sequence_len=128, hidden_size=64, intermediate_size=64, num_experts=4,
                       torch_dtype=0, expert_top_k=1), 1, None),
    # later additions carry a fourth entry: the standard deviation of the FFN biases
    "tf32_gelu_biased": (dict(sequence_len=128, hidden_size=64, intermediate_size=128, num_experts=8,
                              torch_dtype=1, hidden_act=1), 1, None, 0.5),
    "fp16_biased": (dict(sequence_len=128, hidden_size=64, intermediate_size=64, num_experts=16,
                         torch_dtype=3), 1, None, 0.5),
}
STAT_KEYS = ("mean_prob", "mean_count", "gate_loss")  # training-mode gate statistics


def build_case(name):
    kw, world, zipf = CASES[name][:3]
    bias_scale = CASES[name][3] if len(CASES[name]) > 3 else 0.0
    cfg = KleosConfig(**kw)
    packed = [synth.packed_input(cfg, r, world, bias_scale=bias_scale) for r in range(world)]
    views = [synth.split_packed(cfg, p, world) for p in packed]
    bias = synth.zipf_gate_bias(cfg, zipf) * 2.0 if zipf else None
    res = moe_oracle.moe_forward(cfg, world, views, gate_bias=bias)
    out = dict(world=np.int32(world), cfg_keys=np.array(list(kw.keys())),
               cfg_vals=np.array([float(v) for v in kw.values()]),
               bias=np.zeros(0, np.float32) if bias is None else bias)
    for r in range(world):
        out[f"packed_{r}"] = packed[r]
        for k in ("probs", "topk", "slots", "counts", "mcw", "out"):
            out[f"{k}_{r}"] = res[r][k]
        if bias_scale:  # the newer fixtures also pin the gate statistics
            for k in STAT_KEYS:
                out[f"{k}_{r}"] = np.asarray(res[r][k], dtype=np.float64)
    return out


def main():
    for name in CASES:
        path = os.path.join(HERE, f"{name}.npz")
        if os.path.exists(path) and "--all" not in sys.argv:
            continue  # committed fixtures are only rewritten on request
        np.savez_compressed(path, **build_case(name))
        print(path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
