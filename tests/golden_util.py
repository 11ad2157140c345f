"""Loader for the committed golden fixtures (tests/golden/*.npz)."""
import os

import numpy as np

from aristos_b200 import synth
from aristos_b200.config import KleosConfig

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
INT_KEYS = {"sequence_len", "hidden_size", "intermediate_size", "num_experts", "torch_dtype",
            "expert_top_k", "hidden_act", "drop_tokens", "mini_batch"}


def names():
    return sorted(f[:-4] for f in os.listdir(GOLDEN_DIR) if f.endswith(".npz"))


def load(name):
    z = np.load(os.path.join(GOLDEN_DIR, f"{name}.npz"))
    kw = {}
    for k, v in zip(z["cfg_keys"], z["cfg_vals"]):
        kw[str(k)] = int(v) if str(k) in INT_KEYS else float(v)
    cfg = KleosConfig(**kw)
    world = int(z["world"])
    bias = z["bias"] if z["bias"].size else None
    packed = [z[f"packed_{r}"] for r in range(world)]
    views = [synth.split_packed(cfg, p, world) for p in packed]
    expect = [{k: z[f"{k}_{r}"] for k in ("probs", "topk", "slots", "counts", "mcw", "out",
                                          "mean_prob", "mean_count", "gate_loss")
               if f"{k}_{r}" in z.files}
              for r in range(world)]
    return cfg, world, bias, packed, views, expect
