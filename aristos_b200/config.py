"""Layer configuration: the keys of ``kleos_config.json`` and the sizes derived from them.

Mirrors the compile-time ``ACC`` struct of the reference (csrc/include/kleos/types.cuh:442-513)
as run-time arithmetic; the C++ host layer (csrc/config.hpp) computes the same numbers and
``tests/test_config_abi.py`` checks that the two agree.  Key names and enum values follow
csrc/kleos_config.schema.json:5-89.

Two documented extensions over the reference schema:
  * ``capacity_factor`` may be any number >= 1 (the schema says integer, schema.json:6-10);
    ``EC = ceil(ceil(S/E) * CF) * k`` equals the reference's product for integer CF
    (types.cuh:498-499).
  * an optional per-expert gate bias added to the logits (the reference gate has none,
    moe/gate.cuh:87-88); it is supplied through ``kleos_set_gate_bias`` and not stored in the
    JSON file.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, asdict

BLOCK_M = 128  # row granularity of expert cells and task tiles (types.cuh:38-42)
BLOCK_N = 64   # the gate pads the expert dimension to a multiple of this (types.cuh:481)

DTYPE_NAMES = {0: "fp32", 1: "tf32", 2: "bf16", 3: "fp16"}
DTYPE_BYTES = {0: 4, 1: 4, 2: 2, 3: 2}
SUPPORTED_DTYPES = (0, 1, 2, 3)

REQUIRED_KEYS = (
    "capacity_factor", "drop_tokens", "expert_top_k", "is_training", "hidden_act",
    "hidden_size", "intermediate_size", "mini_batch", "moe_frequency", "num_experts",
    "num_layers", "sequence_len", "torch_dtype", "vocab_size",
)


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


@dataclass
class KleosConfig:
    capacity_factor: float = 1
    drop_tokens: int = 1
    expert_top_k: int = 2
    global_batch: int = 256
    is_training: int = 0
    hidden_act: int = 0
    hidden_size: int = 2048
    intermediate_size: int = 2048
    mini_batch: int = 1
    moe_frequency: int = 1
    num_experts: int = 64
    num_layers: int = 1
    sequence_len: int = 8192
    torch_dtype: int = 2
    vocab_size: int = 32000

    # ------------------------------------------------------------------ derived sizes
    @property
    def S(self) -> int:
        """Tokens per rank (types.cuh:471)."""
        return self.sequence_len * self.mini_batch

    @property
    def H(self) -> int:
        return self.hidden_size

    @property
    def I(self) -> int:  # noqa: E743 - the reference calls it P (types.cuh:472)
        return self.intermediate_size

    @property
    def E(self) -> int:
        return self.num_experts

    @property
    def K(self) -> int:
        return self.expert_top_k

    @property
    def PX(self) -> int:
        """Expert dimension padded to the gate tile width (types.cuh:481)."""
        return _ceil_div(self.E, BLOCK_N) * BLOCK_N

    @property
    def EC(self) -> int:
        """Expert capacity per (source rank, expert) (types.cuh:498-499)."""
        base = self.S if not self.drop_tokens else _ceil_div(self.S, self.E)
        return int(math.ceil(base * float(self.capacity_factor) - 1e-9)) * self.K

    @property
    def pEC(self) -> int:
        """Capacity padded to whole 128-row tiles (types.cuh:500)."""
        return _ceil_div(self.EC, BLOCK_M) * BLOCK_M

    @property
    def elem_bytes(self) -> int:
        return DTYPE_BYTES[self.torch_dtype]

    @property
    def dtype_name(self) -> str:
        return DTYPE_NAMES[self.torch_dtype]

    @property
    def dense(self) -> bool:
        """A single-expert layer is the plain FFN (the reference switches kernels at E == 1,
        moe/moe.cuh:174-177): no gate weight in the packed input, no probabilities in the
        packed output (moe/fffn.cuh:47-53), and every rank holds the one expert."""
        return self.E == 1

    def local_experts(self, world: int) -> int:
        return 1 if self.dense else self.E // world

    def owner(self, expert: int, world: int) -> int:
        """Contiguous even sharding (bootstrap.cuh:48-51)."""
        return expert // (self.E // world)

    # packed buffer sizes in elements (moe.cuh:92-98, main.cu:17-30)
    def input_elems(self, world: int) -> int:
        nlx = self.local_experts(world)
        gate = 0 if self.dense else self.PX * self.H
        return self.S * self.H + gate + 2 * nlx * self.I * self.H + nlx * (self.I + self.H)

    def output_elems(self) -> int:
        return (0 if self.dense else self.S * self.PX) + self.S * self.H

    def input_offsets(self, world: int) -> dict:
        """Element offsets of the sections of the packed input buffer."""
        nlx = self.local_experts(world)
        a = 0
        wg = a + self.S * self.H
        w1 = wg + (0 if self.dense else self.PX * self.H)
        w2 = w1 + nlx * self.I * self.H
        b1 = w2 + nlx * self.H * self.I
        b2 = b1 + nlx * self.I
        end = b2 + nlx * self.H
        return dict(A=a, Wg=wg, W1=w1, W2=w2, b1=b1, b2=b2, end=end)

    # ------------------------------------------------------------------ validation / io
    def validate(self, world: int = 1) -> None:
        if self.torch_dtype not in DTYPE_NAMES:
            raise ValueError(f"torch_dtype {self.torch_dtype} not in {{0,1,2,3}}")
        if self.hidden_act not in (0, 1):
            raise ValueError("hidden_act must be 0 (relu) or 1 (gelu)")
        if self.hidden_size % 64 or self.intermediate_size % 64:
            raise ValueError("hidden_size and intermediate_size must be multiples of 64")
        if self.sequence_len % 128:
            raise ValueError("sequence_len must be a multiple of 128")
        if self.expert_top_k < 1 or self.expert_top_k > self.num_experts:
            raise ValueError("expert_top_k must be in [1, num_experts]")
        if self.num_experts < 1 or self.num_experts > 65535:
            raise ValueError("num_experts must be in [1, 65535]")
        if float(self.capacity_factor) < 1:
            raise ValueError("capacity_factor must be >= 1")
        if world < 1 or (not self.dense and self.num_experts % world):
            raise ValueError("num_experts must divide evenly over the world size")

    def to_json(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(asdict(self), f, indent=2)

    @classmethod
    def from_json(cls, path: str) -> "KleosConfig":
        with open(path) as f:
            raw = json.load(f)
        missing = [k for k in REQUIRED_KEYS if k not in raw]
        if missing:
            raise ValueError(f"kleos config is missing required keys: {missing}")
        known = {k: raw[k] for k in cls.__dataclass_fields__ if k in raw}
        return cls(**known)


def baseline_config(name: str) -> tuple[KleosConfig, dict]:
    """The five benchmark layers, by name C1..C5, plus their extras
    (world sizes they are quoted on, whether a Zipf gate bias is applied)."""
    n = name.upper()
    if n == "C1":
        return KleosConfig(sequence_len=256, hidden_size=512, intermediate_size=1024,
                           num_experts=8, torch_dtype=0), dict(worlds=(1,), zipf=None)
    if n == "C2":
        return KleosConfig(sequence_len=4096, hidden_size=2048, intermediate_size=2048,
                           num_experts=16, torch_dtype=0), dict(worlds=(1,), zipf=None)
    if n == "C3":
        return KleosConfig(sequence_len=8192, hidden_size=2048, intermediate_size=2048,
                           num_experts=64, torch_dtype=2), dict(worlds=(1, 2, 4, 8), zipf=None)
    if n == "C4":
        return KleosConfig(sequence_len=16384, hidden_size=2048, intermediate_size=2048,
                           num_experts=128, torch_dtype=2, capacity_factor=1.25), \
            dict(worlds=(8,), zipf=1.2)
    if n == "C5":
        return KleosConfig(sequence_len=4096, hidden_size=4096, intermediate_size=14336,
                           num_experts=8, torch_dtype=2), dict(worlds=(1, 2, 4, 8), zipf=None)
    raise KeyError(name)
