"""Seeded synthetic inputs for the MoE layer, packed the way the reference driver packs them.

The reference driver (csrc/main.cu:17-66) builds one packed buffer
``[A | Wg | W1 | W2 | b1 | b2]`` in fp32, converts it in place to the layer's element type and
copies it to the device.  This module builds the same buffer from a counter-based generator
(NumPy Philox keyed by seed and stream), with the distributions the benchmark configs name:
activations N(0,1) seeded by ``seed + rank``; gate and expert weights N(0, 1/sqrt(fan_in))
seeded by ``seed`` and depending only on the expert's global id, so every world size sees
the same experts; zero biases.  The reference's own driver draws N(0,5) for everything with
a rank-dependent seed (main.cu:42-43); the shapes and packing are the same.
"""
from __future__ import annotations

import numpy as np

from .config import KleosConfig

_STREAM_ACT, _STREAM_GATE, _STREAM_W1, _STREAM_W2, _STREAM_PERM, _STREAM_B1, _STREAM_B2 = 1, 2, 3, 4, 5, 6, 7


def _normal(seed: int, stream: int, index: int, n: int) -> np.ndarray:
    gen = np.random.Generator(np.random.Philox(key=[(seed << 8) | stream, index]))
    return gen.standard_normal(n, dtype=np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bf16 (ties to even), returned as fp32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    r = (u + 0x7FFF + lsb) & 0xFFFF0000
    return r.astype(np.uint32).view(np.float32)


def round_tf32(x: np.ndarray) -> np.ndarray:
    """Round fp32 to TF32 (10-bit mantissa, ties to even), returned as fp32 words."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0xFFF) + ((u >> np.uint32(13)) & np.uint32(1))) & np.uint32(0xFFFFE000)
    return r.astype(np.uint32).view(np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> uint16 bf16 bit patterns (round to nearest even)."""
    return (round_bf16(x).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def round_to_dtype(x: np.ndarray, torch_dtype: int) -> np.ndarray:
    if torch_dtype == 0:
        return np.asarray(x, dtype=np.float32)
    if torch_dtype == 1:
        return round_tf32(x)
    if torch_dtype == 2:
        return round_bf16(x)
    if torch_dtype == 3:
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)
    raise NotImplementedError(f"torch_dtype {torch_dtype}")


def activations(cfg: KleosConfig, rank: int, seed: int = 0) -> np.ndarray:
    return _normal(seed + rank, _STREAM_ACT, 0, cfg.S * cfg.H).reshape(cfg.S, cfg.H)


def gate_weight(cfg: KleosConfig, seed: int = 0) -> np.ndarray:
    """Wg[e][h]; row e belongs to expert e."""
    w = _normal(seed, _STREAM_GATE, 0, cfg.E * cfg.H).reshape(cfg.E, cfg.H)
    return w * np.float32(1.0 / np.sqrt(cfg.H))


def expert_weights(cfg: KleosConfig, expert: int, seed: int = 0):
    """(W1[i][h], W2[h][i]) of one global expert."""
    w1 = _normal(seed, _STREAM_W1, expert, cfg.I * cfg.H).reshape(cfg.I, cfg.H)
    w2 = _normal(seed, _STREAM_W2, expert, cfg.H * cfg.I).reshape(cfg.H, cfg.I)
    return (w1 * np.float32(1.0 / np.sqrt(cfg.H)), w2 * np.float32(1.0 / np.sqrt(cfg.I)))


def expert_biases(cfg: KleosConfig, expert: int, scale: float, seed: int = 0):
    """(b1[i], b2[h]) of one global expert, N(0, scale).  The benchmark layers use zero biases;
    the parity tests also run with scale > 0 so the bias path of both GEMM epilogues is checked."""
    b1 = _normal(seed, _STREAM_B1, expert, cfg.I) * np.float32(scale)
    b2 = _normal(seed, _STREAM_B2, expert, cfg.H) * np.float32(scale)
    return b1, b2


def zipf_gate_bias(cfg: KleosConfig, s: float = 1.2, seed: int = 0) -> np.ndarray:
    """Per-expert logit bias that makes expert popularity follow Zipf(s) over a seeded
    random permutation of the experts: b_e = log(pmf(rank_pi(e)))."""
    gen = np.random.Generator(np.random.Philox(key=[(seed << 8) | _STREAM_PERM, 0]))
    perm = gen.permutation(cfg.E)
    ranks = np.empty(cfg.E, dtype=np.int64)
    ranks[perm] = np.arange(1, cfg.E + 1)
    pmf = ranks.astype(np.float64) ** (-s)
    pmf /= pmf.sum()
    return np.log(pmf).astype(np.float32)


def packed_input(cfg: KleosConfig, rank: int, world: int, seed: int = 0,
                 bias_scale: float = 0.0) -> np.ndarray:
    """fp32 packed input of one rank, already rounded to the layer's element type
    (layout: moe.cuh:92-98).  Rows E..PX-1 of the gate weight are zero.  A single-expert
    (dense) layer has no gate weight section (moe/fffn.cuh:47-53)."""
    off = cfg.input_offsets(world)
    buf = np.zeros(off["end"], dtype=np.float32)
    buf[off["A"]:off["Wg"]] = activations(cfg, rank, seed).ravel()
    if not cfg.dense:
        buf[off["Wg"]:off["Wg"] + cfg.E * cfg.H] = gate_weight(cfg, seed).ravel()
    nlx = cfg.local_experts(world)
    ih = cfg.I * cfg.H
    for le in range(nlx):
        e = 0 if cfg.dense else rank * nlx + le
        w1, w2 = expert_weights(cfg, e, seed)
        buf[off["W1"] + le * ih: off["W1"] + (le + 1) * ih] = w1.ravel()
        buf[off["W2"] + le * ih: off["W2"] + (le + 1) * ih] = w2.ravel()
        if bias_scale:
            b1, b2 = expert_biases(cfg, e, bias_scale, seed)
            buf[off["b1"] + le * cfg.I: off["b1"] + (le + 1) * cfg.I] = b1
            buf[off["b2"] + le * cfg.H: off["b2"] + (le + 1) * cfg.H] = b2
    return round_to_dtype(buf, cfg.torch_dtype)


def encode(buf_f32: np.ndarray, torch_dtype: int) -> np.ndarray:
    """fp32 values -> the byte image the device expects (fp32 words, or bf16 / fp16 halves)."""
    if torch_dtype in (0, 1):
        return np.ascontiguousarray(buf_f32, dtype=np.float32)
    if torch_dtype == 2:
        return to_bf16_bits(buf_f32)
    if torch_dtype == 3:
        return np.asarray(buf_f32, dtype=np.float32).astype(np.float16).view(np.uint16)
    raise NotImplementedError(f"torch_dtype {torch_dtype}")


def decode(raw: np.ndarray, torch_dtype: int) -> np.ndarray:
    if torch_dtype in (0, 1):
        return np.asarray(raw, dtype=np.float32)
    if torch_dtype == 2:
        return from_bf16_bits(np.asarray(raw, dtype=np.uint16))
    if torch_dtype == 3:
        return np.asarray(raw, dtype=np.uint16).view(np.float16).astype(np.float32)
    raise NotImplementedError(f"torch_dtype {torch_dtype}")


def split_packed(cfg: KleosConfig, buf: np.ndarray, world: int) -> dict:
    """Views of the sections of a packed input buffer."""
    off = cfg.input_offsets(world)
    nlx = cfg.local_experts(world)
    return dict(
        A=buf[off["A"]:off["Wg"]].reshape(cfg.S, cfg.H),
        Wg=buf[off["Wg"]:off["W1"]].reshape(-1, cfg.H),
        W1=buf[off["W1"]:off["W2"]].reshape(nlx, cfg.I, cfg.H),
        W2=buf[off["W2"]:off["b1"]].reshape(nlx, cfg.H, cfg.I),
        b1=buf[off["b1"]:off["b2"]].reshape(nlx, cfg.I),
        b2=buf[off["b2"]:off["end"]].reshape(nlx, cfg.H),
    )
