"""ctypes loader for the C oracle (``moe_oracle.c``).  Test infrastructure only."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class OracleCfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("S", "H", "I", "E", "K", "EC", "PX", "dtype", "hidden_act", "world")]


def build(force: bool = False) -> str:
    so = os.path.join(_HERE, "libmoe_oracle.so")
    src = os.path.join(_HERE, "moe_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "libmoe_oracle.so"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.oracle_num_threads.restype = ctypes.c_int
    return _LIB


def _cfg(cfg, world):
    return OracleCfg(cfg.S, cfg.H, cfg.I, cfg.E, cfg.K, cfg.EC, cfg.PX, cfg.torch_dtype,
                     cfg.hidden_act, world)


def _fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def num_threads() -> int:
    return lib().oracle_num_threads()


def use_all_cores() -> int:
    """Let the oracle use every core this process may run on (launchers such as torchrun export
    OMP_NUM_THREADS=1); returns the thread count now in effect."""
    import os
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().oracle_set_threads(n)
    return num_threads()


def gate_stats(cfg, inp, counts, gate_bias=None):
    """Training-mode gate statistics of one rank; twin of the keys mean_prob / mean_count /
    gate_loss that moe_oracle.route returns."""
    L = lib()
    c = _cfg(cfg, 1)
    A = np.ascontiguousarray(inp["A"], dtype=np.float32)
    Wg = np.ascontiguousarray(inp["Wg"], dtype=np.float32)
    bias = None if gate_bias is None else np.ascontiguousarray(gate_bias, dtype=np.float32)
    cnt = np.ascontiguousarray(counts, dtype=np.uint32)
    mp = np.zeros(cfg.E, dtype=np.float64)
    mc = np.zeros(cfg.E, dtype=np.float64)
    loss = ctypes.c_double(0)
    dp = ctypes.POINTER(ctypes.c_double)
    rc = L.oracle_gate_stats(ctypes.byref(c), _fp(A), _fp(Wg), None if bias is None else _fp(bias),
                             cnt.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)),
                             mp.ctypes.data_as(dp), mc.ctypes.data_as(dp), ctypes.byref(loss))
    if rc:
        raise RuntimeError(f"oracle_gate_stats failed: {rc}")
    return dict(mean_prob=mp, mean_count=mc, gate_loss=loss.value)


def dense_ffn(cfg, inp, tokens=None, accum64=True):
    """Single-expert layer (plain FFN) for one rank's tokens; twin of moe_oracle.dense_ffn."""
    L = lib()
    c = _cfg(cfg, 1)
    a = inp["A"] if tokens is None else inp["A"][np.asarray(tokens)]
    a = np.ascontiguousarray(a, dtype=np.float32)
    arrs = [np.ascontiguousarray(inp[k][0], dtype=np.float32) for k in ("W1", "W2", "b1", "b2")]
    out = np.zeros((a.shape[0], cfg.H), dtype=np.float32)
    rc = L.oracle_expert_ffn(ctypes.byref(c), ctypes.c_int(a.shape[0]), _fp(a), *[_fp(x) for x in arrs],
                             _fp(out), ctypes.c_int(1 if accum64 else 0))
    if rc:
        raise RuntimeError(f"oracle_expert_ffn failed: {rc}")
    return out


def moe_forward_rank(cfg, world, rank, inputs, gate_bias=None, tokens=None, accum64=True):
    """Layer output for the tokens of one source rank; same result keys as the NumPy twin."""
    L = lib()
    c = _cfg(cfg, world)
    nlx = cfg.E // world
    me = inputs[rank]
    A = np.ascontiguousarray(me["A"], dtype=np.float32)
    Wg = np.ascontiguousarray(me["Wg"], dtype=np.float32)
    keep = []

    def ptrs(key):
        arr = (ctypes.POINTER(ctypes.c_float) * cfg.E)()
        for e in range(cfg.E):
            owner, le = divmod(e, nlx)
            a = np.ascontiguousarray(inputs[owner][key][le], dtype=np.float32)
            keep.append(a)
            arr[e] = _fp(a)
        return arr

    W1, W2, b1, b2 = ptrs("W1"), ptrs("W2"), ptrs("b1"), ptrs("b2")
    bias = None if gate_bias is None else np.ascontiguousarray(gate_bias, dtype=np.float32)
    tok = None if tokens is None else np.ascontiguousarray(tokens, dtype=np.int32)
    nt = cfg.S if tok is None else len(tok)
    probs = np.zeros((cfg.S, cfg.PX), dtype=np.float32)
    topk = np.zeros((cfg.S, cfg.K), dtype=np.int32)
    mcw = np.zeros(cfg.S, dtype=np.float32)
    slots = np.zeros((cfg.S, cfg.K), dtype=np.int32)
    counts = np.zeros(cfg.E, dtype=np.uint32)
    margin = ctypes.c_double(0)
    out = np.zeros((nt, cfg.H), dtype=np.float32)
    rc = L.oracle_moe_forward_rank(
        ctypes.byref(c), _fp(A), _fp(Wg), W1, W2, b1, b2,
        None if bias is None else _fp(bias),
        None if tok is None else tok.ctypes.data_as(ctypes.POINTER(ctypes.c_int)),
        ctypes.c_int(nt), ctypes.c_int(1 if accum64 else 0), _fp(probs),
        topk.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), _fp(mcw),
        slots.ctypes.data_as(ctypes.POINTER(ctypes.c_int)),
        counts.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), ctypes.byref(margin), _fp(out))
    if rc:
        raise RuntimeError(f"oracle_moe_forward_rank failed: {rc}")
    return dict(probs=probs, topk=topk, mcw=mcw, slots=slots, counts=counts,
                routed=np.minimum(counts, cfg.EC).astype(np.uint32), margin=margin.value,
                out=out)


def route_rank(cfg, A, Wg, gate_bias=None):
    """Routing of one source rank alone (probs, topk, mcw, slots, counts, margin)."""
    L = lib()
    c = _cfg(cfg, 1)
    A = np.ascontiguousarray(A, dtype=np.float32)
    Wg = np.ascontiguousarray(Wg, dtype=np.float32)
    bias = None if gate_bias is None else np.ascontiguousarray(gate_bias, dtype=np.float32)
    probs = np.zeros((cfg.S, cfg.PX), dtype=np.float32)
    topk = np.zeros((cfg.S, cfg.K), dtype=np.int32)
    mcw = np.zeros(cfg.S, dtype=np.float32)
    slots = np.zeros((cfg.S, cfg.K), dtype=np.int32)
    counts = np.zeros(cfg.E, dtype=np.uint32)
    margin = ctypes.c_double(0)
    rc = L.oracle_route(ctypes.byref(c), _fp(A), _fp(Wg), None if bias is None else _fp(bias),
                        _fp(probs), topk.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), _fp(mcw),
                        slots.ctypes.data_as(ctypes.POINTER(ctypes.c_int)),
                        counts.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), ctypes.byref(margin))
    if rc:
        raise RuntimeError(f"oracle_route failed: {rc}")
    return dict(probs=probs, topk=topk, mcw=mcw, slots=slots, counts=counts,
                routed=np.minimum(counts, cfg.EC).astype(np.uint32), margin=margin.value)


def moe_forward_rank_lazy(cfg, A, Wg, get_expert, gate_bias=None, tokens=None, accum64=True):
    """moe_forward_rank for callers that do not hold every expert's weights: routing first, then
    ``get_expert(e) -> (W1 [I,H], W2 [H,I], b1 [I], b2 [H])`` is asked only for the experts that
    the listed tokens were routed to (and kept by)."""
    L = lib()
    c = _cfg(cfg, 1)
    rt = route_rank(cfg, A, Wg, gate_bias)
    tok = np.arange(cfg.S, dtype=np.int32) if tokens is None else np.ascontiguousarray(tokens, dtype=np.int32)
    used = rt["topk"][tok][rt["slots"][tok] != -1]
    keep = []
    arrs = [(ctypes.POINTER(ctypes.c_float) * cfg.E)() for _ in range(4)]
    for e in sorted(set(int(x) for x in used)):
        parts = [np.ascontiguousarray(x, dtype=np.float32) for x in get_expert(e)]
        keep.append(parts)
        for arr, part in zip(arrs, parts):
            arr[e] = _fp(part)
    A = np.ascontiguousarray(A, dtype=np.float32)
    Wg = np.ascontiguousarray(Wg, dtype=np.float32)
    bias = None if gate_bias is None else np.ascontiguousarray(gate_bias, dtype=np.float32)
    out = np.zeros((len(tok), cfg.H), dtype=np.float32)
    margin = ctypes.c_double(0)
    rc = L.oracle_moe_forward_rank(
        ctypes.byref(c), _fp(A), _fp(Wg), *arrs, None if bias is None else _fp(bias),
        tok.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), ctypes.c_int(len(tok)),
        ctypes.c_int(1 if accum64 else 0), _fp(rt["probs"]),
        rt["topk"].ctypes.data_as(ctypes.POINTER(ctypes.c_int)), _fp(rt["mcw"]),
        rt["slots"].ctypes.data_as(ctypes.POINTER(ctypes.c_int)),
        rt["counts"].ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), ctypes.byref(margin), _fp(out))
    if rc:
        raise RuntimeError(f"oracle_moe_forward_rank failed: {rc}")
    rt["out"] = out
    return rt
