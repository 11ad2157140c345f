"""Host-side mirror of the reference's API for the MoE forward path, on top of the C ABI.

Function names and argument meaning follow the reference's host functions:
``initialize`` / ``finalize`` / ``get_rank`` (csrc/include/kleos/bootstrap.cuh:532-588) and
``moe::forwardHost`` / ``forwardHostBench`` (csrc/include/kleos/moe/moe.cuh:146-205).  The
packed device buffers are the reference's (moe.cuh:92-98).  Errors raise ``KleosError``
instead of terminating the process (reference: debug.cuh:19-43).

There is no CPU path: loading fails loudly if ``libkleos_b200.so`` has not been built, and
``initialize`` fails if no sm_100 GPU is present.
"""
from __future__ import annotations

import ctypes
import json
import os
import tempfile
from dataclasses import asdict

from .config import KleosConfig

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkleos_b200.so")

EXPORTS = (
    "kleos_get_unique_id", "kleos_config_probe", "kleos_set_device", "kleos_initialize", "kleos_set_gate_bias",
    "kleos_forward", "kleos_forward_bench", "kleos_forward_host", "kleos_forward_host_async",
    "kleos_host_sync", "kleos_get_rank",
    "kleos_local_experts", "kleos_get_info", "kleos_last_status", "kleos_clear_status", "kleos_debug_routing",
    "kleos_phase_times", "kleos_flow_timeline", "kleos_debug_flow_stamps", "kleos_debug_flow_stalls", "kleos_debug_tile_order", "kleos_launch_count", "kleos_debug_gemm_stats", "kleos_debug_suppress_return_flag", "kleos_gate_stats", "kleos_plan_placement", "kleos_placement_model", "kleos_route_static", "kleos_finalize", "kleos_error_string",
)

PHASE_NAMES = ("route", "slots", "dispatch", "plan", "gemm1", "gemm2", "combine", "total")


class KleosError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: {code}")
        self.code = code


class Status(ctypes.Structure):
    _fields_ = [("code", ctypes.c_int32), ("where", ctypes.c_int32),
                ("detail", ctypes.c_int32), ("epoch", ctypes.c_int32)]


class LayerInfo(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in
                ("rank", "world", "local_experts", "S", "H", "I", "E", "K", "EC", "pEC", "PX",
                 "torch_dtype", "hidden_act", "elem_bytes")] + \
               [("input_elems", ctypes.c_int64), ("output_elems", ctypes.c_int64)]


_lib = None


def load_library() -> ctypes.CDLL:
    """dlopen the in-tree CUDA library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m aristos_b200.build` "
                "(this package has no CPU fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        lib.kleos_error_string.restype = ctypes.c_char_p
        lib.kleos_initialize.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.kleos_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.kleos_forward_bench.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                            ctypes.c_int, ctypes.POINTER(ctypes.c_float)]
        lib.kleos_forward_host.argtypes = [ctypes.c_void_p] * 4
        lib.kleos_forward_host_async.argtypes = [ctypes.c_void_p] * 4
        lib.kleos_set_gate_bias.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.kleos_debug_routing.argtypes = [ctypes.c_void_p] * 4
        lib.kleos_gate_stats.argtypes = [ctypes.c_void_p] * 3
        lib.kleos_phase_times.argtypes = [ctypes.POINTER(ctypes.c_float), ctypes.c_int]
        lib.kleos_get_unique_id.argtypes = [ctypes.c_void_p]
        _lib = lib
    return _lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load_library().kleos_error_string(rc).decode()
        raise KleosError(rc, f"{what}: {msg}")


def get_unique_id() -> bytes:
    """128-byte bootstrap id created on rank 0 and handed to every rank's ``initialize``."""
    buf = ctypes.create_string_buffer(128)
    _check(load_library().kleos_get_unique_id(buf), "kleos_get_unique_id")
    return buf.raw


def set_device(device: int) -> None:
    _check(load_library().kleos_set_device(device), "kleos_set_device")


def initialize(config, rank: int = 0, world: int = 1, unique_id: bytes | None = None) -> LayerInfo:
    """``config`` is a path to a kleos_config.json or a KleosConfig (written to a temp file,
    since the C ABI reads the same JSON file the reference's build reads)."""
    lib = load_library()
    tmp = None
    if isinstance(config, KleosConfig):
        tmp = tempfile.NamedTemporaryFile("w", suffix=".json", delete=False)
        json.dump(asdict(config), tmp)
        tmp.close()
        path = tmp.name
    else:
        path = str(config)
    try:
        idbuf = ctypes.create_string_buffer(unique_id, 128) if unique_id is not None else None
        _check(lib.kleos_initialize(path.encode(), rank, world, idbuf), "kleos_initialize")
    finally:
        if tmp is not None:
            os.unlink(tmp.name)
    return get_info()


def config_probe(path: str, world: int = 1) -> LayerInfo:
    """Sizes the C++ host layer derives from a kleos_config.json; needs no GPU."""
    info = LayerInfo()
    _check(load_library().kleos_config_probe(str(path).encode(), world, ctypes.byref(info)),
           "kleos_config_probe")
    return info


def get_info() -> LayerInfo:
    info = LayerInfo()
    _check(load_library().kleos_get_info(ctypes.byref(info)), "kleos_get_info")
    return info


def get_rank() -> int:
    return load_library().kleos_get_rank()


def local_experts() -> int:
    return load_library().kleos_local_experts()


def set_gate_bias(bias) -> None:
    lib = load_library()
    if bias is None:
        _check(lib.kleos_set_gate_bias(None, 0), "kleos_set_gate_bias")
        return
    import numpy as np
    b = np.ascontiguousarray(bias, dtype=np.float32)
    _check(lib.kleos_set_gate_bias(b.ctypes.data, b.size), "kleos_set_gate_bias")


def forward_host(iP, oP, stream=None) -> None:
    """Asynchronous layer forward on packed DEVICE buffers (torch tensors or raw pointers)."""
    _check(load_library().kleos_forward(_ptr(iP), _ptr(oP), stream), "kleos_forward")


def forward_host_bench(iP, oP, skip: int = 32, trials: int = 32) -> float:
    """Mean milliseconds per forward over ``trials`` launches after ``skip`` warm-ups."""
    ms = ctypes.c_float(0)
    _check(load_library().kleos_forward_bench(_ptr(iP), _ptr(oP), skip, trials, ctypes.byref(ms)),
           "kleos_forward_bench")
    return ms.value


def forward_from_host(host_activations, iP, oP, host_output) -> None:
    """End-to-end step with host buffers: H2D activations, forward, D2H layer output, sync."""
    _check(load_library().kleos_forward_host(_ptr(host_activations), _ptr(iP), _ptr(oP),
                                             _ptr(host_output)), "kleos_forward_host")


def forward_from_host_async(host_activations, iP, oP, host_output) -> None:
    """Queue one end-to-end step (H2D, forward, D2H on three streams); see host_sync()."""
    _check(load_library().kleos_forward_host_async(_ptr(host_activations), _ptr(iP), _ptr(oP),
                                                   _ptr(host_output)), "kleos_forward_host_async")


def host_sync() -> None:
    """Wait for every queued end-to-end step and raise on a device-side error."""
    _check(load_library().kleos_host_sync(), "kleos_host_sync")


def phase_times() -> dict:
    arr = (ctypes.c_float * 8)()
    _check(load_library().kleos_phase_times(arr, 8), "kleos_phase_times")
    return dict(zip(PHASE_NAMES, [float(v) for v in arr]))


def gemm_stats():
    """Per-block stall counters of the last two GEMM launches (needs KLEOS_GEMM_STATS=1)."""
    import numpy as np
    buf = np.zeros(2 * 256 * 12, dtype=np.int64)
    n = load_library().kleos_debug_gemm_stats(buf.ctypes.data_as(ctypes.c_void_p), buf.size)
    if n < 0:
        _check(n, "kleos_debug_gemm_stats")
    return buf[:n].reshape(2, -1, 12)


def route_static(A, Wg, gate_bias, S, H, E, K, torch_dtype, probs, topk, mcw, stream=None) -> None:
    """Router without any device allocation (fixed scratch inside the library): see
    kleos_route_static in include/kleos_b200.h for limits and the no-overlap rule."""
    lib = load_library()
    lib.kleos_route_static.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + \
        [ctypes.c_int] * 5 + [ctypes.c_void_p] * 4
    _check(lib.kleos_route_static(_ptr(A), _ptr(Wg), _ptr(gate_bias), S, H, E, K, torch_dtype,
                                  _ptr(probs), _ptr(topk), _ptr(mcw), stream),
           "kleos_route_static")


FLOW_MILESTONES = ("start", "planned", "first_tile", "last_gemm1_tile", "last_tile", "dispatched",
                   "combined", "end", "routed", "slotted", "gate_logits", "gate_done", "topk_done",
                   "probs_done", "slot_base", "slots_done", "route_begin", "first_operands", "topk_pass1")


def flow_timeline() -> dict:
    """Milestones of the persistent kernel in the most recent forward_host_bench, in milliseconds
    after the kernel's start (see kleos_flow_timeline in include/kleos_b200.h)."""
    buf = (ctypes.c_float * len(FLOW_MILESTONES))()
    lib = load_library()
    lib.kleos_flow_timeline.argtypes = [ctypes.POINTER(ctypes.c_float), ctypes.c_int]
    _check(lib.kleos_flow_timeline(buf, len(FLOW_MILESTONES)), "kleos_flow_timeline")
    return {n: float(buf[i]) for i, n in enumerate(FLOW_MILESTONES)}


def flow_stamps():
    """Milestones of every block of the persistent kernel in the last timed forward of
    forward_host_bench: int64 array [blocks, milestones] of global-timer nanoseconds, 0 where a
    block never passed the milestone (kleos_debug_flow_stamps)."""
    import numpy as np
    lib = load_library()
    lib.kleos_debug_flow_stamps.argtypes = [ctypes.POINTER(ctypes.c_longlong), ctypes.c_int,
                                            ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    nb, per = ctypes.c_int(0), ctypes.c_int(0)
    _check(lib.kleos_debug_flow_stamps(None, 0, ctypes.byref(nb), ctypes.byref(per)), "kleos_debug_flow_stamps")
    out = np.zeros((nb.value, per.value), dtype=np.int64)
    _check(lib.kleos_debug_flow_stamps(out.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong)), out.size,
                                       ctypes.byref(nb), ctypes.byref(per)), "kleos_debug_flow_stamps")
    return out


FLOW_STALLS = ("producer_wait_stage", "producer_wait_data", "producer_total", "mma_wait_accumulator",
               "mma_wait_operands", "mma_wait_task", "mma_total", "readback_wait_accumulator",
               "readback_publish", "readback_store", "readback_total", "producer_proxy_fence")


def flow_stalls() -> dict:
    """Where the tile-stream roles of the persistent kernel waited in the last timed forward
    (kleos_debug_flow_stalls), milliseconds averaged over blocks."""
    buf = (ctypes.c_float * len(FLOW_STALLS))()
    lib = load_library()
    lib.kleos_debug_flow_stalls.argtypes = [ctypes.POINTER(ctypes.c_float), ctypes.c_int]
    _check(lib.kleos_debug_flow_stalls(buf, len(FLOW_STALLS)), "kleos_debug_flow_stalls")
    return {n: float(buf[i]) for i, n in enumerate(FLOW_STALLS) if n != "unused"}


def launch_count() -> int:
    """Kernels the library has launched for forward calls since initialize()."""
    lib = load_library()
    lib.kleos_launch_count.restype = ctypes.c_longlong
    n = lib.kleos_launch_count()
    if n < 0:
        raise KleosError(int(n), "kleos_launch_count")
    return int(n)


def last_status() -> Status:
    st = Status()
    _check(load_library().kleos_last_status(ctypes.byref(st)), "kleos_last_status")
    return st


def debug_routing(info: LayerInfo) -> dict:
    import numpy as np
    topk = np.empty((info.S, info.K), dtype=np.int32)
    slots = np.empty((info.S, info.K), dtype=np.int32)
    counts = np.empty(info.E, dtype=np.uint32)
    mcw = np.empty(info.S, dtype=np.float32)
    _check(load_library().kleos_debug_routing(topk.ctypes.data, slots.ctypes.data,
                                              counts.ctypes.data, mcw.ctypes.data),
           "kleos_debug_routing")
    return dict(topk=topk, slots=slots, counts=counts, mcw=mcw)


class PlacementRequest(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("world", "rank", "num_experts", "expert_cost", "is_training")] + \
               [(n, ctypes.c_uint32) for n in ("moe_stages", "p2p_buffer_mb", "grad_buffer_mb")] + \
               [(n, ctypes.c_void_p) for n in ("alpha", "beta", "rate", "mem")]


class PlacementResult(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("feasible", "group_size", "group_rank", "local_experts",
                                              "expert_slots", "widest_group", "matches_data_path")]


def placement_model(config) -> dict:
    """Cost-model constants of the placement planner for a layer (needs no GPU)."""
    import tempfile
    lib = load_library()
    vals = [ctypes.c_uint32() for _ in range(3)]
    with tempfile.TemporaryDirectory() as d:
        path = config if isinstance(config, str) else os.path.join(d, "kleos_config.json")
        if not isinstance(config, str):
            config.to_json(path)
        _check(lib.kleos_placement_model(path.encode(), *[ctypes.byref(v) for v in vals]),
               "kleos_placement_model")
    return dict(moe_stages=vals[0].value, p2p_buffer=vals[1].value, grad_buffer=vals[2].value)


def plan_placement(alpha, beta, rate, mem, num_experts, model: dict, rank: int = 0,
                   expert_cost: int = 1, training: bool = False) -> dict:
    """Device groups and expert placement from a measured topology (host only)."""
    import numpy as np
    a = np.ascontiguousarray(alpha, dtype=np.float32)
    b = np.ascontiguousarray(beta, dtype=np.float32)
    r = np.ascontiguousarray(rate, dtype=np.float32)
    m = np.ascontiguousarray(mem, dtype=np.uint32)
    world = r.size
    assert a.shape == (world, world) and b.shape == (world, world) and m.size == world
    rq = PlacementRequest(world, rank, num_experts, expert_cost, int(training), model["moe_stages"],
                          model["p2p_buffer"], model["grad_buffer"], a.ctypes.data, b.ctypes.data,
                          r.ctypes.data, m.ctypes.data)
    res = PlacementResult()
    d2g = np.zeros(world, dtype=np.uint32)
    ranks = np.zeros(world, dtype=np.uint32)
    e2m = np.zeros(num_experts, dtype=np.uint32)
    lib = load_library()
    lib.kleos_plan_placement.argtypes = [ctypes.c_void_p] * 5
    _check(lib.kleos_plan_placement(ctypes.byref(rq), ctypes.byref(res), d2g.ctypes.data,
                                    ranks.ctypes.data, e2m.ctypes.data), "kleos_plan_placement")
    out = dict(feasible=bool(res.feasible), device_to_group=d2g.tolist())
    if res.feasible:
        out.update(group_ranks=ranks[:res.group_size].tolist(), group_rank=res.group_rank,
                   expert_to_member=e2m.tolist(), local_experts=res.local_experts,
                   expert_slots=res.expert_slots, widest_group=res.widest_group,
                   matches_data_path=bool(res.matches_data_path))
    return out


def gate_stats(info: LayerInfo) -> dict:
    """Training-mode gate statistics of the last forward: mean probability and mean (unclamped)
    selection count per expert, and the auxiliary loss (needs is_training = 1)."""
    import numpy as np
    mean_prob = np.empty(info.E, dtype=np.float32)
    mean_count = np.empty(info.E, dtype=np.float32)
    loss = np.empty(1, dtype=np.float32)
    _check(load_library().kleos_gate_stats(mean_prob.ctypes.data, mean_count.ctypes.data,
                                           loss.ctypes.data), "kleos_gate_stats")
    return dict(mean_prob=mean_prob, mean_count=mean_count, loss=float(loss[0]))


def finalize() -> None:
    _check(load_library().kleos_finalize(), "kleos_finalize")


def _ptr(x):
    if x is None or isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(type(x))
