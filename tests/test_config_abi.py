"""Host logic that needs no GPU: config derivation (Python mirror vs the C++ host layer), the
exported C ABI, and loud failure when no device / no library is present."""
import ctypes
import json
import os
import re

import pytest

from aristos_b200 import kleos
from aristos_b200.config import KleosConfig, baseline_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name,world", [("C1", 1), ("C2", 1), ("C3", 1), ("C3", 8), ("C4", 8),
                                        ("C5", 2), ("C5", 8)])
def test_cpp_and_python_derive_the_same_sizes(tmp_path, name, world):
    cfg, _ = baseline_config(name)
    p = tmp_path / "kleos_config.json"
    cfg.to_json(str(p))
    info = kleos.config_probe(str(p), world)
    assert (info.S, info.H, info.I, info.E, info.K) == (cfg.S, cfg.H, cfg.I, cfg.E, cfg.K)
    assert (info.EC, info.pEC, info.PX) == (cfg.EC, cfg.pEC, cfg.PX)
    assert info.local_experts == cfg.local_experts(world)
    assert info.input_elems == cfg.input_elems(world)
    assert info.output_elems == cfg.output_elems()
    assert info.elem_bytes == cfg.elem_bytes


@pytest.mark.parametrize("world", [1, 4])
def test_single_expert_layer_is_dense(tmp_path, world):
    """E == 1 is the plain FFN: no gate weight in the packed input, no probabilities in the
    packed output, one local expert on every rank (reference moe/fffn.cuh:47-53)."""
    cfg = KleosConfig(sequence_len=256, hidden_size=128, intermediate_size=192, num_experts=1,
                      expert_top_k=1, torch_dtype=2)
    cfg.validate(world)
    p = tmp_path / "kleos_config.json"
    cfg.to_json(str(p))
    info = kleos.config_probe(str(p), world)
    assert info.local_experts == 1 == cfg.local_experts(world)
    assert info.input_elems == cfg.input_elems(world) == 256 * 128 + 2 * 192 * 128 + 192 + 128
    assert info.output_elems == cfg.output_elems() == 256 * 128


def test_benchmark_layer_table_values():
    """EC / pEC / PX of the five benchmark layers."""
    expect = {"C1": (64, 128, 64), "C2": (512, 512, 64), "C3": (256, 256, 64),
              "C4": (320, 384, 128), "C5": (1024, 1024, 64)}
    for name, (ec, pec, px) in expect.items():
        cfg, _ = baseline_config(name)
        assert (cfg.EC, cfg.pEC, cfg.PX) == (ec, pec, px)


def test_reference_shipped_config_is_accepted(tmp_path):
    """The key set of the reference's own csrc/kleos_config.json."""
    shipped = {"capacity_factor": 1, "drop_tokens": 1, "expert_top_k": 2, "global_batch": 256,
               "is_training": 0, "hidden_act": 0, "hidden_size": 2048, "intermediate_size": 2048,
               "mini_batch": 1, "moe_frequency": 1, "num_experts": 64, "num_layers": 1,
               "sequence_len": 8192, "torch_dtype": 1, "vocab_size": 32000}
    p = tmp_path / "kleos_config.json"
    p.write_text(json.dumps(shipped, indent=2))
    info = kleos.config_probe(str(p), 8)
    assert (info.S, info.EC, info.local_experts, info.elem_bytes) == (8192, 256, 8, 4)
    assert KleosConfig.from_json(str(p)).S == 8192


@pytest.mark.parametrize("bad", [
    {"hidden_size": 100}, {"sequence_len": 100}, {"torch_dtype": 7}, {"expert_top_k": 0},
    {"capacity_factor": 0.5}, {"hidden_act": 3},
])
def test_invalid_configs_are_rejected(tmp_path, bad):
    cfg, _ = baseline_config("C1")
    d = {k: getattr(cfg, k) for k in cfg.__dataclass_fields__}
    d.update(bad)
    p = tmp_path / "bad.json"
    p.write_text(json.dumps(d))
    with pytest.raises(kleos.KleosError) as e:
        kleos.config_probe(str(p), 1)
    assert e.value.code == -1
    with pytest.raises(ValueError):
        KleosConfig(**d).validate()


def test_missing_key_and_uneven_sharding(tmp_path):
    cfg, _ = baseline_config("C1")
    d = {k: getattr(cfg, k) for k in cfg.__dataclass_fields__}
    del d["num_layers"]
    p = tmp_path / "m.json"
    p.write_text(json.dumps(d))
    with pytest.raises(kleos.KleosError):
        kleos.config_probe(str(p), 1)
    d["num_layers"] = 1
    p.write_text(json.dumps(d))
    with pytest.raises(kleos.KleosError):
        kleos.config_probe(str(p), 3)  # 8 experts over 3 ranks


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "kleos_b200.h")).read()
    declared = set(re.findall(r"^(?:int|long long|const char\*)\s+(kleos_\w+)\s*\(", header, flags=re.M))
    assert declared, "no declarations parsed from the header"
    lib = kleos.load_library()
    for name in declared:
        assert isinstance(getattr(lib, name), ctypes._CFuncPtr), name
    assert declared == set(kleos.EXPORTS)


def test_call_order_errors_without_initialise():
    lib = kleos.load_library()
    assert lib.kleos_get_rank() == -2
    assert lib.kleos_forward(None, None, None) == -2
    with pytest.raises(kleos.KleosError):
        kleos.finalize()
    # the tuning accessors of the persistent kernel: argument errors first, then the call order
    nb, per = ctypes.c_int(-1), ctypes.c_int(-1)
    lib.kleos_debug_flow_stamps.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                            ctypes.POINTER(ctypes.c_int)]
    assert lib.kleos_debug_flow_stamps(None, 0, None, None) == -8
    assert lib.kleos_debug_flow_stamps(None, 0, ctypes.byref(nb), ctypes.byref(per)) == -2
    buf = (ctypes.c_float * 32)()
    lib.kleos_flow_timeline.argtypes = [ctypes.POINTER(ctypes.c_float), ctypes.c_int]
    assert lib.kleos_flow_timeline(buf, 11) == -8  # fewer than twelve floats
    assert lib.kleos_flow_timeline(buf, 32) == -2


def test_no_gpu_means_loud_failure():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    cfg, _ = baseline_config("C1")
    with pytest.raises(kleos.KleosError) as e:
        kleos.initialize(cfg)
    assert e.value.code == -3  # no CPU fallback


def test_tile_order_of_the_persistent_kernel():
    """Host-side check of the on-GPU scheduler's segment order: for every number of local experts
    and every lag, each (GEMM, expert) segment appears exactly once, a second-GEMM segment comes
    after the first-GEMM segment it consumes, and exactly `lag` first-GEMM segments (fewer at the
    end) separate the two."""
    import ctypes
    lib = kleos.load_library()
    for n in (1, 2, 3, 8, 31, 64, 128):
        for lag in sorted({1, 2, min(8, n), n}):
            if lag > n:
                continue
            phase = (ctypes.c_int32 * (2 * n))()
            expert = (ctypes.c_int32 * (2 * n))()
            assert lib.kleos_debug_tile_order(n, lag, phase, expert) == 2 * n
            seen = {}
            for s in range(2 * n):
                key = (phase[s], expert[s])
                assert key not in seen and 0 <= expert[s] < n and phase[s] in (0, 1), (n, lag, s, key)
                seen[key] = s
            for e in range(n):
                first, second = seen[(0, e)], seen[(1, e)]
                assert second > first
                between = sum(1 for s in range(first + 1, second) if phase[s] == 0)
                assert between == min(lag, n - 1 - e), (n, lag, e, between)
    phase = (ctypes.c_int32 * 4)()
    assert lib.kleos_debug_tile_order(2, 3, phase, phase) == -8   # lag beyond the experts
