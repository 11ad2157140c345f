"""kleos_route_static: the router entry point that allocates nothing.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test.  Who needs it: callers that cannot allocate device memory at the moment they
route -- code inside another runtime's allocator callback, or a serving loop whose memory
budget is frozen.  The entry point keeps its scratch in a fixed array inside the library, so
the tests below deliberately call it WITHOUT kleos_initialize and twice in a row: the second
call must find the shared array in a usable state (the part that must start at zero is cleared
by every call).  Its output is compared with the regular entry point's (kleos_forward) on the
same inputs and with the CPU oracle's routing, with the tolerances the other routing tests use.
"""
import numpy as np
import pytest

from aristos_b200 import kleos, synth
from aristos_b200.config import KleosConfig
from oracle import moe_oracle
from tests import moe_harness as hz

pytestmark = pytest.mark.gpu


def _call_static(cfg, raw, dtype, bias=None):
    """One call of kleos_route_static on the A and Wg sections of a packed input image;
    returns (topk [S,K], mcw [S], probs [S,PX]) as host arrays."""
    import torch
    off = cfg.input_offsets(1)
    tdt = torch.float32 if dtype == 0 else torch.uint16
    dev = torch.device("cuda", 0)
    A = torch.from_numpy(raw[off["A"]:off["Wg"]].copy()).view(tdt).to(dev)
    Wg = torch.from_numpy(raw[off["Wg"]:off["W1"]].copy()).view(tdt).to(dev)
    bias_d = None if bias is None else torch.from_numpy(np.asarray(bias, dtype=np.float32)).to(dev)
    probs = torch.full((cfg.S * cfg.PX,), 7, dtype=tdt, device=dev)
    topk = torch.full((cfg.S * cfg.K,), -5, dtype=torch.int32, device=dev)
    mcw = torch.full((cfg.S,), -1.0, dtype=torch.float32, device=dev)
    kleos.route_static(A, Wg, bias_d, cfg.S, cfg.H, cfg.E, cfg.K, dtype, probs, topk, mcw)
    torch.cuda.synchronize()
    return (topk.cpu().numpy().reshape(cfg.S, cfg.K), mcw.cpu().numpy(),
            synth.decode(probs.cpu().numpy(), dtype).reshape(cfg.S, cfg.PX))


def _check_routing(cfg, dtype, got, ref_topk, ref_mcw, ref_probs, what):
    topk, mcw, probs = got
    assert np.array_equal(np.sort(topk, axis=1), np.sort(ref_topk, axis=1)), what
    assert np.abs(mcw - ref_mcw).max() <= 1e-5, what
    assert np.abs(probs - ref_probs).max() <= hz.PROB_TOL[dtype], what
    assert np.all(probs[:, cfg.E:] == 0), what


@pytest.mark.parametrize("dtype", [0, 2])
def test_static_router_matches_regular_entry_point_twice(dtype):
    cfg = KleosConfig(sequence_len=256, hidden_size=512, intermediate_size=1024, num_experts=8,
                      torch_dtype=dtype)
    packed, views = hz.make_inputs(cfg, 1)
    # regular entry point: initialise, forward, read routing, finalise
    probs_ref, _, routing_ref = hz.run_layer_single_gpu(cfg, packed[0])
    oracle = moe_oracle.route(cfg, views[0]["A"], views[0]["Wg"])
    raw = synth.encode(packed[0], dtype)
    for call in range(2):
        got = _call_static(cfg, raw, dtype)
        _check_routing(cfg, dtype, got, routing_ref["topk"], routing_ref["mcw"], probs_ref,
                       f"call {call} vs kleos_forward")
        _check_routing(cfg, dtype, got, oracle["topk"], oracle["mcw"], oracle["probs"],
                       f"call {call} vs oracle")


@pytest.mark.parametrize("dtype", [0, 2])
def test_static_router_with_a_gate_bias(dtype):
    """Caller-supplied logit bias (a device array of E floats) instead of the zero bias the
    entry point keeps in its scratch array."""
    cfg = KleosConfig(sequence_len=512, hidden_size=256, intermediate_size=256, num_experts=32,
                      torch_dtype=dtype)
    bias = synth.zipf_gate_bias(cfg, 1.2) * 2.0
    packed, views = hz.make_inputs(cfg, 1)
    oracle = moe_oracle.route(cfg, views[0]["A"], views[0]["Wg"], gate_bias=bias)
    assert oracle["margin"] > 1e-9
    raw = synth.encode(packed[0], dtype)
    for call in range(2):
        got = _call_static(cfg, raw, dtype, bias=bias)
        _check_routing(cfg, dtype, got, oracle["topk"], oracle["mcw"], oracle["probs"], f"call {call}")


def test_static_router_at_the_limits_of_its_scratch_array():
    """S = 4096 tokens, E = 64 experts, top-8, H = 2048: the largest problem the fixed array is
    sized for (every token may land on the near-tie list, whose fp64 logits then fill it)."""
    dtype = 2
    cfg = KleosConfig(sequence_len=4096, hidden_size=2048, intermediate_size=64, num_experts=64,
                      expert_top_k=8, torch_dtype=dtype)
    packed, views = hz.make_inputs(cfg, 1)
    oracle = moe_oracle.route(cfg, views[0]["A"], views[0]["Wg"])
    assert oracle["margin"] > 1e-9
    raw = synth.encode(packed[0], dtype)
    for call in range(2):
        got = _call_static(cfg, raw, dtype)
        _check_routing(cfg, dtype, got, oracle["topk"], oracle["mcw"], oracle["probs"], f"call {call}")


def test_static_router_refuses_sizes_beyond_its_fixed_scratch():
    lib = kleos.load_library()
    one = 16  # non-null, aligned dummy pointers: the size check comes before any device work
    too_many_tokens = lib.kleos_route_static(one, one, None, 8192, 512, 8, 2, 2, one, one, one, None)
    too_many_experts = lib.kleos_route_static(one, one, None, 256, 512, 128, 2, 2, one, one, one, None)
    assert too_many_tokens == -8 and too_many_experts == -8
    # rows of A and Wg are read sixteen bytes at a time: a misaligned base is refused on the host
    assert lib.kleos_route_static(one + 2, one, None, 256, 512, 8, 2, 2, one, one, one, None) == -8
    assert lib.kleos_route_static(one, one + 8, None, 256, 512, 8, 2, 2, one, one, one, None) == -8
