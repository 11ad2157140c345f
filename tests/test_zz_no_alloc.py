"""kleos_route_static: the router entry point that allocates nothing.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test.  Who needs it: callers that cannot allocate device memory at the moment they
route -- code inside another runtime's allocator callback, or a serving loop whose memory
budget is frozen.  The entry point keeps its scratch in a fixed array inside the library, so
the test below deliberately calls it WITHOUT kleos_initialize and twice in a row: the second
call must find the shared array in a usable state (the part that must start at zero is cleared
by every call).  Its output is compared with the regular entry point's (kleos_forward) on the
same inputs, with the tolerances the other routing tests use.
"""
import numpy as np
import pytest

from aristos_b200 import kleos, synth
from aristos_b200.config import KleosConfig
from tests import moe_harness as hz

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [0, 2])
def test_static_router_matches_regular_entry_point_twice(dtype):
    import torch
    cfg = KleosConfig(sequence_len=256, hidden_size=512, intermediate_size=1024, num_experts=8,
                      torch_dtype=dtype)
    packed, _ = hz.make_inputs(cfg, 1)
    # regular entry point: initialise, forward, read routing, finalise
    probs_ref, _, routing_ref = hz.run_layer_single_gpu(cfg, packed[0])

    raw = synth.encode(packed[0], dtype)
    off = cfg.input_offsets(1)
    tdt = torch.float32 if dtype == 0 else torch.uint16
    dev = torch.device("cuda", 0)
    A = torch.from_numpy(raw[off["A"]:off["Wg"]].copy()).view(tdt).to(dev)
    Wg = torch.from_numpy(raw[off["Wg"]:off["W1"]].copy()).view(tdt).to(dev)
    for call in range(2):
        probs = torch.full((cfg.S * cfg.PX,), 7, dtype=tdt, device=dev)
        topk = torch.full((cfg.S * cfg.K,), -5, dtype=torch.int32, device=dev)
        mcw = torch.full((cfg.S,), -1.0, dtype=torch.float32, device=dev)
        kleos.route_static(A, Wg, None, cfg.S, cfg.H, cfg.E, cfg.K, dtype, probs, topk, mcw)
        torch.cuda.synchronize()
        got_topk = topk.cpu().numpy().reshape(cfg.S, cfg.K)
        got_probs = synth.decode(probs.cpu().numpy(), dtype).reshape(cfg.S, cfg.PX)
        assert np.array_equal(np.sort(got_topk, axis=1), np.sort(routing_ref["topk"], axis=1)), call
        assert np.abs(mcw.cpu().numpy() - routing_ref["mcw"]).max() <= 1e-5, call
        assert np.abs(got_probs - probs_ref).max() <= hz.PROB_TOL[dtype], call
        assert np.all(got_probs[:, cfg.E:] == 0)


def test_static_router_refuses_sizes_beyond_its_fixed_scratch():
    lib = kleos.load_library()
    one = 1  # non-null dummy pointers: the size check comes before any device work
    too_many_tokens = lib.kleos_route_static(one, one, None, 8192, 512, 8, 2, 2, one, one, one, None)
    too_many_experts = lib.kleos_route_static(one, one, None, 256, 512, 128, 2, 2, one, one, one, None)
    assert too_many_tokens == -8 and too_many_experts == -8
