"""Shared helpers for the parity tests: run the CUDA layer through the C ABI on seeded inputs
and compare with the CPU oracle.  The oracle is used here as the checker only."""
from __future__ import annotations

import numpy as np

from aristos_b200 import kleos, synth
from aristos_b200.config import KleosConfig

# max_abs(y - y_ref) / max_abs(y_ref): fp32, tf32, bf16, fp16 (fp32 accumulation; tf32 and fp16
# both keep a 10-bit mantissa)
TOL = {0: 1e-5, 1: 4e-3, 2: 2e-2, 3: 4e-3}
PROB_TOL = {0: 2e-6, 1: 5e-4, 2: 4e-3, 3: 5e-4}  # absolute, gate probabilities (one element ulp at p ~ 0.5)


def make_inputs(cfg: KleosConfig, world: int, seed: int = 0, bias_scale: float = 0.0):
    packed = [synth.packed_input(cfg, r, world, seed, bias_scale) for r in range(world)]
    views = [synth.split_packed(cfg, p, world) for p in packed]
    return packed, views


def run_layer_single_gpu(cfg: KleosConfig, packed: np.ndarray, gate_bias=None, forwards: int = 1,
                         via_host: bool = False):
    """One-rank layer on cuda:0 through the C ABI.  Returns (probs, out, routing dict)."""
    import torch
    raw = synth.encode(packed, cfg.torch_dtype)
    info = kleos.initialize(cfg, 0, 1)
    try:
        eb = info.elem_bytes
        assert raw.size == info.input_elems
        iP = torch.from_numpy(raw.view(np.uint8).copy()).cuda()
        oP = torch.zeros(info.output_elems * eb, dtype=torch.uint8, device="cuda")
        if gate_bias is not None:
            kleos.set_gate_bias(gate_bias)
        # all forwards but the last run on OTHER tokens, so that state left behind by an earlier
        # forward (cells, result rows, counts, flags) cannot reproduce the expected answer
        n_act = cfg.S * cfg.H
        act = np.ascontiguousarray(raw[:n_act])
        others = [synth.encode(synth.round_to_dtype(synth.activations(cfg, 0, 4242 + i).ravel(),
                                                    cfg.torch_dtype), cfg.torch_dtype)
                  for i in range(forwards - 1)]
        if via_host:
            host_out = np.zeros(n_act, dtype=raw.dtype)
            for a in others + [act]:
                kleos.forward_from_host(np.ascontiguousarray(a), iP, oP, host_out)
        else:
            for a in others + [act]:
                iP[: n_act * eb].copy_(torch.from_numpy(a.view(np.uint8).copy()))
                kleos.forward_host(iP, oP)
        st = kleos.last_status()
        assert st.code == 0, f"device status code={st.code} where={st.where} detail={st.detail}"
        o = oP.cpu().numpy().view(raw.dtype)
        if cfg.dense:  # no gate: the packed output is the S x H result alone
            routing, probs = None, None
            out = synth.decode(o, cfg.torch_dtype).reshape(cfg.S, cfg.H)
        else:
            routing = kleos.debug_routing(info)
            probs = synth.decode(o[: cfg.S * cfg.PX], cfg.torch_dtype).reshape(cfg.S, cfg.PX)
            out = synth.decode(o[cfg.S * cfg.PX:], cfg.torch_dtype).reshape(cfg.S, cfg.H)
        if via_host:
            out_h = synth.decode(host_out, cfg.torch_dtype).reshape(cfg.S, cfg.H)
            assert np.array_equal(out_h, out)
    finally:
        kleos.finalize()
    return probs, out, routing


def check_against_oracle(cfg: KleosConfig, ref: dict, probs, out, routing, rows=None):
    """Bit-exact routing, outputs within the dtype's tolerance."""
    assert ref["margin"] > 1e-9, f"oracle routing margin too small to be meaningful: {ref['margin']}"
    got_sets = np.sort(routing["topk"], axis=1)
    ref_sets = np.sort(ref["topk"], axis=1)
    assert np.array_equal(got_sets, ref_sets), "top-k expert sets differ"
    assert np.array_equal(routing["counts"], ref["counts"]), "per-expert token counts differ"
    # slots compared per (token, expert), independent of the order inside the top-k list
    def slot_map(topk, slots):
        m = np.full((cfg.S, cfg.E), -2, dtype=np.int64)
        np.put_along_axis(m, topk.astype(np.int64), slots.astype(np.int64), axis=1)
        return m
    assert np.array_equal(slot_map(routing["topk"], routing["slots"]),
                          slot_map(ref["topk"], ref["slots"])), "slot assignment differs"
    assert np.abs(routing["mcw"] - ref["mcw"]).max() <= 1e-5
    assert np.abs(probs - ref["probs"]).max() <= PROB_TOL[cfg.torch_dtype]
    assert np.all(probs[:, cfg.E:] == 0)
    ref_out = ref["out"]
    got = out if rows is None else out[rows]
    denom = np.abs(ref_out).max()
    err = np.abs(got - ref_out).max() / denom
    assert err <= TOL[cfg.torch_dtype], f"layer output error {err} > {TOL[cfg.torch_dtype]}"
    # tokens with every choice dropped produce a zero row
    dropped_all = (ref["slots"] < 0).all(axis=1)
    if rows is not None:
        dropped_all = dropped_all[rows]
    assert np.all(got[dropped_all] == 0)
    return err
