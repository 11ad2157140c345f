"""The two CPU oracles against each other and against the committed golden fixtures."""
import numpy as np
import pytest

from aristos_b200 import synth
from aristos_b200.config import KleosConfig
from oracle import c_oracle, moe_oracle
from tests import golden_util


def _agree(cfg, a, b, out_tol):
    assert np.array_equal(a["topk"], b["topk"])
    assert np.array_equal(a["slots"], b["slots"])
    assert np.array_equal(a["counts"], b["counts"])
    assert np.abs(a["mcw"] - b["mcw"]).max() <= 2e-6
    assert np.abs(a["probs"] - b["probs"]).max() <= (2e-6 if cfg.torch_dtype == 0 else 4e-3)
    denom = max(np.abs(b["out"]).max(), 1e-30)
    assert np.abs(a["out"] - b["out"]).max() / denom <= out_tol


@pytest.mark.parametrize("name", golden_util.names())
def test_numpy_oracle_reproduces_golden(name):
    cfg, world, bias, _, views, expect = golden_util.load(name)
    got = moe_oracle.moe_forward(cfg, world, views, gate_bias=bias)
    for r in range(world):
        _agree(cfg, got[r], expect[r], 0.0 if cfg.torch_dtype == 2 else 1e-6)
        if "mean_prob" in expect[r]:  # training-mode gate statistics pinned by the newer fixtures
            assert np.abs(got[r]["mean_prob"] - expect[r]["mean_prob"]).max() <= 1e-7
            assert np.array_equal(got[r]["mean_count"], expect[r]["mean_count"])
            assert abs(got[r]["gate_loss"] - float(expect[r]["gate_loss"])) <= 1e-8


@pytest.mark.parametrize("name", golden_util.names())
def test_c_oracle_matches_golden(name):
    cfg, world, bias, _, views, expect = golden_util.load(name)
    for r in range(world):
        got = c_oracle.moe_forward_rank(cfg, world, r, views, gate_bias=bias)
        # bf16: identical roundings; fp32: softmax summation order differs in the last ulp
        _agree(cfg, got, expect[r], 4e-3 if cfg.torch_dtype in (1, 2, 3) else 1e-6)


@pytest.mark.parametrize("dtype,world", [(0, 1), (2, 1), (2, 2), (0, 4), (3, 1), (3, 2), (1, 1), (1, 2)])
def test_c_and_numpy_agree_on_fresh_inputs(dtype, world):
    cfg = KleosConfig(sequence_len=128, hidden_size=128, intermediate_size=192, num_experts=8,
                      torch_dtype=dtype)
    views = [synth.split_packed(cfg, synth.packed_input(cfg, r, world, seed=3), world)
             for r in range(world)]
    ref = moe_oracle.moe_forward(cfg, world, views)
    for r in range(world):
        got = c_oracle.moe_forward_rank(cfg, world, r, views)
        _agree(cfg, got, ref[r], 4e-3 if dtype in (1, 2, 3) else 1e-6)


def test_token_subset_equals_full_rows():
    cfg = KleosConfig(sequence_len=128, hidden_size=64, intermediate_size=64, num_experts=8,
                      torch_dtype=2)
    views = [synth.split_packed(cfg, synth.packed_input(cfg, 0, 1), 1)]
    full = c_oracle.moe_forward_rank(cfg, 1, 0, views)
    rows = np.array([0, 5, 17, 127], dtype=np.int32)
    part = c_oracle.moe_forward_rank(cfg, 1, 0, views, tokens=rows)
    assert np.array_equal(part["out"], full["out"][rows])
    part_np = moe_oracle.moe_forward(cfg, 1, views, token_subset=rows)[0]
    assert np.abs(part_np["out"] - full["out"][rows]).max() <= 4e-3 * np.abs(full["out"]).max()


def test_ties_go_to_lowest_expert_id():
    """All experts share one gate row, so every logit ties: top-k must be {0, 1}."""
    cfg = KleosConfig(sequence_len=128, hidden_size=64, intermediate_size=64, num_experts=8,
                      torch_dtype=0)
    packed = synth.packed_input(cfg, 0, 1)
    v = synth.split_packed(cfg, packed, 1)
    v["Wg"][: cfg.E] = v["Wg"][0]
    for res in (moe_oracle.moe_forward(cfg, 1, [v])[0], c_oracle.moe_forward_rank(cfg, 1, 0, [v])):
        assert np.array_equal(np.sort(res["topk"], axis=1),
                              np.tile(np.array([0, 1]), (cfg.S, 1)))
        # capacity EC = ceil(S/E)*k = 32: the first 32 tokens keep their slot, the rest drop
        assert res["counts"][0] == cfg.S and res["counts"][1] == cfg.S
        assert (res["slots"][: cfg.EC] >= 0).all() and (res["slots"][cfg.EC:] < 0).all()
        assert np.all(res["out"][cfg.EC:] == 0)


def test_capacity_formula_and_drops():
    cfg = KleosConfig(sequence_len=256, hidden_size=64, intermediate_size=64, num_experts=16,
                      torch_dtype=2, capacity_factor=1.25)
    assert cfg.EC == 40 and cfg.pEC == 128
    views = [synth.split_packed(cfg, synth.packed_input(cfg, 0, 1), 1)]
    bias = synth.zipf_gate_bias(cfg, 1.2) * 3
    res = moe_oracle.moe_forward(cfg, 1, views, gate_bias=bias)[0]
    assert (res["routed"] <= cfg.EC).all() and (res["counts"] >= res["routed"]).all()
    over = res["counts"] > cfg.EC
    assert over.any(), "the skewed gate should overflow at least one expert"
    kept = (res["slots"] >= 0).sum()
    assert kept == res["routed"].sum()
    assert res["slots"].max() < cfg.EC


@pytest.mark.parametrize("dtype", [0, 2, 3])
def test_dense_layer_twins_agree_and_match_the_general_path(dtype):
    """E == 1: the dense FFN of both twins is the same, and it equals what the routed path gives
    for one expert with top-1 (every token kept, plain copy in the combine)."""
    cfg = KleosConfig(sequence_len=128, hidden_size=64, intermediate_size=192, num_experts=1,
                      expert_top_k=1, torch_dtype=dtype, hidden_act=1)
    packed = synth.packed_input(cfg, 0, 1, seed=3, bias_scale=0.5)
    v = synth.split_packed(cfg, packed, 1)
    assert np.abs(v["b1"]).max() > 0 and np.abs(v["b2"]).max() > 0
    a = moe_oracle.dense_ffn(cfg, v)
    b = c_oracle.dense_ffn(cfg, v)
    assert np.abs(a - b).max() <= 1e-6 * np.abs(a).max()
    sub = moe_oracle.dense_ffn(cfg, v, token_subset=[5, 77])
    assert np.array_equal(sub, a[[5, 77]])
    routed = dict(v, Wg=np.zeros((cfg.PX, cfg.H), dtype=np.float32))
    full = moe_oracle.moe_forward(cfg, 1, [routed])[0]
    assert np.array_equal(full["out"], a)


def test_tf32_rounding_is_nearest_even_on_a_ten_bit_mantissa():
    """torch_dtype 1: fp32 words with the low 13 mantissa bits clear (reference element type
    cute::tfloat32_t, types.cuh:128-131); both twins and the input generator round alike."""
    one = np.float32(1.0)
    ulp = np.float32(2.0 ** -10)
    x = np.array([one + ulp * np.float32(0.5),      # tie: stays at the even neighbour 1.0
                  one + ulp * np.float32(1.5),      # tie: goes up to the even neighbour 1 + 2 ulp
                  one + ulp * np.float32(0.5001),   # above the tie: rounds up
                  np.float32(-3.14159274), np.float32(np.inf)], dtype=np.float32)
    want = np.array([1.0, 1.0 + 2 * 2.0 ** -10, 1.0 + 2.0 ** -10, -3.140625, np.inf], dtype=np.float32)
    assert np.array_equal(moe_oracle.round_elem(x, 1), want)
    assert np.array_equal(synth.round_to_dtype(x[:4], 1), want[:4])
    y = x.copy()
    c_oracle.lib().oracle_round(y.ctypes.data_as(__import__("ctypes").POINTER(__import__("ctypes").c_float)),
                                __import__("ctypes").c_size_t(y.size), 1)
    assert np.array_equal(y, want)


@pytest.mark.parametrize("dtype", [0, 2])
def test_gate_statistics_twins_agree(dtype):
    cfg = KleosConfig(sequence_len=256, hidden_size=128, intermediate_size=128, num_experts=16,
                      torch_dtype=dtype, is_training=1)
    v = synth.split_packed(cfg, synth.packed_input(cfg, 0, 1, seed=9), 1)
    bias = synth.zipf_gate_bias(cfg, 1.2)
    a = moe_oracle.route(cfg, v["A"], v["Wg"], bias)
    b = c_oracle.gate_stats(cfg, v, a["counts"], gate_bias=bias)
    assert np.abs(a["mean_prob"] - b["mean_prob"]).max() <= 1e-7
    assert np.array_equal(a["mean_count"], b["mean_count"])
    assert abs(a["gate_loss"] - b["gate_loss"]) <= 1e-9
    assert abs(a["mean_prob"].sum() - 1.0) <= 1e-6 and abs(a["mean_count"].sum() - cfg.K) <= 1e-12


def _views(cfg, seed=0, world=1, bias_scale=0.0):
    return [synth.split_packed(cfg, synth.packed_input(cfg, r, world, seed, bias_scale), world)
            for r in range(world)]


@pytest.mark.parametrize("dtype", [0, 2])
def test_identical_experts_make_the_layer_a_plain_ffn(dtype):
    """If every expert has the same weights, out[t] = FFN(x[t]) * sum_e p~(t,e) / sum_e p(t,e):
    with top-k = E and nothing dropped the factor is 1 up to the rounding of the probabilities,
    so the routed layer must reproduce the dense FFN (a size-independent check of routing,
    capacity and combine together)."""
    cfg = KleosConfig(sequence_len=128, hidden_size=64, intermediate_size=128, num_experts=4,
                      expert_top_k=4, torch_dtype=dtype, drop_tokens=0)
    v = _views(cfg, seed=2, bias_scale=0.25)[0]
    for k in ("W1", "W2", "b1", "b2"):
        v[k] = np.repeat(v[k][:1], cfg.E, axis=0)
    got = moe_oracle.moe_forward(cfg, 1, [v])[0]
    assert (got["slots"] >= 0).all()
    dense = moe_oracle.expert_ffn(cfg, v["A"], v["W1"][0], v["W2"][0], v["b1"][0], v["b2"][0])
    tol = 1e-5 if dtype == 0 else 3e-2
    assert np.abs(got["out"] - dense).max() <= tol * np.abs(dense).max()
    c = c_oracle.moe_forward_rank(cfg, 1, 0, [v])
    assert np.abs(c["out"] - dense).max() <= tol * np.abs(dense).max()


def test_token_order_only_matters_through_capacity():
    """Without drops the layer is a per-token function: permuting the tokens permutes the rows."""
    cfg = KleosConfig(sequence_len=128, hidden_size=64, intermediate_size=64, num_experts=8,
                      torch_dtype=0, drop_tokens=0)
    v = _views(cfg, seed=4)[0]
    base = moe_oracle.moe_forward(cfg, 1, [v])[0]
    perm = np.random.default_rng(0).permutation(cfg.S)
    pv = dict(v, A=v["A"][perm])
    moved = moe_oracle.moe_forward(cfg, 1, [pv])[0]
    assert np.array_equal(np.sort(moved["topk"], axis=1), np.sort(base["topk"][perm], axis=1))
    assert np.array_equal(moved["counts"], base["counts"])
    assert np.abs(moved["out"] - base["out"][perm]).max() <= 1e-6 * np.abs(base["out"]).max()


@pytest.mark.parametrize("cf", [1, 1.25, 2])
def test_capacity_bookkeeping_is_consistent(cf):
    """Per expert: kept rows = min(count, EC), kept slots are 0..kept-1 in ascending token order,
    and a token's dropped choices still count in the normaliser."""
    cfg = KleosConfig(sequence_len=256, hidden_size=64, intermediate_size=64, num_experts=8,
                      torch_dtype=2, capacity_factor=cf)
    v = _views(cfg, seed=6)[0]
    bias = synth.zipf_gate_bias(cfg, 1.2) * 2.0
    for r in (moe_oracle.route(cfg, v["A"], v["Wg"], bias),
              c_oracle.moe_forward_rank(cfg, 1, 0, [v], gate_bias=bias, tokens=[0])):
        assert r["counts"].sum() == cfg.S * cfg.K
        for e in range(cfg.E):
            hit = r["topk"] == e
            slots = r["slots"][hit]                      # token-major order
            kept = slots[slots >= 0]
            assert len(kept) == min(int(r["counts"][e]), cfg.EC)
            assert np.array_equal(kept, np.arange(len(kept)))
            assert (slots[len(kept):] == moe_oracle.DROPPED).all()
        assert np.array_equal(r["routed"], np.minimum(r["counts"], cfg.EC))
        assert (r["mcw"] > 0).all() and (r["mcw"] <= 1.0 + 1e-6).all()


def _routing_inputs(name):
    """(cfg, gate bias or None, A, Wg) of rank 0 of a benchmark layer without building its expert
    weights (routing needs none of them)."""
    from aristos_b200.config import baseline_config
    cfg, extra = baseline_config(name)
    bias = synth.zipf_gate_bias(cfg, extra["zipf"]) if extra["zipf"] else None
    a = synth.round_to_dtype(synth.activations(cfg, 0, 0), cfg.torch_dtype)
    wg = synth.round_to_dtype(synth.gate_weight(cfg, 0), cfg.torch_dtype)
    return cfg, bias, a, wg


@pytest.mark.parametrize("name", ["C1", "C2", "C3", "C4", "C5"])
def test_reference_selection_rule_picks_the_same_experts(name, capsys):
    """The oracle selects on fp64 logits; the reference selects on fp32 probabilities after expf and
    a division (moe/gate.cuh:574-584,654-670).  On every benchmark layer (rank 0, seed 0) the two
    rules must choose the same expert set for every token, and the smallest probability-domain
    gap between the last expert in and the first expert out is reported: that gap, relative to
    the probability, is what an fp32 pipeline has to resolve."""
    cfg, bias, a, wg = _routing_inputs(name)
    lit = moe_oracle.route_reference_rule(cfg, a, wg, bias)
    ref = c_oracle.route_rank(cfg, a, np.vstack([wg, np.zeros((cfg.PX - cfg.E, cfg.H), np.float32)]), bias)
    differ = np.nonzero((np.sort(lit["topk"], axis=1) != np.sort(ref["topk"], axis=1)).any(axis=1))[0]
    with capsys.disabled():
        print(f"\n{name}: min probability gap {lit['min_prob_gap']:.3e} (relative {lit['min_rel_prob_gap']:.3e}), "
              f"fp64 logit margin {ref['margin']:.3e}, tokens selected differently: {differ.tolist()}")
    # fp32 softmax keeps about 1e-7 relative accuracy: gaps well above that cannot flip
    assert lit["min_rel_prob_gap"] > 2e-6 or differ.size == 0
    assert differ.size == 0, f"{name}: literal rule and fp64-logit rule disagree on tokens {differ.tolist()}"


def test_torch_fp64_restatement_agrees_on_c1():
    """A third, independent restatement (torch.matmul / softmax / topk in fp64) of the whole C1
    layer: same expert sets, same counts, outputs within fp32 rounding of the oracle's."""
    import torch
    from aristos_b200.config import baseline_config
    cfg, _ = baseline_config("C1")
    views = [synth.split_packed(cfg, synth.packed_input(cfg, 0, 1), 1)]
    ref = moe_oracle.moe_forward(cfg, 1, views)[0]
    v = {k: torch.from_numpy(np.ascontiguousarray(x)).double() for k, x in views[0].items()}
    logits = v["A"] @ v["Wg"][: cfg.E].T
    probs = torch.softmax(logits.float(), dim=1)            # fp32 softmax, as the kernel
    top = torch.topk(logits, cfg.K, dim=1).indices            # fp64 selection
    assert np.array_equal(np.sort(top.numpy(), axis=1), np.sort(ref["topk"], axis=1))
    sel = torch.zeros(cfg.S, cfg.E, dtype=torch.int64).scatter_(1, top, 1)
    pos = torch.cumsum(sel, dim=0) - 1                        # slots in ascending token order
    assert np.array_equal(sel.sum(0).numpy().astype(np.uint32), ref["counts"])
    mcw = torch.gather(probs, 1, top).sum(1)
    out = torch.zeros(cfg.S, cfg.H, dtype=torch.float64)
    for e in range(cfg.E):
        rows = torch.nonzero((sel[:, e] == 1) & (pos[:, e] < cfg.EC)).squeeze(1)
        if rows.numel() == 0:
            continue
        y1 = torch.relu(v["A"][rows] @ v["W1"][e].T + v["b1"][e]).float().double()   # Element = float
        y2 = (y1 @ v["W2"][e].T + v["b2"][e]).float()
        scaled = (y2 / mcw[rows, None]).float() * probs[rows, e, None]
        out[rows] = (out[rows].float() + scaled.float()).double()
    err = np.abs(out.numpy() - ref["out"]).max() / np.abs(ref["out"]).max()
    assert err <= 2e-6, err
