"""Parity of the CUDA layer (through the C ABI, one GPU) against the CPU oracle."""
import numpy as np
import pytest

from aristos_b200.config import KleosConfig, baseline_config
from aristos_b200 import synth
from oracle import c_oracle, moe_oracle
from tests import moe_harness as hz

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["launches", "persistent"])
def arrangement(request, monkeypatch):
    """Every case runs twice: as separate launches (the default) and with KLEOS_FLOW=1, where
    16-bit routed layers run as ONE persistent kernel.  Cases whose element type never takes the
    persistent kernel are not repeated."""
    if request.param == "persistent":
        args = getattr(getattr(request.node, "callspec", None), "params", {})
        if args.get("dtype", 2) not in (2, 3) or "tf32" in request.node.name or "dense" in request.node.name \
                or "single_expert" in request.node.name or args.get("name") in ("C2", "fp32_w1", "fp32_top1",
                                                                                "tf32_gelu_biased"):
            pytest.skip("this layer never runs the persistent kernel")
        monkeypatch.setenv("KLEOS_FLOW", "1")
    else:
        monkeypatch.delenv("KLEOS_FLOW", raising=False)
    return request.param


def _small(dtype, **kw):
    base = dict(sequence_len=256, hidden_size=512, intermediate_size=1024, num_experts=8,
                torch_dtype=dtype)
    base.update(kw)
    return KleosConfig(**base)


@pytest.mark.parametrize("dtype", [0, 2, 3])
def test_c1_shape_full_parity(dtype):
    cfg = _small(dtype)
    packed, views = hz.make_inputs(cfg, 1)
    ref = moe_oracle.moe_forward(cfg, 1, views)[0]
    probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0])
    hz.check_against_oracle(cfg, ref, probs, out, routing)


@pytest.mark.parametrize("dtype", [0, 2])
def test_repeat_forwards_and_host_path(dtype):
    """Flags carry an epoch, so back-to-back forwards need no clearing; the host-buffer entry
    point returns the same rows as the device path."""
    cfg = _small(dtype)
    packed, views = hz.make_inputs(cfg, 1)
    ref = moe_oracle.moe_forward(cfg, 1, views)[0]
    probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0], forwards=3, via_host=True)
    hz.check_against_oracle(cfg, ref, probs, out, routing)


@pytest.mark.parametrize("dtype,kw", [
    (2, dict(num_experts=128, sequence_len=512, hidden_size=256, intermediate_size=320,
             capacity_factor=1.25)),          # PX = 128, fractional capacity, N tail (320 % 256)
    (0, dict(num_experts=16, sequence_len=384, hidden_size=192, intermediate_size=192)),
    (2, dict(num_experts=4, sequence_len=128, hidden_size=64, intermediate_size=64, expert_top_k=1)),
    (2, dict(num_experts=8, sequence_len=256, hidden_size=256, intermediate_size=512, expert_top_k=4)),
    (2, dict(hidden_act=1)),                  # GELU
    (0, dict(hidden_act=1)),
    (3, dict(hidden_act=1, num_experts=128, sequence_len=512, hidden_size=256,
             intermediate_size=320)),          # fp16, GELU, PX = 128
    (2, dict(drop_tokens=0, sequence_len=128, hidden_size=128, intermediate_size=128)),
])
def test_shapes_and_modes(dtype, kw):
    cfg = _small(dtype, **kw)
    packed, views = hz.make_inputs(cfg, 1)
    ref = moe_oracle.moe_forward(cfg, 1, views)[0]
    probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0])
    hz.check_against_oracle(cfg, ref, probs, out, routing)


@pytest.mark.parametrize("dtype,kw", [
    (0, dict()), (2, dict()), (3, dict(hidden_act=1)),
    (2, dict(num_experts=128, sequence_len=512, hidden_size=256, intermediate_size=320,
             hidden_act=1)),
])
def test_nonzero_ffn_biases(dtype, kw):
    """b1 and b2 drawn from N(0, 0.5): the bias path of both GEMM epilogues (the benchmark
    layers themselves use zero biases)."""
    cfg = _small(dtype, **kw)
    packed, views = hz.make_inputs(cfg, 1, bias_scale=0.5)
    assert np.abs(views[0]["b1"]).max() > 0.5 and np.abs(views[0]["b2"]).max() > 0.5
    ref = moe_oracle.moe_forward(cfg, 1, views)[0]
    probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0])
    hz.check_against_oracle(cfg, ref, probs, out, routing)


@pytest.mark.parametrize("dtype,kw,via_host", [
    (0, dict(sequence_len=256, hidden_size=192, intermediate_size=320), False),
    (2, dict(sequence_len=384, hidden_size=256, intermediate_size=320), False),   # odd panel count, N tail
    (2, dict(sequence_len=1024, hidden_size=512, intermediate_size=1024, hidden_act=1), True),
    (3, dict(sequence_len=256, hidden_size=128, intermediate_size=256, hidden_act=1), False),
])
def test_single_expert_layer_is_the_dense_ffn(dtype, kw, via_host):
    """num_experts == 1: packed buffers without gate weight / probabilities, output = FFN(A)
    (reference moe/moe.cuh:174-177, moe/fffn.cuh:31-167)."""
    cfg = _small(dtype, num_experts=1, expert_top_k=1, **kw)
    packed, views = hz.make_inputs(cfg, 1, bias_scale=0.5)
    ref = c_oracle.dense_ffn(cfg, views[0])
    _, out, _ = hz.run_layer_single_gpu(cfg, packed[0], forwards=3 if via_host else 1,
                                        via_host=via_host)
    err = np.abs(out - ref).max() / np.abs(ref).max()
    assert err <= hz.TOL[dtype], f"dense layer error {err}"


@pytest.mark.parametrize("simt", [False, True], ids=["tcgen05", "fp32-fma"])
@pytest.mark.parametrize("kw", [
    dict(),                                                     # C1 shape
    dict(num_experts=16, sequence_len=384, hidden_size=192, intermediate_size=320,
         hidden_act=1),                                         # GELU, N tail (320 % 256), K = 6 slices of 32
    dict(num_experts=1, expert_top_k=1, sequence_len=384, hidden_size=256, intermediate_size=320),  # dense
], ids=["c1", "gelu-tail", "dense"])
def test_tf32_layer(monkeypatch, kw, simt):
    """torch_dtype 1: fp32 words with a 10-bit mantissa.  Both GEMM back ends (tcgen05 kind::tf32
    and the FP32 FMA kernel, selected by KLEOS_DEBUG_SIMT_GEMM) against the oracle, nonzero
    biases, routing bit-exact."""
    if simt:
        monkeypatch.setenv("KLEOS_DEBUG_SIMT_GEMM", "1")
    else:
        monkeypatch.delenv("KLEOS_DEBUG_SIMT_GEMM", raising=False)
    cfg = _small(1, **kw)
    packed, views = hz.make_inputs(cfg, 1, bias_scale=0.5)
    probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0])
    assert np.all((out.view(np.uint32) & 0x1FFF) == 0), "outputs must be TF32 words"
    if cfg.dense:
        ref = c_oracle.dense_ffn(cfg, views[0])
        err = np.abs(out - ref).max() / np.abs(ref).max()
        assert err <= hz.TOL[1], f"dense tf32 error {err}"
    else:
        ref = moe_oracle.moe_forward(cfg, 1, views)[0]
        hz.check_against_oracle(cfg, ref, probs, out, routing)


@pytest.mark.parametrize("dtype,kw", [
    (2, dict()), (0, dict()), (1, dict()),
    (2, dict(num_experts=128, sequence_len=512, hidden_size=256, intermediate_size=320)),   # PX = 128
    (0, dict(num_experts=200, sequence_len=256, hidden_size=128, intermediate_size=128)),   # PX = 256, FFMA router
])
def test_training_mode_gate_statistics(dtype, kw):
    """is_training = 1: mean probability per expert, mean selection count and the auxiliary
    loss of the last forward against the oracle (reference moe/gate.cuh:607-635,698-705,763-773);
    the layer output is unaffected."""
    import torch
    from aristos_b200 import kleos
    cfg = _small(dtype, is_training=1, **kw)
    packed, views = hz.make_inputs(cfg, 1)
    ref = moe_oracle.moe_forward(cfg, 1, views)[0]
    raw = synth.encode(packed[0], dtype)
    info = kleos.initialize(cfg, 0, 1)
    try:
        iP = torch.from_numpy(raw.view(np.uint8).copy()).cuda()
        oP = torch.zeros(info.output_elems * info.elem_bytes, dtype=torch.uint8, device="cuda")
        for _ in range(2):  # every forward overwrites the statistics
            kleos.forward_host(iP, oP)
        assert kleos.last_status().code == 0
        st = kleos.gate_stats(info)
        routing = kleos.debug_routing(info)
    finally:
        kleos.finalize()
    assert np.array_equal(routing["counts"], ref["counts"])
    assert np.array_equal(st["mean_count"], (ref["counts"].astype(np.float32) / np.float32(cfg.S)))
    assert np.abs(st["mean_prob"] - ref["mean_prob"]).max() <= 2e-6
    assert abs(st["mean_prob"].sum() - 1.0) <= 1e-5
    assert abs(st["loss"] - ref["gate_loss"]) <= 1e-6 * max(1.0, abs(ref["gate_loss"]))


def test_gate_statistics_need_training_mode():
    from aristos_b200 import kleos
    cfg = _small(2)
    info = kleos.initialize(cfg, 0, 1)
    try:
        with pytest.raises(kleos.KleosError):
            kleos.gate_stats(info)
    finally:
        kleos.finalize()


def test_zipf_bias_hot_experts_and_drops():
    """Skewed routing: hot experts overflow their capacity, cold experts receive nothing."""
    cfg = _small(2, num_experts=32, sequence_len=1024, hidden_size=256, intermediate_size=256,
                 capacity_factor=1.25)
    bias = synth.zipf_gate_bias(cfg, 1.2) * 2.0
    packed, views = hz.make_inputs(cfg, 1)
    ref = moe_oracle.moe_forward(cfg, 1, views, gate_bias=bias)[0]
    assert (ref["slots"] < 0).sum() > 0 and (ref["counts"] == 0).sum() >= 0
    probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0], gate_bias=bias)
    hz.check_against_oracle(cfg, ref, probs, out, routing)


@pytest.mark.parametrize("name", ["C2", "C3"])
def test_baseline_config_sampled(name):
    """Full-size benchmark layers on one GPU: routing checked for every token, layer output
    for a seeded sample of tokens (the oracle's FFN is evaluated only for those)."""
    cfg, _ = baseline_config(name)
    packed, views = hz.make_inputs(cfg, 1)
    rng = np.random.default_rng(0)
    rows = np.sort(rng.choice(cfg.S, size=96, replace=False)).astype(np.int32)
    ref = c_oracle.moe_forward_rank(cfg, 1, 0, views, tokens=rows)
    probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0])
    hz.check_against_oracle(cfg, ref, probs, out, routing, rows=rows)


@pytest.mark.parametrize("name", ["fp32_w1", "bf16_w1", "fp32_top1", "tf32_gelu_biased", "fp16_biased"])
def test_against_committed_golden_fixtures(name):
    from tests import golden_util
    cfg, world, bias, packed, _, expect = golden_util.load(name)
    assert world == 1
    probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0], gate_bias=bias)
    ref = dict(expect[0])
    ref["margin"] = 1.0  # fixtures were generated from seeds whose margins were checked
    hz.check_against_oracle(cfg, ref, probs, out, routing)


@pytest.mark.parametrize("dtype,experts", [(2, 8), (0, 8), (2, 1), (1, 8), (1, 1)])
def test_pipelined_host_path_matches_synchronous_path(dtype, experts):
    """Three queued end-to-end steps with alternating inputs and separate host outputs: each
    must equal what the synchronous host-buffer call returns for the same input."""
    import torch
    from aristos_b200 import kleos
    cfg = _small(dtype, num_experts=experts, expert_top_k=min(2, experts))
    eb = cfg.elem_bytes
    raws = [synth.encode(synth.packed_input(cfg, 0, 1, seed=s), dtype) for s in (0, 5)]
    info = kleos.initialize(cfg, 0, 1)
    try:
        iP = torch.from_numpy(raws[0].view(np.uint8).copy()).cuda()
        oP = torch.zeros(info.output_elems * eb, dtype=torch.uint8, device="cuda")
        n = cfg.S * cfg.H
        acts = [np.ascontiguousarray(r[:n]) for r in raws]
        want = []
        for a in acts:
            o = np.zeros(n, dtype=a.dtype)
            kleos.forward_from_host(a, iP, oP, o)
            want.append(o)
        pinned_in = [torch.from_numpy(a.view(np.uint8).copy()).pin_memory() for a in acts]
        outs = [torch.zeros(n * eb, dtype=torch.uint8).pin_memory() for _ in range(3)]
        for step, which in enumerate((0, 1, 0)):
            kleos.forward_from_host_async(pinned_in[which], iP, oP, outs[step])
        kleos.host_sync()
        for step, which in enumerate((0, 1, 0)):
            got = outs[step].numpy().view(acts[0].dtype)
            assert np.array_equal(got, want[which]), f"step {step}"
    finally:
        kleos.finalize()


def test_bounded_wait_reports_status_and_context_survives():
    """Failure path without faulting anything: with the return flags suppressed the combine's
    wait runs out after KLEOS_WAIT_MS, the status says where, and after clearing it the same
    layer runs correctly again."""
    import os
    import torch
    from aristos_b200 import kleos
    cfg = _small(2)
    packed, views = hz.make_inputs(cfg, 1)
    ref = moe_oracle.moe_forward(cfg, 1, views)[0]
    raw = synth.encode(packed[0], 2)
    old = os.environ.get("KLEOS_WAIT_MS")
    os.environ["KLEOS_WAIT_MS"] = "50"
    try:
        info = kleos.initialize(cfg, 0, 1)
    finally:
        if old is None:
            os.environ.pop("KLEOS_WAIT_MS", None)
        else:
            os.environ["KLEOS_WAIT_MS"] = old
    try:
        lib = kleos.load_library()
        iP = torch.from_numpy(raw.view(np.uint8).copy()).cuda()
        oP = torch.zeros(info.output_elems * 2, dtype=torch.uint8, device="cuda")
        assert lib.kleos_debug_suppress_return_flag(1) == 0
        kleos.forward_host(iP, oP)
        st = kleos.last_status()
        assert st.code == -6 and st.where == 2, (st.code, st.where)  # KLEOS_E_DEVICE at the combine wait
        assert lib.kleos_debug_suppress_return_flag(0) == 0
        assert lib.kleos_clear_status() == 0
        kleos.forward_host(iP, oP)
        st = kleos.last_status()
        assert st.code == 0
        o = oP.cpu().numpy().view(np.uint16)
        out = synth.decode(o[cfg.S * cfg.PX:], 2).reshape(cfg.S, cfg.H)
        err = np.abs(out - ref["out"]).max() / np.abs(ref["out"]).max()
        assert err <= hz.TOL[2]
    finally:
        kleos.finalize()


def test_top_k_equal_to_number_of_experts():
    cfg = _small(2, num_experts=4, expert_top_k=4, sequence_len=128, hidden_size=128,
                 intermediate_size=128)
    packed, views = hz.make_inputs(cfg, 1)
    ref = moe_oracle.moe_forward(cfg, 1, views)[0]
    ref["margin"] = 1.0  # every expert is selected: no k-th / (k+1)-th gap exists
    probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0])
    hz.check_against_oracle(cfg, ref, probs, out, routing)


@pytest.mark.parametrize("name", ["C4", "C5"])
def test_large_baseline_layers_single_gpu_sampled(name):
    """The imbalanced 128-expert layer (Zipf gate bias, capacity 1.25, heavy drops) and the
    large-FFN layer, all experts on one GPU: routing for every token, outputs for a sample."""
    cfg, extra = baseline_config(name)
    packed, views = hz.make_inputs(cfg, 1)
    bias = synth.zipf_gate_bias(cfg, extra["zipf"]) if extra["zipf"] else None
    rng = np.random.default_rng(1)
    rows = np.sort(rng.choice(cfg.S, size=64, replace=False)).astype(np.int32)
    ref = c_oracle.moe_forward_rank(cfg, 1, 0, views, gate_bias=bias, tokens=rows)
    probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0], gate_bias=bias)
    hz.check_against_oracle(cfg, ref, probs, out, routing, rows=rows)


@pytest.mark.parametrize("kw", [
    dict(sequence_len=512, num_experts=16),
    dict(num_experts=128, sequence_len=512, hidden_size=256, intermediate_size=320, capacity_factor=1.25,
         hidden_act=1),
    dict(num_experts=8, sequence_len=256, hidden_size=256, intermediate_size=512, expert_top_k=4),
], ids=["e16", "e128-gelu-tail", "top4"])
def test_separate_launches_give_the_persistent_kernels_results(monkeypatch, kw, arrangement):
    """KLEOS_FLOW=1 runs router, dispatch, plan, GEMM1, GEMM2 and combine as one persistent kernel,
    the default as separate launches; both arrangements must match the oracle, and each other
    bit for bit."""
    if arrangement == "persistent":
        pytest.skip("compares both arrangements itself")
    cfg = _small(2, **kw)
    packed, views = hz.make_inputs(cfg, 1, bias_scale=0.5)
    ref = moe_oracle.moe_forward(cfg, 1, views)[0]
    outs = []
    for flow in ("0", "1"):
        monkeypatch.setenv("KLEOS_FLOW", flow)
        probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0], forwards=3)
        hz.check_against_oracle(cfg, ref, probs, out, routing)
        outs.append(out)
    assert np.array_equal(outs[0], outs[1])


def test_persistent_kernel_reports_its_timeline(arrangement):
    """kleos_forward_bench on a 16-bit routed layer: the milestones of the one kernel are ordered
    (plan, first tile, last GEMM1 tile, last tile, end) and lie inside the forward's duration."""
    import torch
    from aristos_b200 import kleos
    if arrangement != "persistent":
        pytest.skip("separate launches have no kernel timeline")
    cfg = _small(2, sequence_len=1024, num_experts=16)
    raw = synth.encode(synth.packed_input(cfg, 0, 1), 2)
    info = kleos.initialize(cfg, 0, 1)
    try:
        iP = torch.from_numpy(raw.view(np.uint8).copy()).cuda()
        oP = torch.zeros(info.output_elems * 2, dtype=torch.uint8, device="cuda")
        kleos.forward_host_bench(iP, oP, skip=2, trials=4)
        tl = kleos.flow_timeline()
        ph = kleos.phase_times()
        st = kleos.flow_stamps()
    finally:
        kleos.finalize()
    # the same milestones block by block: every block starts and ends, in that order
    assert st.ndim == 2 and st.shape[0] >= 2 and st.shape[1] >= len(kleos.FLOW_MILESTONES)
    i0, i1 = kleos.FLOW_MILESTONES.index("start"), kleos.FLOW_MILESTONES.index("end")
    assert (st[:, i0] > 0).all() and (st[:, i1] >= st[:, i0]).all()
    assert 0 < tl["planned"] <= tl["last_gemm1_tile"] <= tl["last_tile"] <= tl["end"]
    assert tl["first_tile"] <= tl["last_tile"] and tl["dispatched"] <= tl["end"] and tl["combined"] <= tl["end"]
    assert tl["end"] <= ph["total"] * 1.05 + 0.01


def test_dense_layer_in_a_multi_rank_launch_needs_no_connection():
    """num_experts == 1 with world > 1: every rank runs the same FFN on its own tokens, the ranks
    are never connected (no id is passed), and initialise / forward / finalise work on each of
    them alone."""
    import torch
    from aristos_b200 import kleos
    cfg = _small(2, num_experts=1, expert_top_k=1, sequence_len=256, hidden_size=128,
                 intermediate_size=256)
    packed, views = hz.make_inputs(cfg, 1, bias_scale=0.5)
    ref = c_oracle.dense_ffn(cfg, views[0])
    raw = synth.encode(packed[0], 2)
    for rank in (0, 1):
        kleos.set_device(0)
        info = kleos.initialize(cfg, rank, 2, None)
        try:
            assert info.world == 2 and info.local_experts == 1
            iP = torch.from_numpy(raw.view(np.uint8).copy()).cuda()
            oP = torch.zeros(info.output_elems * 2, dtype=torch.uint8, device="cuda")
            kleos.forward_host(iP, oP)
            assert kleos.last_status().code == 0
            out = synth.decode(oP.cpu().numpy().view(np.uint16), 2).reshape(cfg.S, cfg.H)
        finally:
            kleos.finalize()
        assert np.abs(out - ref).max() / np.abs(ref).max() <= hz.TOL[2]


def test_expert_cell_with_more_than_65535_rows():
    """Two experts, top-1, 131072 tokens: the capacity is 65536 rows per expert and the busier
    expert fills it, which a 16-bit row count would wrap to zero."""
    cfg = _small(2, num_experts=2, expert_top_k=1, sequence_len=131072, hidden_size=64,
                 intermediate_size=64)
    assert cfg.EC == 65536
    packed, views = hz.make_inputs(cfg, 1)
    rng = np.random.default_rng(3)
    rows = np.sort(rng.choice(cfg.S, size=256, replace=False)).astype(np.int32)
    ref = c_oracle.moe_forward_rank(cfg, 1, 0, views, tokens=rows)
    assert ref["routed"].max() == 65536
    probs, out, routing = hz.run_layer_single_gpu(cfg, packed[0])
    hz.check_against_oracle(cfg, ref, probs, out, routing, rows=rows)
