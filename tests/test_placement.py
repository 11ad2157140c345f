"""Init-time placement planner (host only): the library's C++ planner against the Python oracle
restating the reference's Decider and expert assignment (os/decider/decider.cuh:37-329), and the
properties the data path relies on.  No GPU is needed."""
import numpy as np
import pytest

from aristos_b200 import kleos
from aristos_b200.config import KleosConfig, baseline_config
from oracle import placement_oracle as po

INTRA = (4.35e-04, 1.29e-02)   # (ms, ms/MB): the two link classes of the reference's own
INTER = (1.12e-02, 5e-02)      # ad-hoc planner driver, csrc/eval.cuh:152-153


def two_level(world, width, intra=INTRA, inter=INTER):
    a = np.zeros((world, world), np.float32)
    b = np.zeros((world, world), np.float32)
    for i in range(world):
        for j in range(world):
            if i != j:
                a[i, j], b[i, j] = intra if i // width == j // width else inter
    return a, b


def model_dict(m: po.Model):
    return dict(moe_stages=m.moe_stages, p2p_buffer=m.p2p_buffer, grad_buffer=m.grad_buffer)


def both(alpha, beta, rate, mem, E, model, rank=0, cost=1, training=False):
    want = po.plan(alpha.tolist(), beta.tolist(), list(rate), list(mem), E, cost, model, training, rank)
    got = kleos.plan_placement(alpha, beta, rate, mem, E, model_dict(model), rank=rank, expert_cost=cost,
                               training=training)
    assert got["feasible"] == want["feasible"]
    assert got["device_to_group"] == want["device_to_group"]
    if want["feasible"]:
        for k in ("group_ranks", "group_rank", "expert_to_member", "local_experts", "expert_slots",
                  "widest_group"):
            assert got[k] == want[k], k
    return got


def test_cost_model_constants_match_the_layer():
    for name in ("C1", "C3", "C5"):
        cfg, _ = baseline_config(name)
        for training in (0, 1):
            cfg.is_training = training
            want = po.model_from_config(cfg)
            assert kleos.placement_model(cfg) == model_dict(want)
    # the reference's shipped layer: 256 stages for inference, 16 MB dispatch buffer
    cfg = KleosConfig()
    m = kleos.placement_model(cfg)
    assert (m["moe_stages"], m["p2p_buffer"]) == (256, 16)


@pytest.mark.parametrize("name,world", [("C3", 8), ("C3", 4), ("C3", 2), ("C4", 8), ("C5", 8)])
def test_uniform_nvswitch_node_gives_the_data_path_sharding(name, world):
    """Identical GPUs, identical links: one group of all ranks, experts split evenly and
    contiguously, which is exactly what kleos_initialize implements."""
    cfg, _ = baseline_config(name)
    model = po.model_from_config(cfg)
    beta = 1.0 / 770e3 * 1e3 * 1.0  # ms per MB at 770 GB/s
    a, b = two_level(world, world, intra=(2e-3, beta))
    rate = [1.0] * world
    mem = [cfg.E] * world
    for rank in (0, world - 1):
        got = both(a, b, rate, mem, cfg.E, model, rank=rank)
        assert got["feasible"] and got["matches_data_path"]
        assert len(set(got["device_to_group"])) == 1
        assert got["group_ranks"] == list(range(world)) and got["group_rank"] == rank
        nlx = cfg.E // world
        assert got["expert_to_member"] == [e // nlx for e in range(cfg.E)]
        assert got["local_experts"] == nlx == got["expert_slots"]


@pytest.mark.parametrize("training", [False, True])
def test_reference_driver_case_two_nodes_of_four(training):
    """Inputs of the reference's ad-hoc planner driver (csrc/eval.cuh:142-233): eight devices in
    two nodes of four, sixteen experts of cost 128, room for eight experts per device."""
    a, b = two_level(8, 4)
    rate = [np.float32(0.43 * 312 * (1e9 / (1024 * 1024 * 1024)))] * 8
    cfg = KleosConfig(is_training=int(training))
    model = po.model_from_config(cfg)
    got = both(a, b, rate, [8] * 8, 16, model, rank=0, cost=128, training=training)
    assert got["feasible"]
    d2g = got["device_to_group"]
    # devices of one node always share a group; a lone device cannot hold the sixteen experts
    assert len(set(d2g[:4])) == 1 and len(set(d2g[4:])) == 1
    assert sorted(np.bincount(got["expert_to_member"], minlength=got["widest_group"]).tolist())[-1] \
        == got["expert_slots"]
    assert sum(1 for e in got["expert_to_member"] if e == got["group_rank"]) == got["local_experts"]


def test_faster_devices_get_more_experts():
    a, b = two_level(4, 4)
    model = po.Model(moe_stages=256, p2p_buffer=16, grad_buffer=100)
    got = both(a, b, [3.0, 1.0, 1.0, 1.0], [64] * 4, 48, model)
    counts = np.bincount(got["expert_to_member"], minlength=4).tolist()
    assert counts[0] == 24 and sum(counts) == 48 and min(counts[1:]) >= 7
    assert not got["matches_data_path"]


def test_memory_limits_are_respected_and_infeasible_is_reported():
    a, b = two_level(4, 4)
    model = po.Model(moe_stages=256, p2p_buffer=16, grad_buffer=100)
    got = both(a, b, [1.0] * 4, [2, 6, 4, 4], 16, model)
    counts = np.bincount(got["expert_to_member"], minlength=4).tolist()
    assert got["feasible"] and counts[0] <= 2 and counts[1] <= 6 and sum(counts) == 16
    bad = both(a, b, [1.0] * 4, [2, 2, 2, 2], 16, model)
    assert not bad["feasible"]


def test_random_topologies_agree_with_the_oracle():
    rng = np.random.default_rng(11)
    for trial in range(60):
        world = int(rng.integers(2, 9))
        width = int(rng.choice([1, 2, 4, world]))
        intra = (float(rng.uniform(1e-4, 1e-3)), float(rng.uniform(5e-3, 2e-2)))
        inter = (float(rng.uniform(5e-3, 5e-2)), float(rng.uniform(2e-2, 2e-1)))
        a, b = two_level(world, max(1, width), intra, inter)
        a *= rng.uniform(0.9, 1.1, a.shape).astype(np.float32)
        rate = rng.uniform(0.5, 4.0, world).astype(np.float32).tolist()
        E = int(rng.choice([8, 16, 24, 64]))
        mem = rng.integers(max(1, E // world), E + 1, world).tolist()
        model = po.Model(moe_stages=int(rng.choice([8, 64, 256])), p2p_buffer=int(rng.choice([1, 16, 64])),
                         grad_buffer=int(rng.choice([10, 500])))
        training = bool(trial % 2)
        cost = int(rng.choice([1, 7, 128]))
        both(a, b, rate, mem, E, model, rank=int(rng.integers(0, world)), cost=cost, training=training)


def test_bad_requests_are_rejected():
    a, b = two_level(2, 2)
    model = dict(moe_stages=1, p2p_buffer=1, grad_buffer=1)
    with pytest.raises(kleos.KleosError):
        kleos.plan_placement(a, b, [1.0, 1.0], [4, 4], 0, model)
    with pytest.raises(kleos.KleosError):
        kleos.plan_placement(a, b, [1.0, 1.0], [4, 4], 8, model, rank=5)


def test_trace_ranges_are_harmless_without_a_profiler(tmp_path):
    """KLEOS_NVTX=1 wraps the entry points in NVTX ranges (domain "Kleos", as the reference's
    telemetry.cuh does); with no tool attached the calls must be no-ops.  Runs in a child process
    because the switch is read once."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import numpy as np\n"
        "from aristos_b200 import kleos\n"
        "a = np.full((2, 2), 1e-3, np.float32); b = np.full((2, 2), 1e-2, np.float32)\n"
        "m = dict(moe_stages=4, p2p_buffer=1, grad_buffer=1)\n"
        "for _ in range(3):\n"
        "    r = kleos.plan_placement(a, b, [1.0, 1.0], [8, 8], 8, m)\n"
        "assert r['feasible'] and r['expert_to_member'] == [0, 0, 0, 0, 1, 1, 1, 1]\n"
        "print('ok')\n")
    env = dict(os.environ, KLEOS_NVTX="1", PYTHONPATH=root)
    out = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True,
                         timeout=120)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr
