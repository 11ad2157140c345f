"""World-size-2 run on CPU (gloo) of the expert-parallel data flow, with the same cell layout
and ownership rules the CUDA kernels use:

  dispatch   row `slot` of cell [source rank][local expert] on the expert's owner rank
  return     row `slot` of cell [global expert] on the source rank
  combine    gate-weighted sum of the returned rows

Each rank routes its own tokens, exchanges cells with its peer over gloo, runs its local experts
and combines; the result must equal the oracle evaluated on the global problem.  This covers the
host-side sharding arithmetic (owner(e), local index, cell addressing, capacity per source
rank) without a GPU; the device path itself is covered by tests/test_gpu_multi.py.
"""
import os
import sys
import tempfile

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from aristos_b200 import synth
    from aristos_b200.config import KleosConfig
    from oracle import moe_oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = KleosConfig(sequence_len=128, hidden_size=64, intermediate_size=128, num_experts=8,
                      torch_dtype=2, capacity_factor=1.25)
    nlx = cfg.local_experts(world)
    mine = synth.split_packed(cfg, synth.packed_input(cfg, rank, world), world)
    rt = moe_oracle.route(cfg, mine["A"], mine["Wg"])

    # dispatch: xcell[owner][src=rank][le][slot][H]; counts travel with the cells
    send = np.zeros((world, nlx, cfg.pEC, cfg.H), dtype=np.float32)
    for t in range(cfg.S):
        for j in range(cfg.K):
            e, slot = int(rt["topk"][t, j]), int(rt["slots"][t, j])
            if slot >= 0:
                send[cfg.owner(e, world), e % nlx, slot] = mine["A"][t]
    routed = rt["routed"].reshape(world, nlx).astype(np.int64)
    recv = [torch.zeros(nlx, cfg.pEC, cfg.H) for _ in range(world)]
    cnt = [torch.zeros(nlx, dtype=torch.int64) for _ in range(world)]
    # gloo has no all_to_all on CPU: every rank gathers everything and keeps its slice
    gathered = [torch.zeros(world, nlx, cfg.pEC, cfg.H) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(send))
    gcnt = [torch.zeros(world, nlx, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(gcnt, torch.from_numpy(routed))
    for src in range(world):
        recv[src] = gathered[src][rank]
        cnt[src] = gcnt[src][rank]

    # local experts on the rows that arrived; results go back to cell [global expert] of the source
    back = np.zeros((world, nlx, cfg.pEC, cfg.H), dtype=np.float32)
    for src in range(world):
        for le in range(nlx):
            n = int(cnt[src][le])
            if n:
                back[src, le, :n] = moe_oracle.expert_ffn(
                    cfg, recv[src][le, :n].numpy(), mine["W1"][le], mine["W2"][le],
                    mine["b1"][le], mine["b2"][le])
    gback = [torch.zeros(world, nlx, cfg.pEC, cfg.H) for _ in range(world)]
    dist.all_gather(gback, torch.from_numpy(back))
    ycell = np.zeros((cfg.E, cfg.pEC, cfg.H), dtype=np.float32)
    for owner in range(world):
        ycell[owner * nlx:(owner + 1) * nlx] = gback[owner][rank].numpy()

    out = np.zeros((cfg.S, cfg.H), dtype=np.float32)
    for t in range(cfg.S):
        for j in range(cfg.K):
            e, slot = int(rt["topk"][t, j]), int(rt["slots"][t, j])
            if slot >= 0:
                v = moe_oracle.round_elem(ycell[e, slot] / rt["mcw"][t], cfg.torch_dtype)
                w = moe_oracle.round_elem(rt["probs"][t, e] * v, cfg.torch_dtype)
                out[t] = moe_oracle.round_elem(out[t] + w, cfg.torch_dtype)
    np.save(os.path.join(out_dir, f"out{rank}.npy"), out)
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_dataflow_world2_gloo():
    import torch.multiprocessing as mp
    sys.path.insert(0, ROOT)
    from aristos_b200 import synth
    from aristos_b200.config import KleosConfig
    from oracle import moe_oracle

    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, 29541, d), nprocs=world, join=True)
        cfg = KleosConfig(sequence_len=128, hidden_size=64, intermediate_size=128, num_experts=8,
                          torch_dtype=2, capacity_factor=1.25)
        views = [synth.split_packed(cfg, synth.packed_input(cfg, r, world), world)
                 for r in range(world)]
        ref = moe_oracle.moe_forward(cfg, world, views)
        for r in range(world):
            got = np.load(os.path.join(d, f"out{r}.npy"))
            assert np.array_equal(got, ref[r]["out"]), f"rank {r}"


def test_bootstrap_id_travels_over_gloo():
    """The 128-byte bootstrap id is opaque bytes; check the broadcast pattern bench.py uses."""
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_id_worker, args=(2, 29543, d), nprocs=2, join=True)
        a = open(os.path.join(d, "id0"), "rb").read()
        b = open(os.path.join(d, "id1"), "rb").read()
        assert a == b and len(a) == 128 and a != bytes(128)


def _id_worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    idt = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        idt.copy_(torch.arange(1, 129, dtype=torch.uint8))
    dist.broadcast(idt, 0)
    open(os.path.join(out_dir, f"id{rank}"), "wb").write(bytes(idt.numpy().tobytes()))
    dist.destroy_process_group()
