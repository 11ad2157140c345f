"""One rank of a multi-GPU parity run (launched by torch.distributed.run from the tests).

Runs the layer through the C ABI on this rank's GPU with seeded inputs and writes gate
probabilities, layer output and routing of the LAST forward to <out_dir>/rank<r>.npz for the
parent test to compare with the CPU oracle.  The 128-byte bootstrap id travels over a gloo
broadcast.  Keys of the JSON spec:
  cfg         KleosConfig fields
  seed        seed of the weights (and of the activations when act_seeds is absent)
  act_seeds   one activation seed per forward: every forward then sees DIFFERENT tokens, so a
              kernel that read a cell, a result row or a flag left over from the forward before
              cannot reproduce the oracle's answer for the last one
  forwards    number of forwards when act_seeds is absent
  rows        token indices whose output rows are saved (default: all)
  bias        optional gate bias, E floats
  sleep       optional {"rank": r, "ms": m}: that rank sleeps on the host before every forward but
              the first, so the ranks enter their forwards skewed in time
  mode        "device" (kleos_forward, default) or "host" (the pipelined host-buffer entry point)
"""
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    from aristos_b200 import kleos, synth
    from aristos_b200.config import KleosConfig

    spec = json.load(open(sys.argv[1]))
    out_dir = sys.argv[2]
    cfg = KleosConfig(**spec["cfg"])
    seed = int(spec.get("seed", 0))
    act_seeds = spec.get("act_seeds") or [seed] * int(spec.get("forwards", 2))
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dist.init_process_group("gloo")
    idt = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        idt.copy_(torch.frombuffer(bytearray(kleos.get_unique_id()), dtype=torch.uint8))
    dist.broadcast(idt, 0)
    torch.cuda.set_device(local)
    kleos.set_device(local)
    info = kleos.initialize(cfg, rank, world, bytes(idt.numpy().tobytes()))
    packed = synth.packed_input(cfg, rank, world, seed=seed)
    raw = synth.encode(packed, cfg.torch_dtype)
    n_act = cfg.S * cfg.H
    iP = torch.from_numpy(raw.view(np.uint8).copy()).cuda()
    oP = torch.zeros(info.output_elems * info.elem_bytes, dtype=torch.uint8, device="cuda")
    if spec.get("bias") is not None:
        kleos.set_gate_bias(np.asarray(spec["bias"], dtype=np.float32))
    acts = {}
    for s in set(act_seeds):
        a = synth.encode(synth.round_to_dtype(synth.activations(cfg, rank, s).ravel(), cfg.torch_dtype),
                         cfg.torch_dtype)
        acts[s] = torch.from_numpy(a.view(np.uint8).copy())
    sleep = spec.get("sleep") or {}
    host_mode = spec.get("mode", "device") == "host"
    host_out = torch.zeros(n_act * info.elem_bytes, dtype=torch.uint8).pin_memory() if host_mode else None
    pinned = {s: a.pin_memory() for s, a in acts.items()} if host_mode else None
    dev_acts = {s: a.cuda() for s, a in acts.items()} if not host_mode else None
    dist.barrier()
    stream = torch.cuda.Stream()  # a caller-owned, non-default stream for the device path
    torch.cuda.synchronize()
    for i, s in enumerate(act_seeds):
        if i and sleep.get("rank") == rank:
            torch.cuda.synchronize()
            time.sleep(float(sleep.get("ms", 0)) * 1e-3)
        if host_mode:
            kleos.forward_from_host_async(pinned[s], iP, oP, host_out)
        else:
            with torch.cuda.stream(stream):
                iP[: n_act * info.elem_bytes].copy_(dev_acts[s], non_blocking=True)
                kleos.forward_host(iP, oP, stream.cuda_stream)
    if host_mode:
        kleos.host_sync()
    torch.cuda.synchronize()
    st = kleos.last_status()
    routing = kleos.debug_routing(info)
    o = oP.cpu().numpy().view(raw.dtype)
    if host_mode:  # the pipelined entry point delivers the layer output to the host buffer only
        out = synth.decode(host_out.numpy().view(raw.dtype), cfg.torch_dtype).reshape(cfg.S, cfg.H)
    else:
        out = synth.decode(o[cfg.S * cfg.PX:], cfg.torch_dtype).reshape(cfg.S, cfg.H)
    rows = spec.get("rows")
    if rows is not None:
        out = out[np.asarray(rows, dtype=np.int64)]
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"),
             probs=synth.decode(o[: cfg.S * cfg.PX], cfg.torch_dtype).reshape(cfg.S, cfg.PX),
             out=out, status=np.array([st.code, st.where, st.detail, st.epoch]), **routing)
    dist.barrier()
    kleos.finalize()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
