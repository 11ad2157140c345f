"""One rank of a multi-GPU parity run (launched by torch.distributed.run from the tests).

Runs the layer through the C ABI on this rank's GPU with seeded inputs, `forwards` times, and
writes probabilities, layer output and routing to <out_dir>/rank<r>.npz for the parent test to
compare with the CPU oracle.  The 128-byte bootstrap id travels over a gloo broadcast.
"""
import json
import os
import sys

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
    forwards = int(spec.get("forwards", 2))
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
    packed = synth.packed_input(cfg, rank, world, seed=int(spec.get("seed", 0)))
    raw = synth.encode(packed, cfg.torch_dtype)
    iP = torch.from_numpy(raw.view(np.uint8).copy()).cuda()
    oP = torch.zeros(info.output_elems * info.elem_bytes, dtype=torch.uint8, device="cuda")
    if spec.get("bias") is not None:
        kleos.set_gate_bias(np.asarray(spec["bias"], dtype=np.float32))
    for _ in range(forwards):
        kleos.forward_host(iP, oP)
    st = kleos.last_status()
    routing = kleos.debug_routing(info)
    o = oP.cpu().numpy().view(raw.dtype)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"),
             probs=synth.decode(o[: cfg.S * cfg.PX], cfg.torch_dtype).reshape(cfg.S, cfg.PX),
             out=synth.decode(o[cfg.S * cfg.PX:], cfg.torch_dtype).reshape(cfg.S, cfg.H),
             status=np.array([st.code, st.where, st.detail, st.epoch]), **routing)
    dist.barrier()
    kleos.finalize()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
