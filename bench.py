#!/usr/bin/env python
"""Benchmark of the MoE layer forward pass.

  python bench.py --gpus N --steps K --warmup W            the CUDA path (this repository)
  python bench.py --impl reference --steps K --warmup W     the CPU restatement of the reference

One "step" is one forward pass of the layer over one batch of synthetic tokens on every rank.
Workload: the 64-expert, 8192-tokens-per-GPU, H = I = 2048, top-2, bf16 layer (benchmark layer
C3), experts sharded evenly over the N ranks; at N = 1 all 64 experts are local.  Prints one
JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from aristos_b200.config import baseline_config  # noqa: E402

METRIC = "moe_layer_fwd_tokens_per_s"
KERNELS_PER_FORWARD = 9  # route, refine, tile histogram, slots, dispatch, plan, GEMM1, GEMM2, combine


def workload(name: str):
    """(config, description).  C3 is the benchmark layer the headline metric is quoted on; C3q is
    the same layer at a quarter of the tokens and experts (same tile shapes, about 0.4 GB on
    the device) and exists so that profiler captures stay small."""
    from aristos_b200.config import KleosConfig
    if name == "C3q":
        return (KleosConfig(sequence_len=2048, hidden_size=2048, intermediate_size=2048,
                            num_experts=16, torch_dtype=2),
                "C3q: S=2048 tokens/rank, H=I=2048, E=16, top-2, CF=1, bf16 (profiling size)")
    if name == "C3r8":
        # what ONE rank of the 8-rank C3 layer computes locally: 8 experts x 2048 routed rows
        return (KleosConfig(sequence_len=8192, hidden_size=2048, intermediate_size=2048,
                            num_experts=8, torch_dtype=2),
                "C3r8: S=8192 tokens, H=I=2048, E=8, top-2, CF=1, bf16 (per-rank shape of C3 at 8 ranks)")
    if name == "C2t":
        # the float benchmark layer C2 with torch_dtype 1: TF32 words on the tensor cores
        return (KleosConfig(sequence_len=4096, hidden_size=2048, intermediate_size=2048,
                            num_experts=16, torch_dtype=1),
                "C2t: S=4096 tokens/rank, H=I=2048, E=16, top-2, CF=1, tf32")
    if name == "F3":
        # single-expert layer = the plain FFN (the reference's dense kernel); 16384 tokens so
        # that activations, intermediate and output (208 MB with the weights) exceed L2
        return (KleosConfig(sequence_len=16384, hidden_size=2048, intermediate_size=2048,
                            num_experts=1, expert_top_k=1, torch_dtype=2),
                "F3: dense FFN (num_experts=1), S=16384 tokens/rank, H=I=2048, bf16")
    if name == "F3q":
        return (KleosConfig(sequence_len=4096, hidden_size=2048, intermediate_size=2048,
                            num_experts=1, expert_top_k=1, torch_dtype=2),
                "F3q: dense FFN (num_experts=1), S=4096 tokens/rank, H=I=2048, bf16 (profiling size)")
    cfg, _ = baseline_config(name)
    return cfg, (f"{name}: S={cfg.S} tokens/rank, H={cfg.H}, I={cfg.I}, E={cfg.E}, "
                 f"top-{cfg.K}, CF={cfg.capacity_factor}, {cfg.dtype_name}")


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tflops=float(p["bf16_tflops"]), hbm=float(p["hbm_gbs"]), source="measured")
    return dict(tflops=1590.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), r[2:]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None,
                    sm_max_mhz=max(mx) if mx else None, reasons=sorted(reasons),
                    samples=len(sm))


def torch_dtype_of(cfg):
    import torch
    return {0: torch.float32, 1: torch.float32, 2: torch.bfloat16, 3: torch.float16}[cfg.torch_dtype]


def synth_on_device(cfg, rank, world, device):
    """Packed bf16 input of one rank, generated on the GPU: activations N(0,1) seeded by rank,
    gate and expert weights N(0, 1/sqrt(fan_in)) seeded per global expert, zero biases."""
    import torch
    tdt = torch_dtype_of(cfg)
    off = cfg.input_offsets(world)
    nlx = cfg.local_experts(world)
    buf = torch.zeros(off["end"], dtype=tdt, device=device)
    gen = torch.Generator(device=device)
    gen.manual_seed(1000 + rank)
    buf[off["A"]:off["Wg"]] = torch.randn(cfg.S * cfg.H, generator=gen, device=device).to(tdt)
    gen.manual_seed(7)
    if not cfg.dense:
        buf[off["Wg"]:off["Wg"] + cfg.E * cfg.H] = (
            torch.randn(cfg.E * cfg.H, generator=gen, device=device) / cfg.H ** 0.5).to(tdt)
    ih = cfg.I * cfg.H
    for le in range(nlx):
        e = 0 if cfg.dense else rank * nlx + le
        gen.manual_seed(100000 + e)
        buf[off["W1"] + le * ih: off["W1"] + (le + 1) * ih] = (
            torch.randn(ih, generator=gen, device=device) / cfg.H ** 0.5).to(tdt)
        buf[off["W2"] + le * ih: off["W2"] + (le + 1) * ih] = (
            torch.randn(ih, generator=gen, device=device) / cfg.I ** 0.5).to(tdt)
    if cfg.torch_dtype == 1:
        # TF32 words: 10-bit mantissa, round to nearest even, low 13 bits clear
        u = buf.view(torch.int32)
        u.copy_((u + 0xFFF + ((u >> 13) & 1)) & ~0x1FFF)
    return buf


def cpu_sample_tokens_per_s(cfg, views, sample_tokens: int, repeats: int = 1):
    """Times the C restatement of the reference's math (fp32 accumulation, all host threads)
    on the first `sample_tokens` tokens of one rank; routing covers all S tokens."""
    from oracle import c_oracle
    c_oracle.use_all_cores()
    rows = np.arange(sample_tokens, dtype=np.int32)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        if cfg.dense:
            c_oracle.dense_ffn(cfg, views[0], tokens=rows, accum64=False)
        else:
            c_oracle.moe_forward_rank(cfg, 1, 0, views, tokens=rows, accum64=False)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return sample_tokens / best, best, c_oracle.num_threads()


def host_views_from_device(cfg, buf, world):
    from aristos_b200 import synth
    host = buf.float().cpu().numpy()
    return [synth.split_packed(cfg, host, world)]


def run_reference(args):
    """The reference's own path restated for the CPU (the reference has no CPU implementation
    and cannot be built for sm_100), timed on the host cores; rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from aristos_b200 import synth
    from oracle import c_oracle
    torch.set_num_threads(c_oracle.use_all_cores())  # launchers export OMP_NUM_THREADS=1
    cfg, _ = baseline_config("C3")
    torch.manual_seed(0)
    off = cfg.input_offsets(1)
    buf = torch.zeros(off["end"], dtype=torch.float32)
    buf[off["A"]:off["Wg"]] = torch.randn(cfg.S * cfg.H)
    buf[off["Wg"]:off["Wg"] + cfg.E * cfg.H] = torch.randn(cfg.E * cfg.H) / cfg.H ** 0.5
    n = 2 * cfg.E * cfg.I * cfg.H
    buf[off["W1"]:off["W1"] + n] = torch.randn(n) / cfg.H ** 0.5  # fan_in H = I for this layer
    host = buf.bfloat16().float().numpy()
    views = [synth.split_packed(cfg, host, 1)]
    sample = args.cpu_sample
    for _ in range(args.warmup):
        cpu_sample_tokens_per_s(cfg, views, sample)
    t0 = time.perf_counter()
    threads = 1
    for _ in range(args.steps):
        _, _, threads = cpu_sample_tokens_per_s(cfg, views, sample)
    dt = time.perf_counter() - t0
    value = sample * args.steps / dt
    line = dict(
        impl="reference", metric=METRIC, value=value, unit="tokens/s", n_gpus=args.gpus,
        steps=args.steps, warmup=args.warmup, ms_per_step=1e3 * dt / args.steps,
        higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload="C3: S=8192 tokens/rank, H=I=2048, E=64, top-2, CF=1, bf16",
                    note="CPU restatement of the reference math; the reference has no CPU path "
                         "and does not compile for sm_100"),
        cpu_baseline=dict(value=value, unit="tokens/s", cores=threads, kind="port",
                          sample=f"each step: first {sample} of 8192 tokens of one rank through "
                                 "all 64 experts, routing over all 8192 tokens, fp32 accumulation"),
        e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
        gpu_launches=0,
    )
    print(json.dumps(line), flush=True)


def run_cuda(args):
    import torch
    import torch.distributed as dist
    from aristos_b200 import kleos

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    uid = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        idt = torch.zeros(128, dtype=torch.uint8, device=device)
        if rank == 0:
            idt.copy_(torch.frombuffer(bytearray(kleos.get_unique_id()), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        uid = bytes(idt.cpu().numpy().tobytes())

    cfg, workload_desc = workload(args.workload)
    tdt = torch_dtype_of(cfg)
    eb = cfg.elem_bytes
    kleos.set_device(local_rank)
    info = kleos.initialize(cfg, rank, world, uid)
    iP = synth_on_device(cfg, rank, world, device)
    if args.workload == "C4":
        from aristos_b200 import synth
        kleos.set_gate_bias(synth.zipf_gate_bias(cfg, 1.2))  # Zipf(1.2) expert popularity
    oP = torch.zeros(info.output_elems, dtype=tdt, device=device)
    stream = torch.cuda.current_stream().cuda_stream

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------------------------------------------------------- device-resident timing
    barrier()  # ranks finish generating their inputs at different times
    # clocks are sampled from the warm-up on (nvidia-smi needs some tens of milliseconds to
    # deliver its first sample, longer than a short timed region) until the end-to-end pass ends
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    for _ in range(max(args.warmup, 64)):
        kleos.forward_host(iP, oP, stream)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        kleos.forward_host(iP, oP, stream)
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    st = kleos.last_status()
    if st.code:
        raise SystemExit(f"device status: where={st.where} detail={st.detail}")

    # ---------------------------------------------------------------- end to end, host buffers
    act_elems = cfg.S * cfg.H
    host_in = torch.empty(act_elems, dtype=tdt).pin_memory()
    host_in.copy_(iP[:act_elems].cpu())
    host_out = torch.empty(act_elems, dtype=tdt).pin_memory()
    # every step copies its activations from pinned host memory and its layer output back; the
    # library overlaps the copies of neighbouring steps with the forward (three streams)
    for _ in range(max(2, args.warmup // 2)):
        kleos.forward_from_host_async(host_in, iP, oP, host_out)
    kleos.host_sync()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        kleos.forward_from_host_async(host_in, iP, oP, host_out)
    kleos.host_sync()
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    clocks = sampler.stop() if rank == 0 else None

    # ---------------------------------------------------------------- per-phase times, roofline
    kleos.forward_host_bench(iP, oP, skip=2, trials=max(4, min(args.steps, 16)))
    phases = kleos.phase_times()
    # a single-expert layer has no routing: every token of every rank goes through the one expert
    routing = dict(counts=np.array([cfg.S], dtype=np.uint32)) if cfg.dense else kleos.debug_routing(info)
    routed_here = int(np.minimum(routing["counts"], info.EC).sum())  # pairs this rank dispatched
    # pairs this rank's experts processed: under even sharding and random routing this equals
    # the pairs it dispatched to within sampling noise; the all-rank sum is identical
    pairs = torch.tensor([routed_here], dtype=torch.float64, device=device)
    routed_vec = torch.from_numpy(np.minimum(routing["counts"], info.EC).astype(np.float64)).to(device)
    if world > 1:
        dist.all_reduce(pairs)
        dist.all_reduce(routed_vec)
    pairs_per_rank = float(pairs.item()) / world
    # experts of this rank that received at least one row (the weights of the others are never read)
    lo = rank * info.local_experts
    active_experts = int((routed_vec[lo:lo + info.local_experts] > 0).sum().item())
    if cfg.dense:
        pairs_per_rank, active_experts = float(cfg.S), 1
    peaks = load_peaks()
    # dominant kernel: one FFN GEMM launch (GEMM1 and GEMM2 do the same work when H == I).
    # Algorithmic work per launch: 2*R*H*I FLOP; bytes = the weights of this rank's experts that
    # received rows, once, plus the R operand rows in and the R result rows out (R = routed
    # pairs this rank's experts process).
    gemm_flops = 2.0 * pairs_per_rank * cfg.H * cfg.I
    gemm_bytes = (active_experts * cfg.I * cfg.H + pairs_per_rank * (cfg.H + cfg.I)) * float(eb)
    gemm_ms = 0.5 * (phases["gemm1"] + phases["gemm2"])
    gemm_ms = max_over_ranks(gemm_ms)
    tflops = gemm_flops / (gemm_ms * 1e-3) / 1e12
    gbs = gemm_bytes / (gemm_ms * 1e-3) / 1e9
    if cfg.torch_dtype == 0:
        # float layers run on FP32 FMA (as in the reference): nominal 148 SMs x 128 FMA x 1.965 GHz
        peaks = dict(peaks, tflops=74.4, source="nominal fp32 FMA rate (no measured figure)")
    elif cfg.torch_dtype == 1:
        peaks = dict(peaks, tflops=1125.0, source="nominal dense TF32 rate, half the bf16 figure (no measured figure)")
    hbm_bound = gemm_bytes / (peaks["hbm"] * 1e9) > gemm_flops / (peaks["tflops"] * 1e12)
    if hbm_bound:
        roof = dict(bound="hbm", achieved=gbs, peak=peaks["hbm"], unit="GB/s", frac=gbs / peaks["hbm"])
    else:
        roof = dict(bound="tensor", achieved=tflops, peak=peaks["tflops"], unit="TFLOP/s",
                    frac=tflops / peaks["tflops"])
    # DRAM traffic per launch from the ncu capture of the quarter-size layer (155.3 MB, see
    # profiles/), scaled by the units processed (experts x4, routed rows x4); one-GPU C3 only
    roof["traffic"] = 621.2e6 if (world == 1 and args.workload == "C3") else None
    roof.update(kernel={0: "ffn_gemm_simt", 1: "ffn_gemm_tf32"}.get(cfg.torch_dtype, "ffn_gemm_tc2") +
                " (mean of the GEMM1 and GEMM2 launches)",
                peak_source=peaks["source"], tensor_tflops=tflops, hbm_gbs=gbs,
                algorithmic_bytes=gemm_bytes, algorithmic_flops=gemm_flops,
                launch_ms=gemm_ms)
    total_flops = (0.0 if cfg.dense else 2.0 * cfg.S * cfg.H * cfg.E) + 4.0 * cfg.H * cfg.I * pairs_per_rank
    remote_pairs = 0.0 if cfg.dense else pairs_per_rank * (world - 1) / world
    link_bytes = 2.0 * remote_pairs * cfg.H * eb
    t_roof_ms = max(total_flops / (peaks["tflops"] * 1e12), link_bytes / 770e9) * 1e3
    ms_per_step = ms_total / args.steps

    if rank == 0:
        tokens = cfg.S * world
        line = dict(
            metric=METRIC, value=tokens / (ms_per_step * 1e-3), unit="tokens/s", n_gpus=world,
            steps=args.steps, warmup=args.warmup, ms_per_step=ms_per_step,
            higher_is_better=True, scaling="weak", vs_baseline=None, dtype=cfg.dtype_name,
            data="synthetic",
            config=dict(workload=workload_desc,
                        experts_per_rank=info.local_experts,
                        parallelism=f"replicas{world}" if cfg.dense else f"ep{world}",
                        l2="working set per step (weights + cells + activations) exceeds L2"),
            e2e=dict(value=tokens * args.steps / e2e_s, unit="tokens/s",
                     h2d_bytes_per_step=act_elems * eb, d2h_bytes_per_step=act_elems * eb),
            gpu_launches=(2 if cfg.dense else KERNELS_PER_FORWARD) * args.steps,
            clocks=clocks,
            roofline=roof,
            layer_roofline=dict(t_roof_ms=t_roof_ms, frac=t_roof_ms / ms_per_step,
                                flops=total_flops, link_bytes_each_way=link_bytes),
            phases_ms=phases,
            routed_pairs_per_rank=pairs_per_rank,
        )
        if args.cpu_baseline and world == 1:
            views = host_views_from_device(cfg, iP, world)
            sample = min(args.cpu_sample, cfg.S)
            v, dt, threads = cpu_sample_tokens_per_s(cfg, views, sample)
            line["cpu_baseline"] = dict(
                value=v, unit="tokens/s", cores=threads, kind="port",
                sample=(f"first {sample} of {cfg.S} tokens through the FFN, fp32 accumulation, {dt:.1f} s"
                        if cfg.dense else
                        f"first {sample} of {cfg.S} tokens of rank 0 through all {cfg.E} experts "
                        f"(routing over all {cfg.S} tokens), fp32 accumulation, {dt:.1f} s"))
        print(json.dumps(line), flush=True)
    kleos.finalize()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--workload", default="C3",
                    help="C3 (default), C4 (Zipf-imbalanced), C5 (large FFN), C1 / C2 (float), "
                         "C2t (C2 as tf32), C3q / C3r8 (profiling sizes), F3 / F3q (dense FFN, num_experts=1)")
    ap.add_argument("--cpu-sample", type=int, default=0,
                    help="tokens in the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.cpu_sample <= 0:
        # reference arm: a quarter of one rank's batch per step; CUDA arm: the whole batch once
        args.cpu_sample = 2048 if args.impl == "reference" else 8192
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
