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
PARITY_ROWS = 64  # output rows per rank compared with the CPU oracle after the timed regions


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
        return dict(tflops=float(p["bf16_tflops"]), hbm=float(p["hbm_gbs"]),
                    tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    source="measured")
    return dict(tflops=1590.0, hbm=6650.0, tflops_sustained=1400.0, source="fallback")


def bind_to_gpu_numa_node(local_rank: int):
    """Pins this process (and therefore the pinned host buffers it allocates afterwards) to the
    CPUs of the NUMA node the GPU hangs off.  Queries only (nvidia-smi, sysfs); returns what it did."""
    try:
        bdf = subprocess.run(["nvidia-smi", "-i", str(local_rank), "--query-gpu=pci.bus_id",
                              "--format=csv,noheader"], capture_output=True, text=True,
                             timeout=20).stdout.strip().lower()
        if len(bdf.split(":")[0]) == 8:  # 00000000:1b:00.0 -> 0000:1b:00.0
            bdf = bdf[4:]
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return dict(numa_node=None, note="the platform reports no NUMA node for the GPU")
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            return dict(numa_node=node, cpus=len(allowed))
        return dict(numa_node=node, note="none of the node's CPUs is available to this process")
    except Exception as exc:  # no sysfs entry, no permission: run unbound
        return dict(numa_node=None, note=f"not bound: {type(exc).__name__}: {exc}"[:160])


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


def expert_weights_on_device(cfg, e, device):
    """(W1 [I,H], W2 [H,I]) of global expert e as fp32 values rounded to the element type: the same
    draws synth_on_device() makes for the rank that owns e, so any rank can rebuild any expert."""
    import torch
    tdt = torch_dtype_of(cfg)
    gen = torch.Generator(device=device)
    gen.manual_seed(100000 + e)
    ih = cfg.I * cfg.H
    w1 = (torch.randn(ih, generator=gen, device=device) / cfg.H ** 0.5).to(tdt)
    w2 = (torch.randn(ih, generator=gen, device=device) / cfg.I ** 0.5).to(tdt)
    return w1.float().reshape(cfg.I, cfg.H), w2.float().reshape(cfg.H, cfg.I)


def parity_check(cfg, info, kleos, iP, oP, rank, world, device, gate_bias):
    """One more forward, outside every timed region, compared with the CPU oracle: routing of all
    of this rank's tokens bit-exact (top-k sets, counts, slots), PARITY_ROWS seeded output rows
    within the dtype's tolerance.  Returns (routing_exact, worst relative error, rows)."""
    import torch
    from oracle import c_oracle
    from aristos_b200 import synth
    tol = {0: 1e-5, 1: 4e-3, 2: 2e-2, 3: 4e-3}[cfg.torch_dtype]
    kleos.forward_host(iP, oP, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    routing = kleos.debug_routing(info)
    off = cfg.input_offsets(world)
    A = iP[off["A"]:off["Wg"]].float().cpu().numpy().reshape(cfg.S, cfg.H)
    Wg = iP[off["Wg"]:off["W1"]].float().cpu().numpy().reshape(-1, cfg.H)
    rng = np.random.default_rng(1234 + rank)
    rows = np.sort(rng.choice(cfg.S, size=min(PARITY_ROWS, cfg.S), replace=False)).astype(np.int32)
    zero_b1, zero_b2 = np.zeros(cfg.I, np.float32), np.zeros(cfg.H, np.float32)

    def get_expert(e):
        w1, w2 = expert_weights_on_device(cfg, e, device)
        return w1.cpu().numpy(), w2.cpu().numpy(), zero_b1, zero_b2

    c_oracle.use_all_cores()
    ref = c_oracle.moe_forward_rank_lazy(cfg, A, Wg, get_expert, gate_bias=gate_bias, tokens=rows)
    got_sets = np.sort(routing["topk"], axis=1)
    ref_sets = np.sort(ref["topk"], axis=1)
    exact = bool(np.array_equal(got_sets, ref_sets) and np.array_equal(routing["counts"], ref["counts"]))
    if exact:
        m_got = np.full((cfg.S, cfg.E), -2, dtype=np.int64)
        m_ref = np.full((cfg.S, cfg.E), -2, dtype=np.int64)
        np.put_along_axis(m_got, routing["topk"].astype(np.int64), routing["slots"].astype(np.int64), axis=1)
        np.put_along_axis(m_ref, ref["topk"].astype(np.int64), ref["slots"].astype(np.int64), axis=1)
        exact = bool(np.array_equal(m_got, m_ref))
    out = oP[cfg.S * cfg.PX:].float().cpu().numpy().reshape(cfg.S, cfg.H)[rows]
    err = float(np.abs(out - ref["out"]).max() / max(np.abs(ref["out"]).max(), 1e-30))
    return exact, err, int(rows.size), tol


def reference_sample_note(cfg, sample):
    return (f"each step: first {sample} of {cfg.S} tokens of one rank through all {cfg.E} experts, "
            f"routing over all {cfg.S} tokens, fp32 accumulation")


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
    cfg, workload_desc = workload(args.workload)
    torch.manual_seed(0)
    off = cfg.input_offsets(1)
    buf = torch.zeros(off["end"], dtype=torch.float32)
    buf[off["A"]:off["Wg"]] = torch.randn(cfg.S * cfg.H)
    if not cfg.dense:
        buf[off["Wg"]:off["Wg"] + cfg.E * cfg.H] = torch.randn(cfg.E * cfg.H) / cfg.H ** 0.5
    n = cfg.E * cfg.I * cfg.H
    buf[off["W1"]:off["W1"] + n] = torch.randn(n) / cfg.H ** 0.5
    buf[off["W2"]:off["W2"] + n] = torch.randn(n) / cfg.I ** 0.5
    host = synth.round_to_dtype(buf.numpy(), cfg.torch_dtype)
    views = [synth.split_packed(cfg, host, 1)]
    sample = min(args.cpu_sample, cfg.S)
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
        higher_is_better=True, scaling="weak", vs_baseline=None, dtype=cfg.dtype_name, data="synthetic",
        config=dict(workload=workload_desc),
        cpu_baseline=dict(value=value, unit="tokens/s", cores=threads, kind="port",
                          sample=reference_sample_note(cfg, sample),
                          note="CPU restatement of the reference math (oracle/moe_oracle.c); the "
                               "reference has no CPU path and does not compile for sm_100"),
        e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
        gpu_launches=0,
    )
    print(json.dumps(line), flush=True)


def run_cuda(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    import torch
    import torch.distributed as dist
    from aristos_b200 import kleos

    # before any pinned allocation: this rank's threads and host buffers on the GPU's NUMA node
    numa = bind_to_gpu_numa_node(local_rank)
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
    gate_bias = None
    if args.workload == "C4":
        from aristos_b200 import synth
        gate_bias = synth.zipf_gate_bias(cfg, 1.2)  # Zipf(1.2) expert popularity
        kleos.set_gate_bias(gate_bias)
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

    def min_over_ranks(v: float) -> float:
        return -max_over_ranks(-v)

    def timed_forwards(n):
        """n device-resident forwards between two CUDA events on the launching stream, a barrier
        and a synchronize on both sides; milliseconds, max over ranks."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(n):
            kleos.forward_host(iP, oP, stream)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

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
    launches0 = kleos.launch_count()
    ms_total = timed_forwards(args.steps)
    launches = kleos.launch_count() - launches0
    st = kleos.last_status()
    if st.code:
        raise SystemExit(f"device status: where={st.where} detail={st.detail}")
    ms_per_step = ms_total / args.steps

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

    # the two copies alone, all ranks at once, same buffers and two streams: what the host side
    # (PCIe, host memory, the root complexes the GPUs share) delivers without any forward
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    dev_in = torch.empty(act_elems, dtype=tdt, device=device)
    dev_out = torch.empty(act_elems, dtype=tdt, device=device)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        with torch.cuda.stream(s_in):
            dev_in.copy_(host_in, non_blocking=True)
        with torch.cuda.stream(s_out):
            host_out.copy_(dev_out, non_blocking=True)
    barrier()
    copy_s = max_over_ranks(time.perf_counter() - t0)
    copy_gbs = act_elems * eb * args.steps / copy_s / 1e9  # per direction and GPU, both running

    # ---------------------------------------------------------------- sustained figure
    # the same loop for at least a second, clocks sampled over this region alone
    sustained = None
    if args.sustain_s > 0:
        n_long = max(args.steps, int(args.sustain_s * 1e3 / max(ms_per_step, 1e-3)))
        long_sampler = ClockSampler(local_rank)
        if rank == 0:
            long_sampler.start()
            time.sleep(0.1)
        ms_long = timed_forwards(n_long)
        long_clocks = long_sampler.stop() if rank == 0 else None
        sustained = dict(steps=n_long, ms_per_step=ms_long / n_long, clocks=long_clocks)
        st = kleos.last_status()
        if st.code:
            raise SystemExit(f"device status: where={st.where} detail={st.detail}")

    # ---------------------------------------------------------------- per-phase times, roofline
    kleos.forward_host_bench(iP, oP, skip=2, trials=max(4, min(args.steps, 16)))
    phases = kleos.phase_times()
    try:
        timeline = kleos.flow_timeline()
        stalls = kleos.flow_stalls()
    except kleos.KleosError:
        timeline, stalls = None, None  # this layer runs as separate launches
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
    if cfg.torch_dtype == 0:
        # float layers run on FP32 FMA (as in the reference): nominal 148 SMs x 128 FMA x 1.965 GHz
        peaks = dict(peaks, tflops=74.4, tflops_sustained=74.4,
                     source="nominal fp32 FMA rate (no measured figure)")
    elif cfg.torch_dtype == 1:
        peaks = dict(peaks, tflops=1125.0, tflops_sustained=1125.0,
                     source="nominal dense TF32 rate, half the bf16 figure (no measured figure)")
    gate_flops = 0.0 if cfg.dense else 2.0 * cfg.S * cfg.H * cfg.E
    ffn_flops = 4.0 * cfg.H * cfg.I * pairs_per_rank
    total_flops = gate_flops + ffn_flops
    remote_pairs = 0.0 if cfg.dense else pairs_per_rank * (world - 1) / world
    link_bytes = 2.0 * remote_pairs * cfg.H * eb
    t_roof_ms = max(total_flops / (peaks["tflops"] * 1e12), link_bytes / 770e9) * 1e3
    if timeline is not None:
        # Dominant kernel = the persistent kernel (router included when it runs inside): one launch
        # per forward.  Algorithmic work per launch: the gate and FFN FLOPs above; bytes = the
        # weights of this rank's experts that received rows (both GEMMs, once), the activations in,
        # the R routed rows written into the cells, and the layer output out (R = routed pairs).
        k_flops = (gate_flops if launches == args.steps else 0.0) + ffn_flops
        k_bytes = (2.0 * active_experts * cfg.I * cfg.H + cfg.S * cfg.H * 2 + pairs_per_rank * cfg.H) * float(eb)
        k_ms = max_over_ranks(timeline["end"])
        kernel_name = "moe_flow_kernel (router, dispatch, plan, GEMM1, GEMM2, combine: one launch per forward)"
    else:
        # Separate launches: dominant kernel = one FFN GEMM launch (GEMM1 and GEMM2 do the same work
        # when H == I).  Per launch: 2*R*H*I FLOP; bytes = the weights of this rank's experts that
        # received rows, once, plus the R operand rows in and the R result rows out.
        k_flops = 0.5 * ffn_flops
        k_bytes = (active_experts * cfg.I * cfg.H + pairs_per_rank * (cfg.H + cfg.I)) * float(eb)
        k_ms = max_over_ranks(0.5 * (phases["gemm1"] + phases["gemm2"]))
        kernel_name = {0: "ffn_gemm_simt", 1: "ffn_gemm_tf32"}.get(cfg.torch_dtype, "ffn_gemm_tc2") + \
            " (mean of the GEMM1 and GEMM2 launches)"
    tflops = k_flops / (k_ms * 1e-3) / 1e12
    gbs = k_bytes / (k_ms * 1e-3) / 1e9
    hbm_bound = k_bytes / (peaks["hbm"] * 1e9) > k_flops / (peaks["tflops"] * 1e12)
    if hbm_bound:
        roof = dict(bound="hbm", achieved=gbs, peak=peaks["hbm"], unit="GB/s", frac=gbs / peaks["hbm"])
    else:
        roof = dict(bound="tensor", achieved=tflops, peak=peaks["tflops"], unit="TFLOP/s",
                    frac=tflops / peaks["tflops"])
    traffic, traffic_source = committed_traffic(args.workload, world, timeline is not None)
    roof.update(traffic=traffic, traffic_source=traffic_source, kernel=kernel_name,
                peak_source=peaks["source"], tensor_tflops=tflops, hbm_gbs=gbs,
                algorithmic_bytes=k_bytes, algorithmic_flops=k_flops, launch_ms=k_ms,
                # the whole layer against the slower of its FLOPs at the tensor peak and its
                # dispatch + combine bytes at the measured 770 GB/s peer rate
                layer_frac=t_roof_ms / ms_per_step, t_roof_ms=t_roof_ms, layer_flops=total_flops,
                link_bytes_each_way=link_bytes, phases_ms=phases, timeline_ms=timeline, role_waits_ms=stalls,
                routed_pairs_per_rank=pairs_per_rank)
    if sustained is not None:
        t_roof_sus = max(total_flops / (peaks["tflops_sustained"] * 1e12), link_bytes / 770e9) * 1e3
        roof.update(sustained_ms_per_step=sustained["ms_per_step"], sustained_steps=sustained["steps"],
                    sustained_clocks=sustained["clocks"], sustained_peak_tflops=peaks["tflops_sustained"],
                    sustained_layer_frac=t_roof_sus / sustained["ms_per_step"])

    # ---------------------------------------------------------------- parity of THIS run
    parity = None
    if not cfg.dense and args.parity:
        exact, err, nrows, tol = parity_check(cfg, info, kleos, iP, oP, rank, world, device, gate_bias)
        ok = exact and err <= tol
        all_exact = min_over_ranks(1.0 if exact else 0.0) > 0.5
        worst = max_over_ranks(err)
        parity = dict(routing_exact=all_exact, out_rel_err=worst, tolerance=tol,
                      rows_checked=nrows * world, tokens_routed=cfg.S * world,
                      checker="oracle/moe_oracle.c on every rank, after the timed regions")
        if min_over_ranks(1.0 if ok else 0.0) < 0.5:
            if rank == 0:
                print(json.dumps(dict(error="parity check failed", parity=parity)), flush=True)
            kleos.finalize()
            raise SystemExit(3)

    # ---------------------------------------------------------------- the persistent kernel, same run
    # 16-bit routed layers can also run as ONE persistent kernel (KLEOS_FLOW=1, the reference's
    # arrangement); it is measured here on the same buffers so that both arrangements appear in
    # one record: device-timed steps, kernel timeline, and its own parity check.
    persistent = None
    if not cfg.dense and cfg.torch_dtype in (2, 3) and args.persistent and timeline is None:
        kleos.finalize()
        os.environ["KLEOS_FLOW"] = "1"
        uid2 = None
        if world > 1:
            idt = torch.zeros(128, dtype=torch.uint8, device=device)
            if rank == 0:
                idt.copy_(torch.frombuffer(bytearray(kleos.get_unique_id()), dtype=torch.uint8))
            dist.broadcast(idt, 0)
            uid2 = bytes(idt.cpu().numpy().tobytes())
        info = kleos.initialize(cfg, rank, world, uid2)
        if gate_bias is not None:
            kleos.set_gate_bias(gate_bias)
        for _ in range(max(args.warmup, 32)):
            kleos.forward_host(iP, oP, stream)
        l0 = kleos.launch_count()
        p_ms = timed_forwards(args.steps) / args.steps
        p_launches = kleos.launch_count() - l0
        st = kleos.last_status()
        if st.code:
            raise SystemExit(f"persistent kernel, device status: where={st.where} detail={st.detail}")
        kleos.forward_host_bench(iP, oP, skip=2, trials=4)
        try:
            p_timeline, p_waits = kleos.flow_timeline(), kleos.flow_stalls()
        except kleos.KleosError:
            p_timeline, p_waits = None, None  # the layer is beyond the kernel's tables
        p_parity = None
        if args.parity and p_timeline is not None:
            exact, err, nrows, tol = parity_check(cfg, info, kleos, iP, oP, rank, world, device, gate_bias)
            p_parity = dict(routing_exact=min_over_ranks(1.0 if exact else 0.0) > 0.5,
                            out_rel_err=max_over_ranks(err), tolerance=tol, rows_checked=nrows * world)
            if min_over_ranks(1.0 if (exact and err <= tol) else 0.0) < 0.5:
                if rank == 0:
                    print(json.dumps(dict(error="parity check of the persistent kernel failed",
                                          parity=p_parity)), flush=True)
                kleos.finalize()
                raise SystemExit(3)
        if p_timeline is not None:
            persistent = dict(ms_per_step=p_ms, tokens_per_s=cfg.S * world / (p_ms * 1e-3),
                              gpu_launches=p_launches, layer_frac=t_roof_ms / p_ms,
                              timeline_ms=p_timeline, role_waits_ms=p_waits, parity=p_parity,
                              how="KLEOS_FLOW=1: router, dispatch, plan, GEMM1, GEMM2, combine in one launch")
    roof["persistent_kernel"] = persistent

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
                        l2="working set per step (weights + cells + activations) exceeds L2",
                        parity=parity, host_binding=numa),
            e2e=dict(value=tokens * args.steps / e2e_s, unit="tokens/s",
                     h2d_bytes_per_step=act_elems * eb, d2h_bytes_per_step=act_elems * eb,
                     copy_only_gbs=copy_gbs,
                     copy_only_tokens_per_s=tokens * args.steps / copy_s),
            gpu_launches=launches,
            clocks=clocks,
            roofline=roof,
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


def committed_traffic(workload_name, world, persistent):
    """DRAM bytes per launch of the dominant kernel from the committed profiler summary for this
    workload (dram__bytes_read.sum + dram__bytes_write.sum of one capture), or (None, why)."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(path) as f:
            table = json.load(f)
        key = f"{workload_name}:{world}:{'flow' if persistent else 'phases'}"
        if key in table:
            return float(table[key]["bytes_per_launch"]), table[key]["source"]
        return None, f"no capture for {key} in profiles/traffic.json"
    except OSError:
        return None, "profiles/traffic.json not present"


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
    ap.add_argument("--no-parity", dest="parity", action="store_false",
                    help="skip the comparison of this run's results with the CPU oracle")
    ap.add_argument("--no-persistent", dest="persistent", action="store_false",
                    help="skip the second pass that times the persistent kernel (KLEOS_FLOW=1)")
    ap.add_argument("--sustain-s", type=float, default=1.0,
                    help="length of the second, long timed region in seconds (0: none)")
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
