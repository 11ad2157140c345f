"""CPU oracle (NumPy) for the distributed MoE layer forward pass.

TEST INFRASTRUCTURE ONLY.  This is a restatement of the reference's kernel math used to check
the CUDA path; nothing in the product imports it.  Only ``tests/``, the smoke check and the
CPU-baseline leg of the benchmark may call it.

PARITY UNPINNED: the reference ships no golden vectors, no known-answer test and no CPU
implementation of this path, and it cannot be compiled for or run on sm_100, so this oracle
is pinned only against its C twin (``moe_oracle.c``) and against the reference's source text.

Reference lines followed (paths inside the reference project):
  * packed buffers                csrc/include/kleos/moe/moe.cuh:92-132
  * softmax over the E real experts   moe/gate.cuh:556-584 (padding excluded, :550)
  * top-k, strict '>' over ascending ids, so ties go to the lowest id   moe/gate.cuh:654-670
  * sum of the k winning probabilities (mCw)   moe/gate.cuh:669
  * slot per (expert, token), kept iff slot < EC   moe/gate.cuh:689-718
  * capacity EC                   types.cuh:498-500
  * routed = min(count, EC)       os/packet.cuh:112-113
  * dispatch copies unscaled rows os/packet.cuh:147-166
  * FFN tile: act(x W1^T + b1) rounded to the element type, then (y1 W2^T + b2) rounded
                                  os/processor/processor.cuh:350-489, gemm.cuh:23-31,
                                  activations types.cuh:143-159
  * combine: out[t] += Element(y2 / mCw) * Element(prob[t,e])   processor.cuh:110-168
  * expert -> rank map (contiguous, even)   bootstrap.cuh:36-52
  * single-expert (dense) layer   moe/moe.cuh:174-177, moe/fffn.cuh:31-167
  * training-mode gate statistics and loss   moe/gate.cuh:607-635,698-705,763-773

Deliberate choices where the reference leaves the outcome open:
  * slot order inside an expert is ascending token index (the reference orders by
    atomicAdd arrival, gate.cuh:698-700, so this is one of its possible outcomes);
  * selection is made on the fp64 logits (softmax is monotone), exact ties to the lowest id;
  * logits and FFN sums are accumulated in fp64 from the dtype-rounded inputs.
"""
from __future__ import annotations

import math

import numpy as np

DROPPED = -1


def _round_bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) & 0xFFFF0000).astype(np.uint32).view(np.float32)


def _round_tf32(x: np.ndarray) -> np.ndarray:
    """fp32 word with a 10-bit mantissa, round to nearest even (reference element type
    cute::tfloat32_t, types.cuh:128-131)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u + np.uint32(0xFFF) + ((u >> np.uint32(13)) & np.uint32(1))) & np.uint32(0xFFFFE000)).astype(np.uint32)
    finite = (u & np.uint32(0x7F800000)) != np.uint32(0x7F800000)
    return np.where(finite, r, u).astype(np.uint32).view(np.float32)


def round_elem(x: np.ndarray, torch_dtype: int) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    if torch_dtype == 1:
        return _round_tf32(x)
    if torch_dtype == 2:
        return _round_bf16(x)
    if torch_dtype == 3:
        return x.astype(np.float16).astype(np.float32)
    return x


def _gelu(x: np.ndarray) -> np.ndarray:
    erf = np.vectorize(math.erf, otypes=[np.float64])
    return 0.5 * x * (1.0 + erf(x / math.sqrt(2.0)))


def route(cfg, a: np.ndarray, wg: np.ndarray, gate_bias=None) -> dict:
    """Routing of one source rank.  a: [S,H], wg: [>=E,H] (dtype-rounded fp32)."""
    S, E, K = cfg.S, cfg.E, cfg.K
    logits = a.astype(np.float64) @ wg[:E].astype(np.float64).T
    if gate_bias is not None:
        logits = logits + np.asarray(gate_bias, dtype=np.float64)[None, :]
    # fp32 softmax over the E real experts
    l32 = logits.astype(np.float32)
    m = l32.max(axis=1, keepdims=True)
    ex = np.exp(l32 - m, dtype=np.float32)
    probs = ex / ex.sum(axis=1, keepdims=True, dtype=np.float32)
    # top-k on logits, ties to the lowest expert id (stable sort of descending values)
    order = np.argsort(-logits, axis=1, kind="stable")
    topk = np.ascontiguousarray(order[:, :K]).astype(np.int32)
    srt = np.take_along_axis(logits, order, axis=1)
    margin = float((srt[:, K - 1] - srt[:, K]).min()) if K < E else float("inf")
    mcw = np.take_along_axis(probs, topk, axis=1).sum(axis=1, dtype=np.float32)
    # slots in ascending token order per expert
    sel = np.zeros((S, E), dtype=np.int64)
    np.put_along_axis(sel, topk.astype(np.int64), 1, axis=1)
    pos = np.cumsum(sel, axis=0) - 1
    counts = sel.sum(axis=0).astype(np.uint32)
    slots = np.take_along_axis(pos, topk.astype(np.int64), axis=1).astype(np.int32)
    slots[slots >= cfg.EC] = DROPPED
    routed = np.minimum(counts, cfg.EC).astype(np.uint32)
    probs_pad = np.zeros((S, cfg.PX), dtype=np.float32)
    probs_pad[:, :E] = round_elem(probs, cfg.torch_dtype)
    # training-mode statistics (moe/gate.cuh:607-635 mean probability per expert, :698-705 mean
    # unclamped selection count, :763-773 loss = sum_e mean_prob * mean_count / E)
    mean_prob = probs.astype(np.float64).mean(axis=0)
    mean_count = counts.astype(np.float64) / S
    gate_loss = float((mean_prob * mean_count).sum() / E)
    return dict(logits=logits, probs_f32=probs, probs=probs_pad, topk=topk, mcw=mcw,
                slots=slots, counts=counts, routed=routed, margin=margin,
                mean_prob=mean_prob, mean_count=mean_count, gate_loss=gate_loss)


def route_reference_rule(cfg, a: np.ndarray, wg: np.ndarray, gate_bias=None) -> dict:
    """The reference gate's selection rule taken literally, as a second opinion on ``route``:
    fp32 logits (fp32 accumulation, BLAS order), fp32 softmax with expf over the E real experts
    (moe/gate.cuh:574-584), then k rounds of arg-max on the PROBABILITIES with strict '>' over
    ascending ids and the winner masked out (:654-670).  Returns the top-k ids in selection order
    and the smallest gap, over all tokens, between the k-th and (k+1)-th largest probability: where
    that gap is far above fp32 rounding, selecting on fp64 logits (``route``) must pick the same
    sets."""
    S, E, K = cfg.S, cfg.E, cfg.K
    l32 = a.astype(np.float32) @ wg[:E].astype(np.float32).T
    if gate_bias is not None:
        l32 = l32 + np.asarray(gate_bias, dtype=np.float32)[None, :]
    m = l32.max(axis=1, keepdims=True)
    ex = np.exp(l32 - m, dtype=np.float32)
    probs = (ex / ex.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)
    work = probs.copy()
    topk = np.zeros((S, K), dtype=np.int32)
    rows = np.arange(S)
    for j in range(K):
        best = np.argmax(work, axis=1)  # first maximum = lowest id among equals, as strict '>' does
        topk[:, j] = best
        work[rows, best] = -1.0
    srt = -np.sort(-probs, axis=1)
    gap = float((srt[:, K - 1] - srt[:, K]).min()) if K < E else float("inf")
    rel_gap = float(((srt[:, K - 1] - srt[:, K]) / srt[:, K - 1]).min()) if K < E else float("inf")
    return dict(topk=topk, probs_f32=probs, min_prob_gap=gap, min_rel_prob_gap=rel_gap)


def expert_ffn(cfg, x: np.ndarray, w1, w2, b1, b2) -> np.ndarray:
    """y2 rows of one expert for token rows x (all dtype-rounded fp32)."""
    z = x.astype(np.float64) @ w1.astype(np.float64).T + b1.astype(np.float64)[None, :]
    z = np.maximum(z, 0.0) if cfg.hidden_act == 0 else _gelu(z)
    y1 = round_elem(z.astype(np.float32), cfg.torch_dtype)
    y2 = y1.astype(np.float64) @ w2.astype(np.float64).T + b2.astype(np.float64)[None, :]
    return round_elem(y2.astype(np.float32), cfg.torch_dtype)


def dense_ffn(cfg, inp: dict, token_subset=None) -> np.ndarray:
    """Single-expert layer: the plain FFN over one rank's tokens, no gate and no scaling
    (the reference runs its dense kernel when E == 1, moe/moe.cuh:174-177; arithmetic
    moe/fffn.cuh:31-167: act(A W1^T + b1) rounded to the element type, then W2^T + b2 rounded)."""
    a = inp["A"] if token_subset is None else inp["A"][np.asarray(token_subset)]
    return expert_ffn(cfg, a, inp["W1"][0], inp["W2"][0], inp["b1"][0], inp["b2"][0])


def moe_forward(cfg, world: int, inputs: list, gate_bias=None, token_subset=None) -> list:
    """Whole layer over all ranks.

    inputs[r] is a dict with A [S,H], Wg [PX,H], W1 [nLx,I,H], W2 [nLx,H,I], b1, b2 of rank r
    (fp32 arrays already rounded to the element type).  Returns one dict per rank with
    probs [S,PX], out [S,H], topk, slots, counts, routed, mcw, margin.

    token_subset: optional list of token indices; the FFN and combine are evaluated only for
    those tokens of every rank (routing is always complete), and ``out`` then has one row per
    listed token.
    """
    nlx = cfg.E // world
    dt = cfg.torch_dtype
    results = []
    for r in range(world):
        rt = route(cfg, inputs[r]["A"], inputs[r]["Wg"], gate_bias)
        toks = np.arange(cfg.S) if token_subset is None else np.asarray(token_subset)
        out = np.zeros((len(toks), cfg.H), dtype=np.float32)
        for e in range(cfg.E):
            owner, le = divmod(e, nlx)
            hit = (rt["topk"][toks] == e) & (rt["slots"][toks] != DROPPED)
            rows = np.nonzero(hit.any(axis=1))[0]
            if rows.size == 0:
                continue
            t = toks[rows]
            own = inputs[owner]
            y2 = expert_ffn(cfg, inputs[r]["A"][t], own["W1"][le], own["W2"][le],
                            own["b1"][le], own["b2"][le])
            if cfg.K > 1:
                v = round_elem(y2 / rt["mcw"][t][:, None], dt)
                w = round_elem(rt["probs"][t, e][:, None] * v, dt)
                out[rows] = round_elem(out[rows] + w, dt)
            else:
                out[rows] = y2  # top-1: plain copy, no scaling (processor.cuh:170-204)
        rt["out"] = out
        results.append(rt)
    return results
