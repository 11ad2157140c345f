"""CPU oracle for the init-time placement planner (device grouping and expert placement).

TEST INFRASTRUCTURE ONLY: a pure-Python restatement of the reference's host-side planner, used
to check the C++ planner of the library; nothing in the product imports it.

PARITY UNPINNED: the reference has no expected outputs for the planner (its ad-hoc driver,
csrc/eval.cuh:142-233, prints the result without checking it) and the planner cannot be built
here (it needs Boost's disjoint sets and CuTe).  This file is pinned against the reference's
source text only; the inputs of that driver are reused as a test case.

Reference lines followed (paths inside the reference project, csrc/include/kleos/...):
  * grouping without gradient all-reduce (inference)   os/decider/decider.cuh:176-268
  * grouping with the all-reduce model (training)      os/decider/decider.cuh:37-174
  * group state, merge test, incremental p2p maximum   os/decider/comps/group.cuh:15-154
  * objective, all-reduce time, merge policy           os/decider/comps/functions.cuh:19-38
  * cost-model arguments                               os/decider/comps/args.cuh:17-88
  * edge ordering (float comparison with tolerance)    os/decider/comps/edge.cuh:18-100
  * expert -> device assignment                        os/decider/decider.cuh:273-329
  * ordered expert set and "closest"                   os/decider/comps/expert.cuh:17-78
  * members of one group                               os/decider/comps/niche.cuh:15-27
  * use at start-up (slots, local experts)             bootstrap.cuh:170-265
  * buffer sizes and stage count from the layer        types.cuh:487-494

Third-party algorithm: the reference keeps the groups in Boost's `disjoint_sets_with_storage`
with `find_with_path_halving` (decider.cuh:29-30; Boost is found on the build host, version not
pinned, CMakeLists.txt).  Union by rank with path-halving finds is restated here from its
published description.

Deliberate choices where the reference leaves the outcome open or undefined:
  * device_to_group holds each device's set representative (the reference copies the raw
    parent array, decider.cuh:168-171,259-262, which is the same once the trees are flat);
  * workers of equal rate keep their rank order (the reference uses an unstable sort,
    decider.cuh:301);
  * where the reference dereferences the end of the expert set (decider.cuh:309-315 when the
    budget exceeds every cost) the last element is taken, which is what that code falls back to;
  * an empty queue of external edges ends the search for the next one (the reference would
    read the top of an empty queue, decider.cuh:113-117);
  * a group objective with no feasible device yet is infinite (the reference would divide by
    an effective world of zero, args.cuh:83-86);
  * a budget that is not a finite int is replaced by the cost still unassigned.
Arithmetic is IEEE single precision in the reference's order of operations.
"""
from __future__ import annotations

import functools
import math
from dataclasses import dataclass, field

import numpy as np

F = np.float32
INF = F(np.inf)
COMM_FREQ = 4          # args.cuh:49
U32 = 0xFFFFFFFF


def float_equal(a, b) -> bool:
    """edge.cuh:18-23: equal within one epsilon of the smaller magnitude."""
    a, b = F(a), F(b)
    small = abs(b) if abs(a) > abs(b) else abs(a)
    return bool(abs(F(a - b)) <= F(small * np.finfo(np.float32).eps))


@dataclass
class Edge:
    node1: int
    node2: int
    weight: np.float32

    def less(self, o: "Edge") -> bool:          # edge.cuh:52-63
        if float_equal(self.weight, o.weight):
            if self.node1 == o.node1:
                return self.node2 < o.node2
            return self.node1 < o.node1
        return bool(self.weight < o.weight)

    def is_limbo(self) -> bool:                  # edge.cuh:88-92
        return self.node1 == self.node2 and float_equal(self.weight, F(0))


def _edge_cmp(a: Edge, b: Edge) -> int:
    return -1 if a.less(b) else (1 if b.less(a) else 0)


class DisjointSet:
    """Union by rank, find with path halving."""

    def __init__(self, n: int):
        self.parent = list(range(n))
        self.rank = [0] * n

    def find(self, v: int) -> int:
        p = self.parent
        parent, grand = p[v], p[p[v]]
        while parent != grand:
            p[v] = grand
            v = grand
            parent, grand = p[v], p[p[v]]
        return parent

    def link(self, i: int, j: int) -> None:
        i, j = self.find(i), self.find(j)
        if i == j:
            return
        if self.rank[i] > self.rank[j]:
            self.parent[j] = i
        else:
            self.parent[i] = j
            if self.rank[i] == self.rank[j]:
                self.rank[j] += 1


@dataclass
class Model:
    """Constants the reference takes from the compiled layer (types.cuh:487-494)."""
    moe_stages: int      # GMS
    p2p_buffer: int      # P2PB, MB
    grad_buffer: int     # GRB, MB


def model_from_config(cfg) -> Model:
    training = 3 if cfg.is_training else 1
    gms = training * (cfg.global_batch // cfg.mini_batch) * (cfg.num_layers // cfg.moe_frequency)
    H = cfg.hidden_size
    pc = H * (cfg.num_layers * (12 * H + 13) + (cfg.vocab_size + H))
    mib = 1024 * 1024
    return Model(moe_stages=gms, p2p_buffer=-(-(cfg.S * H) // mib), grad_buffer=-(-pc // mib))


@dataclass
class ObjArgs:                                   # args.cuh:45-88
    total_cost: int
    effective_world: int
    total_mem: int
    total_rate: np.float32 = F(0)
    all_reduce_time: np.float32 = F(0)
    group_mem: int = 0
    intra_cost: np.float32 = F(0)


def objective(a: ObjArgs, m: Model):             # functions.cuh:19-27
    if a.group_mem < a.total_mem:
        return INF
    if a.effective_world == 0:
        return INF
    gamma = m.moe_stages // a.effective_world
    work = F(F(a.total_cost) / a.total_rate) if a.total_rate != 0 else INF
    inner = F(work + F(F(COMM_FREQ) * a.intra_cost))
    return F(F(F(gamma) * inner) + a.all_reduce_time)


def all_reduce_time(num_groups: int, bottleneck) -> np.float32:   # functions.cuh:29-33
    n = (num_groups - 1) & U32
    return F(2.0 * float(n) * float(bottleneck))   # computed in double, returned as float


def bottleneck(alpha, beta, buf: int, n: int) -> np.float32:      # args.cuh:33-42
    n &= U32
    if n == 0:
        return F(0)
    return F(F(alpha) + F(F(beta) * F(F(buf) / F(n))))


def p2p_time(alpha, beta, size) -> np.float32:                    # args.cuh:70-74
    return F(F(alpha) + F(F(beta) * F(size)))


class Group:                                     # group.cuh:15-154
    def __init__(self, gid, mem, rate, world, args: ObjArgs, dp, m: Model):
        self.m = m
        self.visited = {}
        self.p2p = [(F(a), F(b)) for a, b in dp]
        self.nodes = {gid}
        self.id = gid
        self.mem = mem
        self.rate = F(rate)
        self.art = F(0)
        self.args = args
        self.world = world
        self.cached_obj = F(0)
        self.cached_art = F(0)
        self.cur = objective(self.args, m)

    def construct(self, art, effective):
        self.args.group_mem = self.mem
        self.args.effective_world = effective
        self.args.all_reduce_time = self.art = F(art)
        self.args.total_rate = self.rate
        self.cur = objective(self.args, self.m)

    def num_nodes(self):
        return len(self.nodes)

    def current(self):
        return F(F(self.cur - self.art) + self.cached_art)

    def _eval_p2p(self, nb: "Group", n: int):
        size = F(F(self.m.p2p_buffer) / F(n))
        best = F(0)
        for node in list(self.nodes) + list(nb.nodes):
            t = p2p_time(F(self.p2p[node][0] + nb.p2p[node][0]),
                         F(self.p2p[node][1] + nb.p2p[node][1]), size)
            best = max(best, t)
        return best

    def should_merge(self, nb: "Group", art, effective_w) -> bool:
        if nb.id in self.visited:
            mine, theirs = self.visited[nb.id]
            if mine == self.num_nodes() and theirs == nb.num_nodes():
                return False
        self.visited.setdefault(nb.id, (self.num_nodes(), nb.num_nodes()))
        a = self.args
        a.effective_world = effective_w
        saved = a.effective_world
        if self.mem + nb.mem >= a.total_mem:
            if a.effective_world < self.world and self.mem < a.total_mem:
                a.effective_world += self.num_nodes()
            if a.effective_world < self.world and nb.mem < a.total_mem:
                a.effective_world += self.num_nodes()      # own size, as the reference has it
        a.total_rate = F(self.rate + nb.rate)
        a.group_mem = self.mem + nb.mem
        self.cached_art = nb.cached_art = F(art)
        a.intra_cost = self._eval_p2p(nb, self.num_nodes() + nb.num_nodes())
        a.all_reduce_time = self.cached_art
        self.cached_obj = nb.cached_obj = objective(a, self.m)
        a.effective_world = saved
        o1, o2 = self.current(), nb.current()
        if math.isinf(o1) and math.isinf(o2):              # functions.cuh:35-38
            return True
        return bool(self.cached_obj <= max(o1, o2))

    def subsume(self, nb: "Group"):
        self.p2p = [(F(a + c), F(b + d)) for (a, b), (c, d) in zip(self.p2p, nb.p2p)]
        self.nodes |= nb.nodes
        self.cur = self.cached_obj
        self.mem += nb.mem
        self.rate = F(self.rate + nb.rate)
        self.art = self.cached_art


def _setup(alpha, beta, rate, mem, total_cost, total_mem, m: Model):
    world = len(rate)
    infeasible = {i for i in range(world) if mem[i] < total_mem}
    effective = world - len(infeasible)
    groups = DisjointSet(world)
    cand, info = [], {}
    for i in range(world):
        dp = [(F(0), F(0))] * world
        dp = list(dp)
        for j in range(world):
            if i != j:
                cand.append(Edge(i, j, p2p_time(alpha[i][j], beta[i][j], F(m.p2p_buffer))))
                dp[j] = (F(alpha[j][i]), F(beta[j][i]))        # inverted edge
        info[i] = Group(i, int(mem[i]), rate[i], world, ObjArgs(total_cost, effective, total_mem), dp, m)
    return world, infeasible, effective, groups, cand, info


def _merge(groups, info, infeasible, effective, g1, g2, satisfies):
    groups.link(g1, g2)
    parent, child = g1, g2
    if g1 != groups.find(g1):
        parent, child = g2, g1
    if satisfies:
        if parent in infeasible:
            infeasible.discard(parent)
            effective += info[parent].num_nodes()
        if child in infeasible:
            infeasible.discard(child)
            effective += info[child].num_nodes()
    else:
        infeasible.discard(child)
    info[parent].subsume(info[child])
    del info[child]
    return effective


def decide_inference(alpha, beta, rate, mem, total_cost, total_mem, m: Model):
    """decider.cuh:176-268.  Returns (device_to_group, feasible)."""
    world, infeasible, effective, groups, cand, info = _setup(alpha, beta, rate, mem, total_cost, total_mem, m)
    cand.sort(key=functools.cmp_to_key(_edge_cmp))
    for c in cand:
        g1, g2 = groups.find(c.node1), groups.find(c.node2)
        if g1 == g2:
            continue
        satisfies = info[g1].mem + info[g2].mem >= total_mem
        if info[g1].should_merge(info[g2], F(0), effective):
            effective = _merge(groups, info, infeasible, effective, g1, g2, satisfies)
    return [groups.find(i) for i in range(world)], len(infeasible) == 0


def decide_training(alpha, beta, rate, mem, total_cost, total_mem, m: Model):
    """decider.cuh:37-174.  Returns (device_to_group, feasible)."""
    world, infeasible, effective, groups, cand, info = _setup(alpha, beta, rate, mem, total_cost, total_mem, m)
    ext = [Edge(i, j, bottleneck(alpha[i][j], beta[i][j], m.grad_buffer, 2))
           for i in range(world) for j in range(world) if i != j]
    key = functools.cmp_to_key(_edge_cmp)

    def top():
        return max(ext, key=key)

    def pop():
        ext.remove(top())

    if world < 2:
        return [0] * world, len(infeasible) == 0
    e = top()
    ar_alpha, ar_beta = F(alpha[e.node1][e.node2]), F(beta[e.node1][e.node2])
    art = all_reduce_time(effective, bottleneck(ar_alpha, ar_beta, m.grad_buffer, effective))
    for g in info.values():
        g.construct(art, effective)

    def same_pair(a0, a1, b0, b1):                      # niche.cuh:29-36
        return (a0 == b0 and a1 == b1) or (a0 == b1 and a1 == b0)

    limbo = Edge(0, 0, F(0))
    cand.sort(key=key)
    for c in cand:
        g1, g2 = groups.find(c.node1), groups.find(c.node2)
        if g1 == g2:
            continue
        e = top()
        x1, x2 = groups.find(e.node1), groups.find(e.node2)
        if len(info) > 2 and same_pair(x1, x2, g1, g2):
            limbo = e
        while len(info) > 2 and (groups.find(e.node1) == groups.find(e.node2)
                                 or same_pair(groups.find(e.node1), groups.find(e.node2), g1, g2)):
            pop()
            if not ext:
                break
            e = top()
        satisfies = info[g1].mem + info[g2].mem >= total_mem
        num_groups = (len(info) - len(infeasible)) & U32
        if g1 in infeasible and g2 in infeasible:
            if satisfies:
                num_groups = (num_groups + 1) & U32
        elif g1 not in infeasible and g2 not in infeasible:
            num_groups = (num_groups - 1) & U32
        ar_alpha, ar_beta = F(alpha[e.node1][e.node2]), F(beta[e.node1][e.node2])
        art_now = all_reduce_time(num_groups, bottleneck(ar_alpha, ar_beta, m.grad_buffer, num_groups))
        if info[g1].should_merge(info[g2], art_now, effective):
            limbo = Edge(0, 0, F(0))
            effective = _merge(groups, info, infeasible, effective, g1, g2, satisfies)
        if not limbo.is_limbo():
            ext.append(limbo)
    return [groups.find(i) for i in range(world)], len(infeasible) == 0


def members(device_to_group, gid):               # niche.cuh:15-27
    return [i for i, g in enumerate(device_to_group) if g == gid]


def assign(rates, mems, costs):
    """decider.cuh:273-329.  rates/mems per group member (index = rank inside the group),
    costs per expert.  Returns expert -> member index."""
    world, n = len(rates), len(costs)
    t = sorted(range(n), key=lambda e: (costs[e], -e))           # cost ascending, id descending
    total_cost, total_mem = sum(costs), n
    req = -(-total_mem // world)
    well = all(mems[i] >= req for i in range(world))
    total_rate = F(0)
    for r in rates:
        total_rate = F(total_rate + F(r))
    order = sorted(range(world), key=lambda i: -float(F(rates[i])))   # stable: ties keep rank order
    w_rate = [F(rates[i]) for i in order]
    w_mem = [int(mems[i]) for i in order]
    out = [0] * n
    if sum(w_mem) < n:
        raise ValueError("the group cannot hold every expert")
    j = 0
    while t:
        with np.errstate(all="ignore"):
            raw = F(F(w_rate[j] * F(total_cost)) / total_rate)
        b = math.floor(float(raw)) if math.isfinite(float(raw)) and abs(float(raw)) < 2 ** 31 else total_cost
        budget = max(int(b), 1)
        allocated = budget
        while budget > 0 and w_mem[j] > 0 and t:
            want = budget & 0xFFFF                       # the sentinel's cost is 16 bits wide
            # first element not ordered before (want, id 0)
            lower = next((k for k, e in enumerate(t)
                          if not (costs[e] < want or (costs[e] == want and e > 0))), len(t))
            best = t[-1]
            if lower < len(t):
                if costs[t[lower]] == budget or lower == 0:
                    best = t[lower]
                else:
                    upper = next((k for k, e in enumerate(t) if costs[e] > want), len(t))
                    if upper < len(t):
                        lo, hi = t[lower], t[upper]
                        lm = abs(want - costs[lo]) & 0xFFFF
                        rm = abs(want - costs[hi]) & 0xFFFF
                        best = lo if lm <= rm else hi
                    else:
                        best = t[lower]
            out[best] = order[j]
            t.remove(best)
            w_mem[j] -= 1
            budget -= costs[best]
        total_cost -= allocated - budget
        if w_mem[j] == 0 or well:
            total_rate = F(total_rate - w_rate[j])
        j = (j + 1) % world
    return out


def plan(alpha, beta, rate, mem, num_experts, expert_cost, m: Model, training: bool, rank: int):
    """bootstrap.cuh:170-265 for one rank: groups, this rank's group, experts of the group's
    members, local expert count and the slot count (largest count on any device of any group)."""
    total_cost = num_experts * expert_cost
    decide = decide_training if training else decide_inference
    d2g, feasible = decide(alpha, beta, rate, mem, total_cost, num_experts, m)
    if not feasible:
        return dict(feasible=False, device_to_group=d2g)
    mine = members(d2g, d2g[rank])
    costs = [expert_cost] * num_experts
    e2m = assign([rate[i] for i in mine], [mem[i] for i in mine], costs)
    tally = [0] * len(mine)
    for e in e2m:
        tally[e] += 1
    slots, widest = max(tally), len(mine)
    for gid in sorted(set(d2g)):
        if gid == d2g[rank]:
            continue
        other = members(d2g, gid)
        widest = max(widest, len(other))
        oe = assign([rate[i] for i in other], [mem[i] for i in other], costs)
        ot = [0] * len(other)
        for e in oe:
            ot[e] += 1
        slots = max(slots, max(ot))
    return dict(feasible=True, device_to_group=d2g, group_ranks=mine, group_rank=mine.index(rank),
                expert_to_member=e2m, local_experts=tally[mine.index(rank)], expert_slots=slots,
                widest_group=widest)
