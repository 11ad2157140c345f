// Init-time placement planner (host only): which devices form an expert-parallel group, and
// which device of a group holds which expert.
//
// The reference runs this once at start-up from a measured latency / inverse-bandwidth matrix,
// per-device throughput and memory (bootstrap.cuh:170-265): a greedy, Kruskal-style merge of
// devices into groups under a cost model (os/decider/decider.cuh:37-268, comps/group.cuh,
// comps/functions.cuh, comps/args.cuh), then a throughput-proportional assignment of experts
// to the devices of a group (decider.cuh:273-329).  On one NVSwitch node with identical GPUs
// the result is a single group with the experts split evenly and contiguously, which is the
// placement the data path of this library implements; the planner is provided so that a host
// can check that, or plan for a machine where it does not hold.
//
// Arithmetic is single precision in the reference's order of operations, so that the decisions
// agree with it.  Where the reference's behaviour is undefined the choices are: ties between
// workers of equal rate keep rank order (stable sort); looking past the end of the expert set
// takes its last element; an exhausted queue of external edges ends the search; an objective
// with no feasible device is infinite; a budget that is not a finite int becomes the cost that
// is still unassigned.  Groups are kept in a union-by-rank forest with path-halving finds, the
// structure the reference takes from Boost (decider.cuh:29-30).
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <map>
#include <set>
#include <string>
#include <vector>

namespace kleos {
namespace placement {

struct Model {
    uint32_t moe_stages;   // types.cuh:487-488
    uint32_t p2p_buffer;   // MB, types.cuh:494
    uint32_t grad_buffer;  // MB, types.cuh:493
};

struct Inputs {
    int world = 0;
    std::vector<float> alpha, beta;  // [world*world], entry (i, j) = link i -> j; ms and ms/MB
    std::vector<float> rate;         // [world]
    std::vector<uint32_t> mem;       // [world] experts that fit on the device
    uint32_t num_experts = 0, expert_cost = 1;
    bool training = false;
    Model model{};
};

struct Plan {
    bool feasible = false;
    std::vector<uint32_t> device_to_group;   // [world] representative device of each device's group
    std::vector<uint32_t> group_ranks;       // devices of the asking rank's group, ascending
    uint32_t group_rank = 0;                 // position of the asking rank inside its group
    std::vector<uint32_t> expert_to_member;  // [E] index into group_ranks
    uint32_t local_experts = 0, expert_slots = 0, widest_group = 0;
};

constexpr float kInf = std::numeric_limits<float>::infinity();
constexpr uint32_t kCommFreq = 4;  // comps/args.cuh:49

inline bool float_equal(float a, float b) {  // comps/edge.cuh:18-23
    const float small = std::fabs(a) > std::fabs(b) ? std::fabs(b) : std::fabs(a);
    return std::fabs(a - b) <= small * std::numeric_limits<float>::epsilon();
}

struct Edge {
    uint32_t a = 0, b = 0;
    float w = 0.f;
    bool before(const Edge& o) const {  // comps/edge.cuh:52-63
        if (float_equal(w, o.w)) return a == o.a ? b < o.b : a < o.a;
        return w < o.w;
    }
    bool null_edge() const { return a == b && float_equal(w, 0.f); }
};

class Forest {
public:
    explicit Forest(int n) : parent_(n), rank_(n, 0) {
        for (int i = 0; i < n; ++i) parent_[i] = i;
    }
    uint32_t find(uint32_t v) {
        uint32_t p = parent_[v], g = parent_[p];
        while (p != g) {
            parent_[v] = g;
            v = g;
            p = parent_[v];
            g = parent_[p];
        }
        return p;
    }
    void link(uint32_t i, uint32_t j) {
        i = find(i);
        j = find(j);
        if (i == j) return;
        if (rank_[i] > rank_[j]) {
            parent_[j] = i;
        } else {
            parent_[i] = j;
            if (rank_[i] == rank_[j]) ++rank_[j];
        }
    }

private:
    std::vector<uint32_t> parent_;
    std::vector<int> rank_;
};

struct Cost {  // comps/args.cuh:45-88
    uint32_t total_cost = 0, effective_world = 0, total_mem = 0, group_mem = 0;
    float total_rate = 0.f, all_reduce = 0.f, intra = 0.f;
};

inline float objective(const Cost& c, const Model& m) {  // comps/functions.cuh:19-27
    if (c.group_mem < c.total_mem || c.effective_world == 0) return kInf;
    const uint32_t gamma = m.moe_stages / c.effective_world;
    const float work = c.total_rate != 0.f ? static_cast<float>(c.total_cost) / c.total_rate : kInf;
    const float inner = work + static_cast<float>(kCommFreq) * c.intra;
    return static_cast<float>(gamma) * inner + c.all_reduce;
}
inline float bottleneck(float alpha, float beta, uint32_t buf, uint32_t n) {  // comps/args.cuh:33-42
    return n == 0 ? 0.f : alpha + beta * (static_cast<float>(buf) / static_cast<float>(n));
}
inline float all_reduce_time(uint32_t groups, float bottleneck_time) {  // comps/functions.cuh:29-33
    return static_cast<float>(2.0 * static_cast<double>(groups - 1u) * static_cast<double>(bottleneck_time));
}
inline float p2p_time(float alpha, float beta, float size) { return alpha + beta * size; }

struct Group {  // comps/group.cuh:15-154
    std::map<uint32_t, std::pair<uint32_t, uint32_t>> seen;
    std::vector<float> pa, pb;  // summed inverted-edge alpha / beta towards every device
    std::set<uint32_t> nodes;
    uint32_t id = 0, mem = 0, world = 0;
    float rate = 0.f, art = 0.f, cur = 0.f, cached_obj = 0.f, cached_art = 0.f;
    Cost cost;

    float current() const { return (cur - art) + cached_art; }
    uint32_t size() const { return static_cast<uint32_t>(nodes.size()); }

    void construct(float a, uint32_t effective, const Model& m) {
        cost.group_mem = mem;
        cost.effective_world = effective;
        cost.all_reduce = art = a;
        cost.total_rate = rate;
        cur = objective(cost, m);
    }
    float pair_p2p(const Group& nb, uint32_t n, const Model& m) const {
        const float size = static_cast<float>(m.p2p_buffer) / static_cast<float>(n);
        float best = 0.f;
        for (uint32_t v : nodes) best = std::max(best, p2p_time(pa[v] + nb.pa[v], pb[v] + nb.pb[v], size));
        for (uint32_t v : nb.nodes) best = std::max(best, p2p_time(pa[v] + nb.pa[v], pb[v] + nb.pb[v], size));
        return best;
    }
    bool should_merge(Group& nb, float a, uint32_t effective, const Model& m) {
        auto it = seen.find(nb.id);
        if (it != seen.end() && it->second.first == size() && it->second.second == nb.size()) return false;
        seen.emplace(nb.id, std::make_pair(size(), nb.size()));  // keeps an older entry
        cost.effective_world = effective;
        const uint32_t saved = cost.effective_world;
        if (mem + nb.mem >= cost.total_mem) {
            if (cost.effective_world < world && mem < cost.total_mem) cost.effective_world += size();
            // own size again, as in the reference (group.cuh:66-68)
            if (cost.effective_world < world && nb.mem < cost.total_mem) cost.effective_world += size();
        }
        cost.total_rate = rate + nb.rate;
        cost.group_mem = mem + nb.mem;
        cached_art = nb.cached_art = a;
        cost.intra = pair_p2p(nb, size() + nb.size(), m);
        cost.all_reduce = cached_art;
        cached_obj = nb.cached_obj = objective(cost, m);
        cost.effective_world = saved;
        const float o1 = current(), o2 = nb.current();
        if (std::isinf(o1) && std::isinf(o2)) return true;  // comps/functions.cuh:35-38
        return cached_obj <= std::max(o1, o2);
    }
    void subsume(const Group& nb) {
        for (size_t i = 0; i < pa.size(); ++i) {
            pa[i] += nb.pa[i];
            pb[i] += nb.pb[i];
        }
        nodes.insert(nb.nodes.begin(), nb.nodes.end());
        cur = cached_obj;
        mem += nb.mem;
        rate += nb.rate;
        art = cached_art;
    }
};

// Device grouping; both job types (decider.cuh:37-174 training, :176-268 inference).
inline bool decide(const Inputs& in, std::vector<uint32_t>* device_to_group) {
    const int W = in.world;
    const uint32_t total_cost = in.num_experts * in.expert_cost, total_mem = in.num_experts;
    const Model& m = in.model;
    auto A = [&](uint32_t i, uint32_t j) { return in.alpha[(size_t)i * W + j]; };
    auto B = [&](uint32_t i, uint32_t j) { return in.beta[(size_t)i * W + j]; };
    std::set<uint32_t> infeasible;
    for (int i = 0; i < W; ++i)
        if (in.mem[i] < total_mem) infeasible.insert(i);
    uint32_t effective = W - static_cast<uint32_t>(infeasible.size());
    Forest forest(W);
    std::vector<Edge> cand, ext;
    std::map<uint32_t, Group> info;
    for (int i = 0; i < W; ++i) {
        Group g;
        g.id = i;
        g.mem = in.mem[i];
        g.rate = in.rate[i];
        g.world = W;
        g.nodes.insert(i);
        g.pa.assign(W, 0.f);
        g.pb.assign(W, 0.f);
        for (int j = 0; j < W; ++j) {
            if (i == j) continue;
            cand.push_back(Edge{(uint32_t)i, (uint32_t)j, p2p_time(A(i, j), B(i, j), static_cast<float>(m.p2p_buffer))});
            if (in.training) ext.push_back(Edge{(uint32_t)i, (uint32_t)j, bottleneck(A(i, j), B(i, j), m.grad_buffer, 2)});
            g.pa[j] = A(j, i);  // inverted edge
            g.pb[j] = B(j, i);
        }
        g.cost.total_cost = total_cost;
        g.cost.effective_world = effective;
        g.cost.total_mem = total_mem;
        g.cur = objective(g.cost, m);
        info.emplace(i, std::move(g));
    }
    auto top = [&]() {
        size_t best = 0;
        for (size_t k = 1; k < ext.size(); ++k)
            if (ext[best].before(ext[k])) best = k;
        return best;
    };
    auto same_pair = [](uint32_t a0, uint32_t a1, uint32_t b0, uint32_t b1) {  // comps/niche.cuh:29-36
        return (a0 == b0 && a1 == b1) || (a0 == b1 && a1 == b0);
    };
    auto merge = [&](uint32_t g1, uint32_t g2, bool satisfies) {
        forest.link(g1, g2);
        uint32_t parent = g1, child = g2;
        if (g1 != forest.find(g1)) std::swap(parent, child);
        if (satisfies) {
            if (infeasible.erase(parent)) effective += info.at(parent).size();
            if (infeasible.erase(child)) effective += info.at(child).size();
        } else {
            infeasible.erase(child);
        }
        info.at(parent).subsume(info.at(child));
        info.erase(child);
    };
    std::stable_sort(cand.begin(), cand.end(), [](const Edge& x, const Edge& y) { return x.before(y); });

    if (!in.training) {
        for (const Edge& c : cand) {
            const uint32_t g1 = forest.find(c.a), g2 = forest.find(c.b);
            if (g1 == g2) continue;
            const bool satisfies = info.at(g1).mem + info.at(g2).mem >= total_mem;
            if (info.at(g1).should_merge(info.at(g2), 0.f, effective, m)) merge(g1, g2, satisfies);
        }
    } else if (W >= 2) {
        Edge e = ext[top()];
        const float art0 = all_reduce_time(effective, bottleneck(A(e.a, e.b), B(e.a, e.b), m.grad_buffer, effective));
        for (auto& kv : info) kv.second.construct(art0, effective, m);
        Edge limbo{};
        for (const Edge& c : cand) {
            const uint32_t g1 = forest.find(c.a), g2 = forest.find(c.b);
            if (g1 == g2) continue;
            e = ext[top()];
            if (info.size() > 2 && same_pair(forest.find(e.a), forest.find(e.b), g1, g2)) limbo = e;
            while (info.size() > 2 && (forest.find(e.a) == forest.find(e.b) ||
                                       same_pair(forest.find(e.a), forest.find(e.b), g1, g2))) {
                ext.erase(ext.begin() + top());
                if (ext.empty()) break;
                e = ext[top()];
            }
            const bool satisfies = info.at(g1).mem + info.at(g2).mem >= total_mem;
            uint32_t groups = static_cast<uint32_t>(info.size()) - static_cast<uint32_t>(infeasible.size());
            const bool bad1 = infeasible.count(g1) != 0, bad2 = infeasible.count(g2) != 0;
            if (bad1 && bad2) {
                if (satisfies) groups += 1;
            } else if (!bad1 && !bad2) {
                groups -= 1;
            }
            const float art = all_reduce_time(groups, bottleneck(A(e.a, e.b), B(e.a, e.b), m.grad_buffer, groups));
            if (info.at(g1).should_merge(info.at(g2), art, effective, m)) {
                limbo = Edge{};
                merge(g1, g2, satisfies);
            }
            if (!limbo.null_edge()) ext.push_back(limbo);
        }
    }
    device_to_group->resize(W);
    for (int i = 0; i < W; ++i) (*device_to_group)[i] = forest.find(i);
    return infeasible.empty();
}

// Experts to the members of one group (decider.cuh:273-329).  rates / mems are indexed by the
// member's position in the group; returns false when the group cannot hold every expert.
inline bool assign(const std::vector<float>& rates, const std::vector<uint32_t>& mems,
                   const std::vector<uint32_t>& costs, std::vector<uint32_t>* out) {
    const int W = static_cast<int>(rates.size()), n = static_cast<int>(costs.size());
    // ordered expert set: cost ascending, id descending (decider.cuh:279-282)
    std::vector<uint32_t> t(n);
    for (int e = 0; e < n; ++e) t[e] = e;
    std::stable_sort(t.begin(), t.end(), [&](uint32_t x, uint32_t y) {
        return costs[x] == costs[y] ? x > y : costs[x] < costs[y];
    });
    long long total_cost = 0, have = 0;
    for (int e = 0; e < n; ++e) total_cost += costs[e];
    const long long total_mem = n;
    const long long req = (total_mem + W - 1) / W;
    bool well = true;
    float total_rate = 0.f;
    for (int i = 0; i < W; ++i) {
        well = well && mems[i] >= req;
        total_rate += rates[i];
        have += mems[i];
    }
    if (have < n) return false;
    std::vector<int> order(W);
    for (int i = 0; i < W; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return rates[x] > rates[y]; });
    std::vector<float> w_rate(W);
    std::vector<long long> w_mem(W);
    for (int i = 0; i < W; ++i) {
        w_rate[i] = rates[order[i]];
        w_mem[i] = mems[order[i]];
    }
    out->assign(n, 0);
    int j = 0;
    while (!t.empty()) {
        const float raw = w_rate[j] * static_cast<float>(total_cost) / total_rate;
        long long b = (std::isfinite(raw) && std::fabs(raw) < 2147483648.f)
                          ? static_cast<long long>(std::floor(raw)) : total_cost;
        long long budget = std::max<long long>(b, 1);
        const long long allocated = budget;
        while (budget > 0 && w_mem[j] > 0 && !t.empty()) {
            const uint32_t want = static_cast<uint32_t>(budget) & 0xFFFFu;  // 16-bit sentinel cost
            size_t lower = t.size();
            for (size_t k = 0; k < t.size(); ++k) {
                const uint32_t e = t[k];
                if (!(costs[e] < want || (costs[e] == want && e > 0))) {
                    lower = k;
                    break;
                }
            }
            uint32_t best = t.back();
            if (lower < t.size()) {
                if (static_cast<long long>(costs[t[lower]]) == budget || lower == 0) {
                    best = t[lower];
                } else {
                    size_t upper = t.size();
                    for (size_t k = 0; k < t.size(); ++k)
                        if (costs[t[k]] > want) {
                            upper = k;
                            break;
                        }
                    if (upper < t.size()) {  // comps/expert.cuh:73-77
                        const uint32_t lo = t[lower], hi = t[upper];
                        const uint32_t lm = (want > costs[lo] ? want - costs[lo] : costs[lo] - want) & 0xFFFFu;
                        const uint32_t rm = (want > costs[hi] ? want - costs[hi] : costs[hi] - want) & 0xFFFFu;
                        best = lm <= rm ? lo : hi;
                    } else {
                        best = t[lower];
                    }
                }
            }
            (*out)[best] = order[j];
            t.erase(std::find(t.begin(), t.end(), best));
            w_mem[j] -= 1;
            budget -= costs[best];
        }
        total_cost -= allocated - budget;
        if (w_mem[j] == 0 || well) total_rate -= w_rate[j];
        j = (j + 1) % W;
    }
    return true;
}

// What one rank needs at start-up (bootstrap.cuh:170-265).
inline bool make_plan(const Inputs& in, int rank, Plan* p, std::string* why) {
    if (in.world < 1 || rank < 0 || rank >= in.world || in.num_experts == 0 ||
        (int)in.rate.size() != in.world || (int)in.mem.size() != in.world ||
        in.alpha.size() != (size_t)in.world * in.world || in.beta.size() != in.alpha.size()) {
        *why = "inconsistent planner inputs";
        return false;
    }
    p->feasible = decide(in, &p->device_to_group);
    if (!p->feasible) return true;
    auto members = [&](uint32_t gid) {  // comps/niche.cuh:15-27
        std::vector<uint32_t> v;
        for (int i = 0; i < in.world; ++i)
            if (p->device_to_group[i] == gid) v.push_back(i);
        return v;
    };
    const std::vector<uint32_t> costs(in.num_experts, in.expert_cost);
    auto tally_of = [&](const std::vector<uint32_t>& grp, std::vector<uint32_t>* e2m, std::vector<uint32_t>* tally) {
        std::vector<float> r;
        std::vector<uint32_t> mm;
        for (uint32_t d : grp) {
            r.push_back(in.rate[d]);
            mm.push_back(in.mem[d]);
        }
        if (!assign(r, mm, costs, e2m)) return false;
        tally->assign(grp.size(), 0);
        for (uint32_t e : *e2m) (*tally)[e] += 1;
        return true;
    };
    const uint32_t my_group = p->device_to_group[rank];
    p->group_ranks = members(my_group);
    p->group_rank = static_cast<uint32_t>(std::find(p->group_ranks.begin(), p->group_ranks.end(), (uint32_t)rank) -
                                          p->group_ranks.begin());
    std::vector<uint32_t> tally;
    if (!tally_of(p->group_ranks, &p->expert_to_member, &tally)) {
        *why = "the group cannot hold every expert";
        return false;
    }
    p->local_experts = tally[p->group_rank];
    p->expert_slots = *std::max_element(tally.begin(), tally.end());
    p->widest_group = static_cast<uint32_t>(p->group_ranks.size());
    std::set<uint32_t> gids(p->device_to_group.begin(), p->device_to_group.end());
    for (uint32_t gid : gids) {
        if (gid == my_group) continue;
        const std::vector<uint32_t> other = members(gid);
        p->widest_group = std::max<uint32_t>(p->widest_group, (uint32_t)other.size());
        std::vector<uint32_t> e2m, ot;
        if (!tally_of(other, &e2m, &ot)) {
            *why = "a group cannot hold every expert";
            return false;
        }
        p->expert_slots = std::max(p->expert_slots, *std::max_element(ot.begin(), ot.end()));
    }
    return true;
}

}  // namespace placement
}  // namespace kleos
