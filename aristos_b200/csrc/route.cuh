// Router: gate GEMM + softmax + top-k, near-tie refinement, slot assignment.
//
// Semantics follow the reference gate (moe/gate.cuh:470-720): logits = A * Wg^T with fp32
// accumulation, softmax over the E real experts, k rounds of masked arg-max with ties to the
// lowest expert id (:654-670), mCw = sum of the k winning probabilities (:669), slot per
// (expert, token) kept iff slot < EC (:689-718).  Two deliberate differences: slots are
// handed out in ascending token order (the reference uses atomicAdd arrival order,
// :698-700), and tokens whose k-th / (k+1)-th logits are closer than fp32 summation error
// are re-evaluated in fp64 so the selected set does not depend on accumulation order.
#pragma once

#include "common.cuh"

namespace kleos {

struct RouteArgs {
    const void* A;        // [S,H] activations
    const void* Wg;       // [PX,H] gate weight, row e = expert e
    const float* bias;    // [E] logit bias (zeros when unused)
    void* probs;          // [S,PX] gate probabilities (element type)
    int* topk;            // [S,K]
    float* mcw;           // [S]
    int* refine_list;     // token ids needing fp64 re-evaluation
    int* refine_count;
    double* refine_logits;  // [S,E] fp64 logits of listed tokens
    int* refine_done;       // [S] per listed token: logits finished (zero between forwards)
    int S, H, E, K, PX;
    float tie_eps;
    // training mode only, else null: [router blocks][PX] column sums of the fp32 probabilities
    // of each block's tokens, summed in a fixed order (the reference accumulates the same
    // per-expert mean with atomicAdd, moe/gate.cuh:607-635)
    float* col_partial;
};

// One token's routing decision from its fp32 logits (in shared memory):
// a single ascending pass keeps the K+1 largest logits in order (strict '>' on insertion, so
// equal values keep the lower expert id in front -- the reference's tie rule,
// moe/gate.cuh:662-667), a second pass sums the exponentials.  Writes top-k ids and the sum of
// the k winning probabilities, and returns the softmax statistics and the k-th / (k+1)-th
// margin used to decide whether the token needs the fp64 re-evaluation.
struct RowDecision {
    float max, inv_den, kth, margin;
};

// KT is a compile-time bound on K: the insertion chain is KT+1 registers long, so a top-2
// layer does not pay for the eight-deep chain of the largest supported k.
template <int KT>
__device__ __forceinline__ RowDecision decide_row_k(const float* l, int E, int K, int* topk_out,
                                                    float* mcw_out) {
    float val[KT + 1];
    int idx[KT + 1];
#pragma unroll
    for (int j = 0; j <= KT; ++j) {
        val[j] = -INFINITY;
        idx[j] = 0;
    }
    for (int e = 0; e < E; ++e) {
        float v = l[e];
        int id = e;
#pragma unroll
        for (int j = 0; j <= KT; ++j) {
            if (j <= K && v > val[j]) {
                const float tv = val[j];
                const int ti = idx[j];
                val[j] = v;
                idx[j] = id;
                v = tv;
                id = ti;
            }
        }
    }
    const float m = val[0];
    float d = 0.f;
    for (int e = 0; e < E; ++e) d += __expf(l[e] - m);
    const float inv = 1.f / d;
    float w = 0.f, kth = 0.f, next = -INFINITY;
#pragma unroll
    for (int j = 0; j <= KT; ++j) {
        if (j < K) {
            topk_out[j] = idx[j];
            w += __expf(val[j] - m) * inv;
            kth = val[j];
        } else if (j == K) {
            next = val[j];
        }
    }
    *mcw_out = w;
    RowDecision r;
    r.max = m;
    r.inv_den = inv;
    r.kth = kth;
    r.margin = (K < E) ? kth - next : INFINITY;
    return r;
}

__device__ __forceinline__ RowDecision decide_row(const float* l, int E, int K, int* topk_out,
                                                  float* mcw_out) {
    if (K <= 1) return decide_row_k<1>(l, E, K, topk_out, mcw_out);
    if (K <= 2) return decide_row_k<2>(l, E, K, topk_out, mcw_out);
    if (K <= 4) return decide_row_k<4>(l, E, K, topk_out, mcw_out);
    return decide_row_k<kMaxTopK>(l, E, K, topk_out, mcw_out);
}

// One block = 64 tokens x PXT experts, 256 threads, each thread a 4 x (PXT/16) register tile.
template <typename T, int PXT>
__global__ void __launch_bounds__(256) route_kernel(RouteArgs a) {
    constexpr int BM = 64, BK = 32, TN = PXT / 16;
    constexpr int LDA = BM + 1, LDB = PXT + 1, LDL = PXT + 1;
    extern __shared__ float smem[];
    float* As = smem;                  // [BK][LDA]
    float* Bs = smem + BK * LDA;       // [BK][LDB]
    float* Ls = smem;                  // [BM][LDL], reused after the K loop
    float* rowmax = smem + BM * LDL;   // [BM]
    float* rowden = rowmax + BM;       // [BM]

    const T* A = static_cast<const T*>(a.A);
    const T* Wg = static_cast<const T*>(a.Wg);
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int row0 = blockIdx.x * BM;
    const int H = a.H;

    float acc[4][TN];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    const int lrow = tid >> 2, lk = (tid & 3) * 8;
    for (int k0 = 0; k0 < H; k0 += BK) {
        {
            const int gr = row0 + lrow;
            float v[8];
            if (gr < a.S) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = Elem<T>::to_f(A[(size_t)gr * H + k0 + lk + i]);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) As[(lk + i) * LDA + lrow] = v[i];
        }
#pragma unroll
        for (int it = 0; it < PXT / 64; ++it) {
            const int br = lrow + it * 64;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                Bs[(lk + i) * LDB + br] = Elem<T>::to_f(Wg[(size_t)br * H + k0 + lk + i]);
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < BK; ++k) {
            float av[4], bv[TN];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[k * LDA + ty * 4 + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) bv[j] = Bs[k * LDB + tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
    // logits (+bias) into shared memory
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int e = tx + 16 * j;
            Ls[(ty * 4 + i) * LDL + e] = acc[i][j] + (e < a.E ? a.bias[e] : 0.f);
        }
    __syncthreads();

    // one thread per token: softmax statistics, top-k, near-tie detection
    if (tid < BM && row0 + tid < a.S) {
        const RowDecision r = decide_row(Ls + tid * LDL, a.E, a.K,
                                         a.topk + (size_t)(row0 + tid) * a.K, a.mcw + row0 + tid);
        rowmax[tid] = r.max;
        rowden[tid] = r.inv_den;
        if (r.margin < a.tie_eps * fmaxf(1.f, fabsf(r.kth))) {
            const int pos = atomicAdd(a.refine_count, 1);
            a.refine_list[pos] = row0 + tid;  // list has room for every token
        }
    }
    __syncthreads();
    // probabilities, coalesced, padding columns zero (PX == PXT: both are E rounded up to 64)
    T* probs = static_cast<T*>(a.probs);
    float colsum = 0.f;  // 256 % PXT == 0: a thread always visits the same expert column
    for (int idx = tid; idx < BM * PXT; idx += 256) {
        const int r = idx / PXT, e = idx % PXT;
        if (row0 + r >= a.S) break;
        float p = 0.f;
        if (e < a.E) p = __expf(Ls[r * LDL + e] - rowmax[r]) * rowden[r];
        colsum += p;
        probs[(size_t)(row0 + r) * PXT + e] = Elem<T>::from_f(p);
    }
    if (a.col_partial != nullptr) {
        __syncthreads();  // everyone is done with the logit tile: reuse it
        smem[tid] = colsum;
        __syncthreads();
        if (tid < PXT) {
            float sum = 0.f;
            for (int k = 0; k < 256 / PXT; ++k) sum += smem[tid + k * PXT];
            a.col_partial[(size_t)blockIdx.x * PXT + tid] = sum;
        }
    }
}

// Training-mode gate statistics of one rank's tokens, as the reference keeps them in its
// bookkeeping (types.cuh:944-960): mean probability per expert (moe/gate.cuh:607-635), fraction
// of the tokens that chose each expert (unclamped, :698-705) and the auxiliary loss
// sum_e mean_prob[e] * mean_count[e] / E (:763-773).  One block; all sums in a fixed order.
// out = [mean_prob E][mean_count E][loss 1].
__global__ void __launch_bounds__(256) gate_stats_kernel(const float* col_partial, int blocks,
                                                         int PX, const unsigned* counts, int S,
                                                         int E, float* out) {
    __shared__ float term[256];
    const int e = threadIdx.x;
    float t = 0.f;
    if (e < E) {
        float sum = 0.f;
        for (int b = 0; b < blocks; ++b) sum += col_partial[(size_t)b * PX + e];
        const float mp = sum / (float)S, mc = (float)counts[e] / (float)S;
        out[e] = mp;
        out[E + e] = mc;
        t = mp * mc / (float)E;
    }
    term[e] = t;
    __syncthreads();
    if (e == 0) {
        float loss = 0.f;
        for (int i = 0; i < E; ++i) loss += term[i];
        out[2 * E] = loss;
    }
}

template <int PXT>
constexpr size_t route_smem_bytes() {
    constexpr int BM = 64, BK = 32;
    constexpr size_t k_loop = sizeof(float) * (BK * (BM + 1) + BK * (PXT + 1));
    constexpr size_t epi = sizeof(float) * (BM * (PXT + 1) + 2 * BM);
    return k_loop > epi ? k_loop : epi;
}

// fp64 re-evaluation of the tokens on the refine list.  One warp per (listed token, expert)
// dot product; the warp that completes a token's last logit redoes that token's selection.
template <typename T>
__global__ void __launch_bounds__(256) refine_kernel(RouteArgs a) {
    constexpr int VEC = 16 / sizeof(T);
    const T* A = static_cast<const T*>(a.A);
    const T* Wg = static_cast<const T*>(a.Wg);
    const int n = *a.refine_count;
    const int lane = threadIdx.x & 31;
    const int warps = gridDim.x * (blockDim.x >> 5);
    for (int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); item < n * a.E;
         item += warps) {
        const int i = item / a.E, e = item - i * a.E;
        const int t = a.refine_list[i];
        const T* x = A + (size_t)t * a.H;
        const T* w = Wg + (size_t)e * a.H;
        double s = 0.0;
#pragma unroll 4
        for (int h = lane * VEC; h < a.H; h += 32 * VEC) {
            const uint4 xr = *reinterpret_cast<const uint4*>(x + h);
            const uint4 wr = *reinterpret_cast<const uint4*>(w + h);
            const T* xv = reinterpret_cast<const T*>(&xr);
            const T* wv = reinterpret_cast<const T*>(&wr);
#pragma unroll
            for (int q = 0; q < VEC; ++q)
                s += (double)Elem<T>::to_f(xv[q]) * (double)Elem<T>::to_f(wv[q]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        int done = 0;
        if (lane == 0) {
            a.refine_logits[(size_t)i * a.E + e] = s + (double)a.bias[e];
            __threadfence();
            done = atomicAdd(a.refine_done + i, 1);
        }
        done = __shfl_sync(0xffffffffu, done, 0);
        if (done != a.E - 1) continue;
        // last logit of token i: the whole warp redoes the selection on the fp64 logits
        // (k rounds of warp arg-max, ties to the lowest expert id) and the fp32 softmax
        __threadfence();
        constexpr int PER_LANE = 8;  // E <= 256
        const double* l64 = a.refine_logits + (size_t)i * a.E;
        double cand[PER_LANE];
        float lf[PER_LANE];
#pragma unroll
        for (int q = 0; q < PER_LANE; ++q) {
            const int ee = lane + 32 * q;
            cand[q] = ee < a.E ? __ldcg(l64 + ee) : -INFINITY;
            lf[q] = (float)cand[q];
        }
        float m = -INFINITY;
#pragma unroll
        for (int q = 0; q < PER_LANE; ++q) m = fmaxf(m, lf[q]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float d = 0.f;
#pragma unroll
        for (int q = 0; q < PER_LANE; ++q)
            if (lane + 32 * q < a.E) d += __expf(lf[q] - m);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        const float inv = 1.f / d;
        float wsum = 0.f;
        for (int j = 0; j < a.K; ++j) {
            double bv = -INFINITY;
            int be = 0x7fffffff;
#pragma unroll
            for (int q = 0; q < PER_LANE; ++q) {
                const int ee = lane + 32 * q;  // ascending per lane, so '>' keeps the lower id
                if (cand[q] > bv) {
                    bv = cand[q];
                    be = ee;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const double ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oe = __shfl_xor_sync(0xffffffffu, be, o);
                if (ov > bv || (ov == bv && oe < be)) {
                    bv = ov;
                    be = oe;
                }
            }
            // every lane now agrees on (bv, be); its owner retires the candidate
#pragma unroll
            for (int q = 0; q < PER_LANE; ++q)
                if (lane + 32 * q == be) cand[q] = -INFINITY;
            if (lane == 0) a.topk[(size_t)t * a.K + j] = be;
            wsum += __expf((float)bv - m) * inv;
        }
        if (lane == 0) {
            a.mcw[t] = wsum;
            a.refine_done[i] = 0;  // ready for the next forward
        }
        T* probs = static_cast<T*>(a.probs);
#pragma unroll
        for (int q = 0; q < PER_LANE; ++q) {
            const int ee = lane + 32 * q;
            if (ee < a.E) probs[(size_t)t * a.PX + ee] = Elem<T>::from_f(__expf(lf[q] - m) * inv);
        }
    }
}

struct SlotArgs {
    const int* topk;        // [S,K]
    int* slots;             // [S,K] slot or kDropped
    int* cell_tokens;       // [E,pEC] token id held by each slot
    unsigned* counts;       // [E] unclamped
    int* tile_hist;         // [tiles, E] per-tile histogram of the chosen experts
    int S, K, E, EC, pEC;
    // count flags: cflag[owner][rank*nLx + le] = (epoch<<32)|routed, one 8-byte peer store per
    // expert (the reference's first-stage signal carries the same count, types.cuh:300-317)
    char* peer_arena[kMaxWorld];
    size_t cflag_offset;
    int rank, nLx;
    uint32_t epoch;
};

// Slots in ascending token order (the reference hands them out in atomicAdd arrival order,
// moe/gate.cuh:689-718; ascending order is one of its possible outcomes and is reproducible).
// Two small launches over tiles of 128 tokens:
//   tile_hist_kernel  per-tile histogram of the chosen experts;
//   slot_kernel       base slot of every expert for the tile = sum of the earlier tiles'
//                     histograms, then each token's rank inside the tile; the last block also
//                     has the totals and publishes them: counts[e] and one count flag per
//                     expert to the expert's owner rank.
constexpr int kSlotTile = 128;

__global__ void __launch_bounds__(256) tile_hist_kernel(SlotArgs a) {
    __shared__ int hist[256];  // E <= 256
    const int tid = threadIdx.x, tok0 = blockIdx.x * kSlotTile;
    for (int e = tid; e < a.E; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const int n_own = min(kSlotTile, a.S - tok0) * a.K;
    for (int i = tid; i < n_own; i += blockDim.x) atomicAdd(&hist[a.topk[(size_t)tok0 * a.K + i]], 1);
    __syncthreads();
    for (int e = tid; e < a.E; e += blockDim.x) a.tile_hist[(size_t)blockIdx.x * a.E + e] = hist[e];
}

__global__ void __launch_bounds__(256) slot_kernel(SlotArgs a) {
    __shared__ int base[256];
    const int tid = threadIdx.x, b = blockIdx.x;
    const int tok0 = b * kSlotTile;
    const bool last = b == (int)gridDim.x - 1;
    // base slot of every expert = sum of the earlier tiles' histograms; the tiles are split
    // over the threads that share an expert so the loads are independent and coalesced
    __shared__ int part[256];
    {
        int ep = 1;
        while (ep < a.E) ep <<= 1;            // experts rounded up to a power of two (<= 256)
        const int groups = blockDim.x / ep;   // threads per expert
        const int e = tid % ep, grp = tid / ep;
        int run = 0;
        if (e < a.E && grp < groups)
            for (int t = grp; t < b; t += groups) run += a.tile_hist[(size_t)t * a.E + e];
        part[tid] = run;
        __syncthreads();
        if (tid < a.E) {
            int sum = 0;
            for (int gi = 0; gi < groups; ++gi) sum += part[gi * ep + tid];
            base[tid] = sum;
        }
        __syncthreads();
    }
    for (int e = tid; e < a.E; e += blockDim.x) {
        const int run = base[e];
        if (last) {
            const int total = run + a.tile_hist[(size_t)b * a.E + e];
            a.counts[e] = (unsigned)total;
            const int owner = e / a.nLx, le = e - owner * a.nLx;
            st_release_sys(reinterpret_cast<unsigned long long*>(a.peer_arena[owner] + a.cflag_offset) +
                               ((size_t)a.rank * a.nLx + le),
                           make_flag(a.epoch, (unsigned)min(total, a.EC)));
        }
    }
    // Rank of every (token, choice) entry among the earlier entries of the tile that chose the
    // same expert.  Entries are taken in order, 256 at a time: inside a warp the rank comes from
    // a match mask, across the eight warps from a per-warp count table, and `base` carries the
    // running total into the next group of 256.
    __shared__ int wcount[8][256];
    for (int i = tid; i < 8 * 256; i += blockDim.x) (&wcount[0][0])[i] = 0;
    const int n_own = min(kSlotTile, a.S - tok0) * a.K;
    const int warp = tid >> 5, lane = tid & 31;
    __syncthreads();
    for (int i0 = 0; i0 < n_own; i0 += 256) {
        const int i = i0 + tid;
        const int e = i < n_own ? a.topk[(size_t)tok0 * a.K + i] : -1;
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int before = __popc(peers & ((1u << lane) - 1u));
        const bool leader = e >= 0 && before == 0;
        if (leader) wcount[warp][e] = __popc(peers);
        __syncthreads();
        if (e >= 0) {
            int pos = base[e] + before;
            for (int w = 0; w < warp; ++w) pos += wcount[w][e];
            if (pos < a.EC) {
                a.slots[(size_t)tok0 * a.K + i] = pos;
                a.cell_tokens[(size_t)e * a.pEC + pos] = tok0 + i / a.K;
            } else {
                a.slots[(size_t)tok0 * a.K + i] = kDropped;
            }
        }
        __syncthreads();
        if (leader) {
            atomicAdd(&base[e], wcount[warp][e]);
            wcount[warp][e] = 0;
        }
        __syncthreads();
    }
}

}  // namespace kleos
