// Token dispatch into the expert ranks' cells, the tile plan built from the arrived counts,
// and the gate-weighted combine of the returned rows.
//
// Roles follow the reference: packet::dispatch (os/packet.cuh:35-286) copies the routed,
// unscaled rows into cell [source rank][local expert] on the expert's rank and raises one
// flag per (source, expert) carrying the routed count, also when the count is zero
// (:240-259); the decoder turns arrived packets into 128-row tasks (:304-398); combine
// (os/processor/processor.cuh:27-205) scales returned rows and accumulates them per token.
// Here every peer is reached with plain 16-byte stores into its mapped cells over NVLink and
// the combine is a deterministic gather-sum instead of element-wise atomics.
#pragma once

#include "common.cuh"

namespace kleos {

// Offsets of the regions inside each rank's symmetric arena (identical on every rank).
struct ArenaLayout {
    size_t xcell;  // [world*nLx][pEC][H] dispatched token rows, by (source rank, local expert)
    size_t ycell;  // [E][pEC][H] returned FFN rows, by global expert
    size_t xflag;  // [world*nLx] u64: (epoch<<32)|routed count, raised when the cell's rows are stored
    size_t cflag;  // [world*nLx] u64: (epoch<<32)|routed count, raised as soon as the count is known
    size_t yflag;  // [world] u64: (epoch<<32)|1 when that expert rank has returned everything
    size_t ypflag; // [E][pEC/128] u64: (epoch<<32)|1 when that 128-row panel of results has arrived
    size_t bytes;
};

struct DispatchArgs {
    const void* A;             // [S,H]
    const int* cell_tokens;    // [E,pEC]
    const unsigned* counts;    // [E]
    PeerTable peers;
    ArenaLayout lay;
    unsigned* done_counter;    // zero between launches
    int H, E, EC, pEC, nLx, rank, world;
    uint32_t epoch;
    int elem_bytes;
    int le_begin, le_end;      // only experts whose local index is in [le_begin, le_end) are moved
};

// Warp per routed row; rows are spread over the whole grid.
__global__ void __launch_bounds__(256) dispatch_kernel(DispatchArgs a) {
    __shared__ unsigned prefix[257];  // E <= 256
    __shared__ bool last_block;
    const int tid = threadIdx.x;
    // Rows are sent in this order: local expert index first, and for each of them the owner
    // ranks starting with the one after this rank.  At any moment the source ranks therefore
    // write to DIFFERENT owners, instead of all pushing into the same GPU's NVLink ingress.
    // prefix[i] = rows before order position i (zero-length outside this launch's range).
    for (int i = tid; i < a.E; i += blockDim.x) {
        const int le = i / a.world, owner = (a.rank + 1 + i % a.world) % a.world;
        const int e = owner * a.nLx + le;
        prefix[i + 1] = (le >= a.le_begin && le < a.le_end) ? min(a.counts[e], (unsigned)a.EC) : 0u;
    }
    __syncthreads();
    if (tid == 0) {
        unsigned run = 0;
        for (int e = 0; e < a.E; ++e) {
            const unsigned n = prefix[e + 1];
            prefix[e] = run;
            run += n;
        }
        prefix[a.E] = run;
    }
    __syncthreads();
    const unsigned total = prefix[a.E];
    const int lane = tid & 31;
    const unsigned warps = gridDim.x * (blockDim.x >> 5);
    const unsigned row_chunks = (unsigned)((size_t)a.H * a.elem_bytes / 16);
    for (unsigned g = blockIdx.x * (blockDim.x >> 5) + (tid >> 5); g < total; g += warps) {
        int lo = 0, hi = a.E;  // last order position with prefix[] <= g
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (prefix[mid] <= g) lo = mid; else hi = mid;
        }
        const unsigned slot = g - prefix[lo];
        const int le = lo / a.world, owner = (a.rank + 1 + lo % a.world) % a.world;
        const int e = owner * a.nLx + le;
        const int tok = a.cell_tokens[(size_t)e * a.pEC + slot];
        const uint4* src = reinterpret_cast<const uint4*>(
            static_cast<const char*>(a.A) + (size_t)tok * a.H * a.elem_bytes);
        uint4* dst = reinterpret_cast<uint4*>(
            a.peers.arena[owner] + a.lay.xcell +
            (((size_t)a.rank * a.nLx + le) * a.pEC + slot) * a.H * a.elem_bytes);
        // eight 16-byte loads in flight per lane before the first store is issued
        for (unsigned c0 = lane; c0 < row_chunks; c0 += 256) {
            uint4 v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (c0 + 32 * q < row_chunks) v[q] = __ldg(src + c0 + 32 * q);
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (c0 + 32 * q < row_chunks) dst[c0 + 32 * q] = v[q];
        }
    }
    // publish: every block fences its peer stores, the last block to finish raises the flags
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        const unsigned prev = atomicAdd(a.done_counter, 1u);
        last_block = (prev == gridDim.x - 1);
    }
    __syncthreads();
    if (last_block) {
        __threadfence_system();
        for (int e = tid; e < a.E; e += blockDim.x) {
            const int owner = e / a.nLx, le = e - owner * a.nLx;
            if (le < a.le_begin || le >= a.le_end) continue;
            unsigned long long* f = reinterpret_cast<unsigned long long*>(
                a.peers.arena[owner] + a.lay.xflag) + ((size_t)a.rank * a.nLx + le);
            st_release_sys(f, make_flag(a.epoch, min(a.counts[e], (unsigned)a.EC)));
        }
        if (tid == 0) *a.done_counter = 0u;
    }
}

// One 128-row panel of one cell: what a GEMM m-tile works on.
struct PanelEntry {
    int row_base;  // first row in the xcell / y1cell row space
    int rows;      // valid rows (1..128)
    int le;        // local expert
    int src;       // source rank
};

struct PlanArgs {
    const char* arena;       // this rank's arena
    ArenaLayout lay;
    PanelEntry* panels;      // [world*nLx*pEC/128]
    int* le_start;           // [nLx+1] panels of local expert le are [le_start[le], le_start[le+1])
    unsigned* cell_counts;   // [world*nLx] routed count per (source, local expert)
    DeviceStatus* status;
    int world, nLx, pEC;
    uint32_t epoch;
    long long wait_cycles;
    int le_begin, le_end;    // local experts planned by this launch; panels are appended
    int rank;
};

// Single block.  Waits (bounded) for the count flag of every (source, local expert) cell, then
// lists the panels grouped by local expert so that tiles sharing a weight tile run together.
__global__ void __launch_bounds__(1024) plan_kernel(PlanArgs a) {
    __shared__ int failed;
    __shared__ int cnt_s[2048];  // world * nLx <= 8 * 256; a count can reach pEC, which has no 16-bit limit
    const int cells = a.world * a.nLx;
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    const unsigned long long* flags =
        reinterpret_cast<const unsigned long long*>(a.arena + a.lay.xflag);
    for (int c = threadIdx.x; c < cells; c += blockDim.x) {
        const int cle = c % a.nLx;
        if (cle < a.le_begin || cle >= a.le_end) continue;
        unsigned long long v = 0;
        if (!wait_flag(flags + c, a.epoch, a.wait_cycles, &v)) {
            report_error(a.status, KLEOS_AT_PLAN_WAIT, c, (int)a.epoch);
            atomicExch(&failed, 1);
            a.cell_counts[c] = 0;
            cnt_s[c] = 0;
        } else {
            const unsigned n = min((unsigned)(v & 0xffffffffu), (unsigned)a.pEC);
            a.cell_counts[c] = n;
            cnt_s[c] = (int)n;
        }
    }
    __syncthreads();
    // plan order: local expert by local expert, sources starting with the rank after this one
    // (so that the expert ranks' result stores fan out over different source ranks instead of
    // converging on one).  One thread scans the panel counts of the cells in that order, then
    // every cell writes its own panels.
    __shared__ int off_s[2049];
    const int ncell = (a.le_end - a.le_begin) * a.world;
    if (threadIdx.x == 0) {
        int n = a.le_begin == 0 ? 0 : a.le_start[a.le_begin];  // continue the previous launch's list
        for (int o = 0; o < ncell; ++o) {
            const int le = a.le_begin + o / a.world, src = (a.rank + 1 + o % a.world) % a.world;
            if (o % a.world == 0) a.le_start[le] = n;
            off_s[o] = n;
            if (!failed) n += (cnt_s[src * a.nLx + le] + kTileM - 1) / kTileM;
        }
        a.le_start[a.le_end] = n;
    }
    __syncthreads();
    if (failed) return;
    for (int o = threadIdx.x; o < ncell; o += blockDim.x) {
        const int le = a.le_begin + o / a.world, src = (a.rank + 1 + o % a.world) % a.world;
        const int c = src * a.nLx + le;
        const int cnt = cnt_s[c];
        int n = off_s[o];
        for (int r = 0; r < cnt; r += kTileM)
            a.panels[n++] = PanelEntry{c * a.pEC + r, min(kTileM, cnt - r), le, src};
    }
}

struct CombineArgs {
    const char* arena;   // this rank's arena (ycell, yflag)
    ArenaLayout lay;
    const void* probs;   // [S,PX] element-rounded gate probabilities
    const int* topk;     // [S,K]
    const int* slots;    // [S,K]
    const float* mcw;    // [S]
    void* out;           // [S,H]
    DeviceStatus* status;
    int S, H, K, PX, pEC, world;
    uint32_t epoch;
    long long wait_cycles;
};

// out[t] = sum_j Element(prob[t,e_j]) * Element(y2[e_j][slot_j] / mCw[t]) over kept choices
// (reference processor.cuh:110-168); with k == 1 the row is copied unscaled (:170-204).
// Rows of tokens whose every choice was dropped are written as zeros.  Warp per token; KT is
// the compile-time top-k (0 = read it from the arguments), which lets the k row loads of
// several 16-byte chunks be issued together.
template <typename T, int KT>
__global__ void __launch_bounds__(256) combine_kernel(CombineArgs a) {
    __shared__ int failed;
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    if (threadIdx.x < a.world) {
        const unsigned long long* f =
            reinterpret_cast<const unsigned long long*>(a.arena + a.lay.yflag) + threadIdx.x;
        unsigned long long v;
        if (!wait_flag(f, a.epoch, a.wait_cycles, &v)) {
            report_error(a.status, KLEOS_AT_COMBINE_WAIT, threadIdx.x, (int)a.epoch);
            atomicExch(&failed, 1);
        }
    }
    __syncthreads();
    if (failed) return;

    constexpr int VEC = 16 / sizeof(T);
    constexpr int KMAX = KT > 0 ? KT : kMaxTopK;
    constexpr int UNR = KT > 0 && KT <= 2 ? 4 : 1;
    const int K = KT > 0 ? KT : a.K;
    const int lane = threadIdx.x & 31;
    const int warps = gridDim.x * (blockDim.x >> 5);
    const T* probs = static_cast<const T*>(a.probs);
    const T* ycell = reinterpret_cast<const T*>(a.arena + a.lay.ycell);
    const int chunks = a.H / VEC;
    for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < a.S; t += warps) {
        const T* yrow[KMAX];
        float p[KMAX];
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
            yrow[j] = nullptr;
            p[j] = 0.f;
            if (j < K) {
                const int e = a.topk[(size_t)t * K + j];
                const int sl = a.slots[(size_t)t * K + j];
                p[j] = Elem<T>::to_f(probs[(size_t)t * a.PX + e]);
                if (sl != kDropped) yrow[j] = ycell + ((size_t)e * a.pEC + sl) * a.H;
            }
        }
        const float w = a.mcw[t];
        const float inv_w = 1.f / w;
        T* orow = static_cast<T*>(a.out) + (size_t)t * a.H;
        for (int c0 = lane; c0 < chunks; c0 += 32 * UNR) {
            uint4 raw[UNR][KMAX];
#pragma unroll
            for (int u = 0; u < UNR; ++u)
#pragma unroll
                for (int j = 0; j < KMAX; ++j)
                    if (j < K && yrow[j] != nullptr && c0 + 32 * u < chunks)
                        raw[u][j] = ld_cg_v4(yrow[j] + (size_t)(c0 + 32 * u) * VEC);
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const int c = c0 + 32 * u;
                if (c >= chunks) break;
                uint4 o;
                if constexpr (sizeof(T) == 2) {
                    // 16-bit elements: Element(y / mCw) is one fp32 multiply and a packed round; the product
                    // with the bf16 probability and the running sum are single-rounding bf16x2
                    // instructions, which is exactly the element-type arithmetic of the
                    // reference's combine
                    using P2 = Pack2<T>;
                    typename P2::type acc2[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc2[i] = P2::from_f2(0.f, 0.f);
#pragma unroll
                    for (int j = 0; j < KMAX; ++j)
                        if (j < K && yrow[j] != nullptr) {
                            const typename P2::type* y2 = reinterpret_cast<const typename P2::type*>(&raw[u][j]);
                            const typename P2::type pj = P2::from_f2(p[j], p[j]);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                if (K > 1) {
                                    const float2 yf = P2::to_f2(y2[i]);
                                    const typename P2::type v = P2::from_f2(yf.x * inv_w, yf.y * inv_w);
                                    acc2[i] = P2::add(acc2[i], P2::mul(pj, v));
                                } else {
                                    acc2[i] = y2[i];
                                }
                            }
                        }
                    o = *reinterpret_cast<const uint4*>(acc2);
                } else {
                    float acc[VEC];
#pragma unroll
                    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
#pragma unroll
                    for (int j = 0; j < KMAX; ++j)
                        if (j < K && yrow[j] != nullptr) {
                            const T* yv = reinterpret_cast<const T*>(&raw[u][j]);
#pragma unroll
                            for (int i = 0; i < VEC; ++i) {
                                if (K > 1) {
                                    const float v = Elem<T>::round(Elem<T>::to_f(yv[i]) / w);
                                    const float sc = Elem<T>::round(p[j] * v);
                                    acc[i] = Elem<T>::round(acc[i] + sc);
                                } else {
                                    acc[i] = Elem<T>::to_f(yv[i]);
                                }
                            }
                        }
                    T* ov = reinterpret_cast<T*>(&o);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) ov[i] = Elem<T>::from_f(acc[i]);
                }
                *reinterpret_cast<uint4*>(orow + (size_t)c * VEC) = o;
            }
        }
    }
}

// Flag raised by the last GEMM2 block: tells every source rank that this expert rank has
// stored all of its result rows.
struct ReturnFlagArgs {
    PeerTable peers;
    ArenaLayout lay;
    unsigned* done_counter;
    int rank, world;
    uint32_t epoch;
    int suppress;  // test hook: do not raise the flags (exercises the bounded wait in combine)
};

__device__ __forceinline__ void publish_return_flags(const ReturnFlagArgs& r, bool* smem_last) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(r.done_counter, 1u);
        *smem_last = (prev == gridDim.x - 1);
    }
    __syncthreads();
    if (*smem_last) {
        __threadfence_system();
        if ((int)threadIdx.x < r.world && !r.suppress) {
            unsigned long long* f = reinterpret_cast<unsigned long long*>(
                r.peers.arena[threadIdx.x] + r.lay.yflag) + r.rank;
            st_release_sys(f, make_flag(r.epoch, 1u));
        }
        if (threadIdx.x == 0) *r.done_counter = 0u;
    }
}

}  // namespace kleos
