// The persistent MoE kernel: router (gate GEMM, softmax, top-k, slots), token dispatch, tile plan,
// both expert GEMMs and the gate-weighted combine of one forward in ONE launch, driven by an
// on-GPU tile scheduler.
//
// This is the counterpart of the reference's fused kernel with its in-kernel "OS"
// (moe/moe.cuh:77-144: dispatch blocks, processors and one scheduler / subscriber block run
// concurrently; os/scheduler.cuh:303-441, os/subscriber.cuh:56-332, os/processor/processor.cuh:
// 643-790).  What is kept: work starts as soon as its packet has landed, GEMM2 tasks of a row
// panel are released when the panel's GEMM1 tiles are done (processor.cuh:717-729), results go
// straight back into the source rank's memory with one signal per returned unit (:745-769), and
// control never returns to the host in between.  What is different on this machine:
//   * no central scheduler block and no 128-byte task descriptors: every rank first learns the
//     routed COUNT of every (source, local expert) cell (the count flags the router publishes),
//     from which each block derives the same complete tile list; a tile is then an integer, and
//     the "task queue" is one global atomic counter per rank from which block pairs claim the
//     next tile (a small shared-memory ring hands the claimed index to the roles of both
//     blocks of the pair);
//   * one 384-thread block per SM, paired with its neighbour (tcgen05 cta_group::2):
//       warp 0      TMA producer             warp 1      MMA issuer (leader block)
//       warp 2      tensor-memory owner      warp 3      subscriber (polls the flag the producer's
//                                                        NEXT tile depends on; abort propagation)
//       warps 4-7   accumulator read-back, bias / activation, stores (local y1 or the SOURCE
//                   rank's result cell over NVLink), completion counters and return flags
//       warps 8-11  transport: first this rank's token rows into the owners' cells (per-cell
//                   data flag when the cell's last row is stored), then the combine of every
//                   token whose result rows have come back;
//   * tile order G1(0) G1(1) G2(0) G1(2) G2(1) ... so a GEMM2 tile's inputs (all GEMM1 tiles of
//     its row-panel pair) always have smaller indices: claims are handed out in order, so a
//     waiting block can only wait for blocks that are already running.
// With Args::fuse_route the kernel begins with the router (reference gate::forward followed by a
// grid barrier, moe/moe.cuh:134, moe/gate.cuh:722-789): block pairs compute the gate logits of
// 256 tokens at a time on the same tensor-core pipeline (M = 256, N = the padded expert count),
// the read-back warps do softmax and top-k straight from tensor memory (one thread per token,
// no shared-memory logit tile), re-evaluate near-ties in fp64 on the spot, and write the per-tile
// expert histogram; after a grid barrier every tile ranks its tokens (slots in ascending token
// order) and the last tile publishes the counts; a second grid barrier precedes the dispatch.
// Every wait is bounded; a wait that runs out records where, raises the abort word that every
// loop polls, and the kernel returns normally.  Peer memory is only ever written (plain
// stores); nothing is loaded from a peer and no load is multicast.
#pragma once

#include <cuda.h>

#include "gemm_tc2.cuh"

namespace kleos {
namespace flow {

using gemm_tc2::A_STAGE_BYTES;
using gemm_tc2::BK;
using gemm_tc2::BM;
using gemm_tc2::BN;
using gemm_tc2::kSlices;
using gemm_tc2::SLICE_BYTES;
using gemm_tc2::TMEM_COLS;
using gemm_tc2::UMMA_K;

constexpr int kThreads = 384;      // 12 warps
constexpr int kRing = 8;           // claimed-tile ring per block (see hand_out())
constexpr int kMaxPanels = 384;    // 128-row panels one rank can plan
constexpr int kMaxLocal = 128;     // local experts per rank
constexpr int kMaxCells = 256;     // (source, local expert) cells = number of experts
constexpr int kUnitRows = 8;       // most rows of one cell a transport warp sends between two publications (Args::unit_rows)
constexpr int kCombineBlock = 8;   // tokens a warp classifies at a time (one per lane, first lanes)
constexpr int kMaxPasses = 8;      // combine passes (tokens grouped by when their last row returns)
constexpr int kRoleWarps = 10;     // producer, MMA, 4 read-back, 4 transport
constexpr int kCtlBytes = 32768;
constexpr int SMEM_BYTES = kSlices * SLICE_BYTES + 1024 + kCtlBytes;
constexpr int kStampSlots = 20;    // per block: see Stamp
constexpr int kStallSlots = 12;    // per block: see Stall

// Per-rank scheduler state in global memory.  Two copies: the forward of epoch n works on copy
// n & 1 and clears the other one for the forward after it, so nothing is memset between launches.
struct Counters {
    unsigned tile_next;        // the task queue: next unclaimed tile of the unified tile order
    unsigned unit_next;        // next unclaimed dispatch unit
    unsigned item_next;        // next unclaimed combine item
    unsigned panels_returned;  // row panels whose results have all been stored at their source
    unsigned abort_all;        // raised by whoever gives up; every loop polls it
    unsigned grid_bar[2];      // arrivals at the two grid barriers of the routing phase
    unsigned pad;
    unsigned cell_done[kMaxCells];    // rows of this rank's tokens stored so far, per expert
    unsigned pair_done[kMaxPanels];   // read-back warps that finished a GEMM1 tile, per panel pair
    unsigned panel_ret[kMaxPanels];   // read-back warps that finished a GEMM2 tile, per panel
};

enum Stamp {
    kStart = 0, kPlanned, kFirstTile, kLastGemm1, kLastTile, kDispatched, kCombined, kEnd,
    kRouted, kSlotted,  // the two grid barriers of the routing phase passed
    kGateAcc,           // gate logits of the block's last token tile complete in tensor memory
    kGateDone,          // ... and turned into probabilities, choices and the tile histogram
    kTopkDone,          // between the two: top-k and softmax sum of the tile known (before near-ties)
    kProbsDone,         // ... near-ties re-evaluated and probabilities stored
    kSlotBase,          // slot stage: base slot of every expert for the block's last tile known
    kSlotsDone,         // ... and the block's slots written (before the second grid barrier)
    kRouteBegin,        // set-up over (barriers, tensor memory, cluster barrier): the gate GEMM starts
    kFirstOperands,     // first K slice of the gate GEMM has landed in shared memory (leader block)
    kTopkPass1          // first pass over the logits (the K + 1 largest) done
};

// Cycles per block, tile stream only (a tuning aid, filled when Args::stalls is set).
enum Stall {
    kProdEmpty = 0,  // producer: waiting for a free pipeline stage
    kProdReady,      // producer: waiting for a cell's data flag or a pair's GEMM1 counter
    kProdTotal,      // producer: whole tile stream
    kMmaAcc,         // MMA issuer: waiting for a free accumulator
    kMmaFull,        // MMA issuer: waiting for operands
    kMmaTask,        // MMA issuer: waiting for the next claimed tile
    kMmaTotal,
    kBackAcc,        // read-back warp 0: waiting for a finished accumulator
    kBackPublish,    // ... publishing (fence + counters)
    kBackRead,       // ... reading back and storing
    kBackTotal,
    kProdFence       // producer: proxy fences in front of each tile's loads
};

struct Control {
    unsigned long long full[kSlices];    // used on the leader
    unsigned long long empty[kSlices];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];     // used on the leader, 8 arrivals
    unsigned long long task_full[kRing];
    int task_s[kRing];
    uint32_t tmem_base;
    int abort;
    int roles_done;
    int total_tiles, total_panels, lag;
    unsigned total_units;
    unsigned sub_req;   // producer -> subscriber: (sequence << 16) | (kind << 15) | index, see the subscriber warp
    unsigned seen_s[kMaxPanels / 32];  // return flags (expert, panel) some warp of this block has seen up

    int le_start[kMaxLocal + 1];             // first panel of every local expert
    int seg_prefix[2 * kMaxLocal + 1];       // tiles before every segment of the tile order
    __align__(16) float bias_s[4][256];
    __align__(16) uint4 stage_s[4][32 * 8];
    uint2 panel_s[kMaxPanels];               // {row_base, rows | le << 8 | src << 16}
    int cnt_s[kMaxCells];                    // routed rows per (source, local expert) cell
    int poff_s[kMaxCells + 1];               // first panel of every cell, cells in plan order
    unsigned prefix_s[kMaxCells + 1];        // dispatch units before every expert, sending order
    int own_s[kMaxCells];                    // routed rows of this rank's tokens per expert, sending order
    unsigned char ready_s[kMaxCells];        // producer's memo: the cell's data flag has been seen
    unsigned char pair_ready_s[kMaxPanels];  // producer's memo: the pair's GEMM1 tiles are done
};
static_assert(sizeof(Control) <= kCtlBytes, "control block must fit the shared memory set aside for it");

struct Args {
    const void* tokens;      // [S,H] this rank's activations
    const void* b1;          // [nLx,I]
    const void* b2;          // [nLx,H]
    void* y1;                // [cells*pEC][I] GEMM1 results, this rank's memory
    void* out;               // [S,H]
    void* probs;             // [S,PX] element-rounded gate probabilities
    int* topk;               // [S,K]
    int* slots;              // [S,K]
    float* mcw;              // [S]
    int* cell_tokens;        // [E,pEC]
    unsigned* counts;        // [E] unclamped counts of this rank's tokens
    PeerTable peers;
    ArenaLayout lay;
    Counters* ctr;           // [2]
    DeviceStatus* status;
    long long* stamps;       // optional [grid][kStampSlots] global-timer values, or null
    long long* stalls;       // optional [grid][kStallSlots] cycles the roles of the tile stream spent waiting, or null
    int debug;               // tuning switches (KLEOS_FLOW_DEBUG): 1 = combine only after the last tile, 2 = static tile split
    long long wait_cycles;
    int S, H, I, E, K, PX, EC, pEC, nLx, rank, world;
    uint32_t epoch;
    int suppress;            // test hook: no return flags (the combine's bounded wait then runs out)
    int sub;                 // 64-wide K slices per pipeline stage: 1 or 2
    int unit_rows;           // rows per dispatch unit, 1..kUnitRows: bounds the stores a warp has in flight
    // routing inside the kernel (fuse_route != 0): the kernel then WRITES probs, topk, slots, mcw,
    // cell_tokens and counts before it reads them
    int fuse_route;
    int route_only;          // with fuse_route: leave after the routing phase (router of the separate launches)
    const void* Wg;          // [PX,H] gate weight, row e = expert e
    const float* gate_bias;  // [E]
    int* tile_hist;          // [S/128][E] per-tile histogram of the chosen experts
    float tie_eps;
};

struct Tile {
    int phase;    // 0: GEMM1, 1: GEMM2
    int le, nt;
    int panel0;   // first panel of the pair
    int n_left;   // panels from panel0 to the end of the local expert (1: the pair has no second panel)
};

__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_relaxed_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Release fences of the publication patterns below.  (__threadfence() and __threadfence_system()
// are the sequentially consistent forms, which cost several times as much under memory load.)
__device__ __forceinline__ void fence_release_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ void fence_release_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

__device__ __forceinline__ bool mbar_try_wait_cluster(unsigned long long* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(tc::smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

// Segment s of the tile order for n local experts and lag D (1 <= D <= n):
//   G1(0) .. G1(D-1),  then G1(i), G2(i-D) for i = D .. n-1,  then G2(n-D) .. G2(n-1).
// A GEMM2 segment therefore follows the GEMM1 segment it depends on by D GEMM1 segments and D-1
// GEMM2 segments; D is chosen in the plan so that this distance exceeds the number of tiles in
// flight (one per block pair): by the time a GEMM2 tile is claimed, the GEMM1 tiles of its row
// panels have normally been finished and nobody waits.
__host__ __device__ __forceinline__ void segment_of(int s, int n, int D, int* phase, int* le) {
    if (s < D) {
        *phase = 0;
        *le = s;
    } else if (s < 2 * n - D) {
        const int r = s - D;
        *phase = r & 1;
        *le = (r & 1) ? (r >> 1) : D + (r >> 1);
    } else {
        *phase = 1;
        *le = s - n;  // n - D + (s - (2n - D))
    }
}

// Exclusive prefix sum of f(0) .. f(n-1), n <= 256, by one warp: out[i] = f(0) + .. + f(i-1) for
// i = 0 .. n.  Returns the total in every lane.
template <typename F, typename O>
__device__ __forceinline__ int warp_prefix(F f, O* out, int n, int lane) {
    int v[8], local = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int i = lane * 8 + k;
        v[k] = i < n ? f(i) : 0;
        local += v[k];
    }
    int incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    int run = incl - local;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int i = lane * 8 + k;
        if (i < n) out[i] = (O)run;
        run += v[k];
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    if (lane == 0) out[n] = (O)total;
    return total;
}

__device__ __forceinline__ Tile decode_tile(const Control* ctl, int t, int nLx) {
    int lo = 0, hi = 2 * nLx;  // last segment whose first tile is <= t
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (ctl->seg_prefix[mid] <= t) lo = mid; else hi = mid;
    }
    Tile ti;
    segment_of(lo, nLx, ctl->lag, &ti.phase, &ti.le);
    const int r = t - ctl->seg_prefix[lo];
    const int p0 = ctl->le_start[ti.le], np = ctl->le_start[ti.le + 1] - p0;
    const int npair = (np + 1) >> 1;
    ti.nt = r / npair;
    const int pi = r - ti.nt * npair;
    ti.panel0 = p0 + 2 * pi;
    ti.n_left = np - 2 * pi;
    return ti;
}

__device__ __forceinline__ PanelEntry panel_of(const Control* ctl, int i) {
    const uint2 e = ctl->panel_s[i];
    return PanelEntry{(int)e.x, (int)(e.y & 0xff), (int)((e.y >> 8) & 0xff), (int)(e.y >> 16)};
}

// One token's output row: sum over its kept choices of Element(p) * Element(y2 / mCw)
// (reference processor.cuh:110-168; with k == 1 a plain copy, :170-204), zeros when every choice
// was dropped.  The whole warp works on the row, 16 bytes per lane and step.
template <typename T, int KT>
__device__ __forceinline__ void combine_row(const T* const* yrow, const float* p, float w, T* orow,
                                            int chunks, int lane, int K) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int KMAX = KT > 0 ? KT : kMaxTopK;
    constexpr int UNR = KT > 0 && KT <= 2 ? 8 : 1;  // 16-byte loads in flight per lane and choice
    using P2 = Pack2<T>;
    const float inv_w = 1.f / w;
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
            *reinterpret_cast<uint4*>(orow + (size_t)c * VEC) = *reinterpret_cast<const uint4*>(acc2);
        }
    }
}

// Read-back of this warp's 32 accumulator rows of one 256-column tile: bias, activation, rounding
// to the element type, and stores of rows_w rows (whole 128-byte lines per row segment, through a
// swizzled shared-memory transpose).  The accumulator is handed back to the MMA issuer as soon
// as its last column is in registers.
template <typename TE, int kEpi>
__device__ __forceinline__ void read_back(uint32_t taddr, const float* bias_q, uint4* stg, TE* obase,
                                          size_t ld, int rows_w, int n0, int N, int lane,
                                          uint32_t acc_empty_leader) {
    using namespace tc;
    using TE2 = typename Pack2<TE>::type;
    uint32_t r[2][32];
    tmem_ld_32x32(taddr, r[0]);
#pragma unroll
    for (int c = 0; c < BN / 32; ++c) {
        tmem_ld_wait();
        if (c + 1 < BN / 32) {
            tmem_ld_32x32(taddr + (c + 1) * 32, r[(c + 1) & 1]);
        } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
        }
        const uint32_t* rc = r[c & 1];
        const float4* bq = reinterpret_cast<const float4*>(bias_q + c * 32);
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float4 bf = bq[j >> 1];
            float v0 = __uint_as_float(rc[2 * j]) + ((j & 1) ? bf.z : bf.x);
            float v1 = __uint_as_float(rc[2 * j + 1]) + ((j & 1) ? bf.w : bf.y);
            if constexpr (kEpi == 0) {
                v0 = fmaxf(v0, 0.f);
                v1 = fmaxf(v1, 0.f);
            } else if constexpr (kEpi == 1) {
                v0 = apply_act(v0, 1);
                v1 = apply_act(v1, 1);
            }
            const TE2 h = Pack2<TE>::from_f2(v0, v1);
            packed[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int ch = (c & 1) * 4 + j;
            stg[lane * 8 + (ch ^ (lane & 7))] =
                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
        }
        if (c & 1) {
            __syncwarp();
            const int col0 = (c - 1) * 32;
            if (n0 + col0 < N) {
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int rr = it * 4 + (lane >> 3), ch = lane & 7;
                    const uint4 v = stg[rr * 8 + (ch ^ (rr & 7))];
                    if (rr < rows_w) *reinterpret_cast<uint4*>(obase + (size_t)rr * ld + col0 + ch * 8) = v;
                }
            }
            __syncwarp();
        }
    }
}


// 16-bit element through L2 (values another block of this kernel may have written)
template <typename T>
__device__ __forceinline__ float ld_cg_elem(const T* p) {
    unsigned short raw;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(raw) : "l"(p));
    return Elem<T>::to_f(*reinterpret_cast<const T*>(&raw));
}

// fp64 dot product of one token row and one gate-weight row, by the whole warp.
template <typename T>
__device__ __forceinline__ double warp_dot64(const T* x, const T* w, int H, int lane) {
    constexpr int VEC = 16 / sizeof(T);
    double s = 0.0;
#pragma unroll 4
    for (int h = lane * VEC; h < H; h += 32 * VEC) {
        const uint4 xr = __ldg(reinterpret_cast<const uint4*>(x + h));
        const uint4 wr = __ldg(reinterpret_cast<const uint4*>(w + h));
        const T* xv = reinterpret_cast<const T*>(&xr);
        const T* wv = reinterpret_cast<const T*>(&wr);
#pragma unroll
        for (int q = 0; q < VEC; ++q) s += (double)Elem<T>::to_f(xv[q]) * (double)Elem<T>::to_f(wv[q]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    return s;
}

}  // namespace flow

// kAct: the expert's activation (0 ReLU, 1 GELU); KT: compile-time top-k of the combine (0 = read
// it from the arguments).  Args::sub = 64-wide K slices per pipeline stage (1: six shallow stages,
// 2: three deep ones, see gemm_tc2.cuh).
template <typename TE, int kAct, int KT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(flow::kThreads, 1)
moe_flow_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w1,
                const __grid_constant__ CUtensorMap map_y1, const __grid_constant__ CUtensorMap map_w2,
                const __grid_constant__ CUtensorMap map_act, const __grid_constant__ CUtensorMap map_wg,
                flow::Args a) {
    using namespace tc;
    using namespace flow;
    const int SUB = a.sub, NST = kSlices / SUB, STAGE_BYTES = SUB * SLICE_BYTES;
    constexpr uint32_t kInstrDesc = make_instr_desc_16b(2 * BM, BN, Pack2<TE>::kMmaFormat);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    Control* ctl = reinterpret_cast<Control*>(tiles + kSlices * SLICE_BYTES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t cta_rank = cluster_ctarank();
    const bool leader = cta_rank == 0;
    volatile int* abort_flag = &ctl->abort;
    Counters* ctr = a.ctr + (a.epoch & 1u);
    const long long budget = a.wait_cycles;
    long long* stamp = a.stamps ? a.stamps + (size_t)blockIdx.x * kStampSlots : nullptr;
    if (stamp && tid == 0) stamp[kStart] = global_ns();
    long long* stall = a.stalls ? a.stalls + (size_t)blockIdx.x * kStallSlots : nullptr;
    // waits of the tile stream, timed only when the caller asked for the counters
    auto timed_wait = [&](unsigned long long* bar, uint32_t parity, long long* acc) -> bool {
        if (!stall) return mbar_wait(bar, parity, budget, abort_flag);
        const long long c0 = clock64();
        const bool ok = mbar_wait(bar, parity, budget, abort_flag);
        *acc += clock64() - c0;
        return ok;
    };

    // Giving up: remember where, stop this block and, through the rank's abort word that every
    // block's monitor warp mirrors, all others.
    auto give_up = [&](int where, int detail) {
        report_error(a.status, where, detail, (int)a.epoch);
        *abort_flag = 1;
        atomicExch(&ctr->abort_all, 1u);
    };

    if (tid == 0) {
        for (int s = 0; s < kSlices; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], 8);
        }
        for (int r = 0; r < kRing; ++r) mbar_init(&ctl->task_full[r], 1);
        ctl->abort = 0;
        ctl->roles_done = 0;
        ctl->sub_req = 0;
        for (int i = 0; i < kMaxPanels / 32; ++i) ctl->seen_s[i] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&ctl->tmem_base)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    if (blockIdx.x == 0) {
        // the forward after this one finds its copy of the scheduler state cleared
        unsigned* nxt = reinterpret_cast<unsigned*>(a.ctr + ((a.epoch + 1u) & 1u));
        for (int i = tid; i < (int)(sizeof(Counters) / sizeof(unsigned)); i += kThreads) nxt[i] = 0u;
    }

    // What the routing phase leaves behind for the tile stream: how many K slices and how many
    // accumulators this block pair has pushed through the shared pipeline (barrier phases and
    // the accumulator in turn continue from there).  The routing phase always runs the six
    // 32 KiB slices as six stages, whatever stage depth the tile stream uses afterwards.
    uint32_t route_slices = 0, route_tiles = 0;

    if (a.fuse_route) {
        // ================================================================== routing phase
        tc_fence_before();
        __syncthreads();
        cluster_sync_all();  // both blocks' barriers exist before anything remote touches them
        tc_fence_after();
        if (stamp && tid == 0) stamp[kRouteBegin] = global_ns();
        const uint32_t tmem_r = ctl->tmem_base;
        const int n_clusters = (int)gridDim.x >> 1, cluster_id = (int)blockIdx.x >> 1;
        const int n_rt = (a.S + 2 * BM - 1) / (2 * BM);  // gate tiles of 256 tokens (128 per block)
        const int KSr = a.H / BK;
        route_tiles = n_rt > cluster_id ? (uint32_t)((n_rt - cluster_id + n_clusters - 1) / n_clusters) : 0u;
        route_slices = route_tiles * (uint32_t)KSr;
        const uint32_t b_bytes = (uint32_t)(a.PX / 2) * BK * 2;  // this block's half of the gate-weight slice
        float* bias_r = &ctl->bias_s[0][0];  // logit bias of every expert (E <= 256 floats)
        int* hist_s = ctl->cnt_s;            // this block's 128-token histogram (E <= 256 ints)
        for (int e = tid; e < kMaxCells; e += kThreads) {
            bias_r[e] = e < a.E ? a.gate_bias[e] : 0.f;
            hist_s[e] = 0;
        }
        __syncthreads();
        if (warp == 0) {
            if (lane == 0) {
                uint32_t it = 0;
                for (int rt = cluster_id; rt < n_rt && !*abort_flag; rt += n_clusters) {
                    for (int kb = 0; kb < KSr; ++kb, ++it) {
                        const int s = it % kSlices;
                        const uint32_t ph = (it / kSlices) & 1;
                        if (!mbar_wait(&ctl->empty[s], ph ^ 1, budget, abort_flag)) {
                            if (!*abort_flag) give_up(KLEOS_AT_GEMM_PRODUCER, -100 - rt);
                            break;
                        }
                        if (leader) mbar_expect_tx(&ctl->full[s], 2 * (A_STAGE_BYTES + b_bytes));
                        const uint32_t full_leader = map_to_cta(smem_u32(&ctl->full[s]), 0);
                        uint8_t* sa = tiles + s * SLICE_BYTES;
                        tma_load_2d_pair(sa, &map_act, kb * BK, rt * 2 * BM + (int)cta_rank * BM, full_leader);
                        tma_load_2d_pair(sa + A_STAGE_BYTES, &map_wg, kb * BK, (int)cta_rank * (a.PX / 2),
                                         full_leader);
                    }
                }
            }
            __syncwarp();
        } else if (warp == 1) {
            if (leader && lane == 0) {
                const uint32_t idesc = make_instr_desc_16b(2 * BM, a.PX, Pack2<TE>::kMmaFormat);
                uint32_t it = 0, tn = 0;
                for (int rt = cluster_id; rt < n_rt && !*abort_flag; rt += n_clusters, ++tn) {
                    const uint32_t buf = tn & 1, use = tn >> 1;
                    if (!mbar_wait(&ctl->acc_empty[buf], (use & 1) ^ 1, budget, abort_flag)) {
                        if (!*abort_flag) give_up(KLEOS_AT_GEMM_MMA, -100 - rt);
                        break;
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_r + buf * BN;
                    bool ok = true;
                    for (int kb = 0; kb < KSr; ++kb, ++it) {
                        const int s = it % kSlices;
                        const uint32_t ph = (it / kSlices) & 1;
                        if (!mbar_wait(&ctl->full[s], ph, budget, abort_flag)) {
                            if (!*abort_flag) give_up(KLEOS_AT_GEMM_MMA, -100 - rt);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        if (stamp && it == 0) stamp[kFirstOperands] = global_ns();
                        const uint32_t sa = smem_u32(tiles + s * SLICE_BYTES);
                        const uint64_t da = make_smem_desc(sa);
                        const uint64_t db = make_smem_desc(sa + A_STAGE_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            umma_bf16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                        const uint32_t e_local = smem_u32(&ctl->empty[s]);
                        umma_commit_pair(map_to_cta(e_local, 0));
                        umma_commit_pair(map_to_cta(e_local, 1));
                    }
                    if (!ok) break;
                    const uint32_t f_local = smem_u32(&ctl->acc_full[buf]);
                    umma_commit_pair(map_to_cta(f_local, 0));
                    umma_commit_pair(map_to_cta(f_local, 1));
                }
            }
            __syncwarp();
        } else if (warp >= 4 && warp < 8) {
            // One thread per token: the token's logit row is this thread's tensor-memory lane.
            // Selection rules are the reference gate's (moe/gate.cuh:556-584 softmax over the E real
            // experts, :654-670 k rounds of arg-max with ties to the lowest id, :669 mCw): a single
            // ascending pass keeps the K+1 largest logits in order (strict '>' on insertion keeps
            // the lower id in front), a second pass sums the exponentials, a third writes the
            // probabilities.  Tensor memory is simply read three times.
            constexpr int KC = KT > 0 ? KT : kMaxTopK;
            const int q = warp - 4;
            const int K = KT > 0 ? KT : a.K;
            const int chunks = a.PX / 32;
            const TE* A = static_cast<const TE*>(a.tokens);
            const TE* Wg = static_cast<const TE*>(a.Wg);
            TE* probs = static_cast<TE*>(a.probs);
            // per-warp scratch for the near-tie re-evaluation (the read-back staging tile, unused here)
            unsigned char* scratch = reinterpret_cast<unsigned char*>(ctl->stage_s[q]);
            short* band_id = reinterpret_cast<short*>(scratch);           // [<= 256]
            float* band_l = reinterpret_cast<float*>(scratch + 512);      // fp32 logit of each member
            double* band_v = reinterpret_cast<double*>(scratch + 1536);   // fp64 logit of each member
            short* sel_id = reinterpret_cast<short*>(scratch + 3584);     // [<= 8] re-selected ids
            float* sel_l = reinterpret_cast<float*>(scratch + 3616);      // and their fp32 logits
            uint32_t tn = 0;
            for (int rt = cluster_id; rt < n_rt; rt += n_clusters, ++tn) {
                const uint32_t buf = tn & 1, use = tn >> 1;
                if (!mbar_wait(&ctl->acc_full[buf], use & 1, budget, abort_flag)) {
                    if (!*abort_flag && lane == 0) give_up(KLEOS_AT_GEMM_EPILOGUE, -100 - rt);
                    break;
                }
                tc_fence_after();
                if (stamp && q == 0 && lane == 0) stamp[kGateAcc] = global_ns();
                const int row_w = rt * 2 * BM + (int)cta_rank * BM + q * 32;  // this warp's first token
                const int row = row_w + lane;
                const bool valid = row < a.S;
                const uint32_t taddr = tmem_r + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
                float val[KC + 1];
                int idx[KC + 1];
#pragma unroll
                for (int j = 0; j <= KC; ++j) {
                    val[j] = -INFINITY;
                    idx[j] = 0;
                }
#pragma unroll 1
                for (int c = 0; c < chunks; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) {
                        const int e = c * 32 + jj;
                        if (e < a.E) {
                            float x = __uint_as_float(v[jj]) + bias_r[e];
                            int id = e;
#pragma unroll
                            for (int j = 0; j <= KC; ++j) {
                                if (j <= K && x > val[j]) {
                                    const float tv = val[j];
                                    const int ti = idx[j];
                                    val[j] = x;
                                    idx[j] = id;
                                    x = tv;
                                    id = ti;
                                }
                            }
                        }
                    }
                }
                if (stamp && q == 0 && lane == 0) stamp[kTopkPass1] = global_ns();
                const float m = val[0];
                float d = 0.f;
#pragma unroll 1
                for (int c = 0; c < chunks; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) {
                        const int e = c * 32 + jj;
                        if (e < a.E) d += __expf(__uint_as_float(v[jj]) + bias_r[e] - m);
                    }
                }
                const float inv = 1.f / d;
                if (stamp && q == 0 && lane == 0) stamp[kTopkDone] = global_ns();
                float kth = 0.f, next = -INFINITY;
#pragma unroll
                for (int j = 0; j <= KC; ++j) {
                    if (j == K - 1) kth = val[j];
                    if (j == K) next = val[j];
                }
                // Near-ties: when the k-th and (k+1)-th logits are closer than fp32 summation error
                // can move them, the experts within that distance of the k-th are re-evaluated in
                // fp64 and the open places of the top-k are filled from them (larger value first,
                // equal values to the lower id).  Experts further above are in the set and experts
                // further below are out of it whatever the summation order, so this equals a
                // selection on fp64 logits.
                const float eps = a.tie_eps * fmaxf(1.f, fabsf(kth));
                const bool flag = valid && K < a.E && (kth - next) < eps;
                unsigned flagged = __ballot_sync(0xffffffffu, flag);
                while (flagged) {
                    const int src = __ffs(flagged) - 1;
                    flagged &= flagged - 1;
                    int nb = 0;
#pragma unroll 1
                    for (int c = 0; c < chunks; ++c) {
                        uint32_t v[32];
                        tmem_ld_32x32(taddr + c * 32, v);
                        tmem_ld_wait();
                        if (lane == src) {
#pragma unroll
                            for (int jj = 0; jj < 32; ++jj) {
                                const int e = c * 32 + jj;
                                const float x = __uint_as_float(v[jj]) + bias_r[e < a.E ? e : 0];
                                if (e < a.E && fabsf(x - kth) <= eps) {
                                    band_id[nb] = (short)e;
                                    band_l[nb] = x;
                                    ++nb;
                                }
                            }
                        }
                    }
                    nb = __shfl_sync(0xffffffffu, nb, src);
                    __syncwarp();
                    const TE* xrow = A + (size_t)(row_w + src) * a.H;
                    for (int b = 0; b < nb; ++b) {
                        const int e = band_id[b];
                        const double sdot = warp_dot64<TE>(xrow, Wg + (size_t)e * a.H, a.H, lane);
                        if (lane == 0) band_v[b] = sdot + (double)bias_r[e];
                    }
                    __syncwarp();
                    if (lane == src) {
                        int c_in = 0;
#pragma unroll
                        for (int j = 0; j < KC; ++j)
                            if (j < K && val[j] > kth + eps) ++c_in;
                        const int need = K - c_in;
                        for (int r = 0; r < need; ++r) {
                            int best = -1;
                            for (int b = 0; b < nb; ++b) {
                                if (band_id[b] < 0) continue;
                                if (best < 0 || band_v[b] > band_v[best] ||
                                    (band_v[b] == band_v[best] && band_id[b] < band_id[best]))
                                    best = b;
                            }
                            sel_id[r] = band_id[best];
                            sel_l[r] = band_l[best];
                            band_id[best] = -1;
                        }
#pragma unroll
                        for (int j = 0; j < KC; ++j)
                            if (j < K && j >= c_in) {
                                idx[j] = sel_id[j - c_in];
                                val[j] = sel_l[j - c_in];
                            }
                    }
                    __syncwarp();
                }
                float wsum = 0.f;
#pragma unroll
                for (int j = 0; j < KC; ++j)
                    if (j < K) wsum += __expf(val[j] - m) * inv;
                // probabilities, padding columns zero, one 16-byte store per eight experts
#pragma unroll 1
                for (int c = 0; c < chunks; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + c * 32, v);
                    tmem_ld_wait();
                    if (c + 1 == chunks) {
                        // last read of this accumulator: hand it back to the MMA issuer
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->acc_empty[buf]), 0));
                    }
                    if (valid) {
                        using TE2 = typename Pack2<TE>::type;
#pragma unroll
                        for (int g8 = 0; g8 < 4; ++g8) {
                            uint32_t packed[4];
#pragma unroll
                            for (int h2 = 0; h2 < 4; ++h2) {
                                const int jj = g8 * 8 + h2 * 2, e = c * 32 + jj;
                                const float p0 = e < a.E ? __expf(__uint_as_float(v[jj]) + bias_r[e] - m) * inv : 0.f;
                                const float p1 = e + 1 < a.E ? __expf(__uint_as_float(v[jj + 1]) + bias_r[e + 1] - m) * inv : 0.f;
                                const TE2 h = Pack2<TE>::from_f2(p0, p1);
                                packed[h2] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                            *reinterpret_cast<uint4*>(probs + (size_t)row * a.PX + c * 32 + g8 * 8) =
                                make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        }
                    }
                }
                if (stamp && q == 0 && lane == 0) stamp[kProbsDone] = global_ns();
                if (valid) {
#pragma unroll
                    for (int j = 0; j < KC; ++j)
                        if (j < K) {
                            a.topk[(size_t)row * K + j] = idx[j];
                            atomicAdd(&hist_s[idx[j]], 1);
                        }
                    a.mcw[row] = wsum;
                }
                // the four read-back warps share the histogram of the block's 128 tokens
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int tile = rt * 2 + (int)cta_rank;
                if (tile * BM < a.S)
                    for (int e = tid - 128; e < a.E; e += 128) a.tile_hist[(size_t)tile * a.E + e] = hist_s[e];
                asm volatile("bar.sync 1, 128;" ::: "memory");
                for (int e = tid - 128; e < a.E; e += 128) hist_s[e] = 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (stamp && q == 0 && lane == 0) stamp[kGateDone] = global_ns();
            }
        }

        // -------------------------------------------------------------- grid barrier, slots, grid barrier
        auto grid_barrier = [&](int which) {
            __syncthreads();
            if (tid == 0) {
                fence_release_gpu();  // cumulative over the block's writes observed through the barrier
                atomicAdd(&ctr->grid_bar[which], 1u);
                const long long t0 = clock64();
                while (ld_acquire_gpu(&ctr->grid_bar[which]) < gridDim.x) {
                    __nanosleep(100);
                    if (ld_relaxed_gpu(&ctr->abort_all)) {
                        *abort_flag = 1;
                        break;
                    }
                    if (clock64() - t0 > budget) {
                        give_up(KLEOS_AT_GRID_BARRIER, which);
                        break;
                    }
                }
            }
            __syncthreads();
        };
        if (*abort_flag) atomicExch(&ctr->abort_all, 1u);
        grid_barrier(0);
        if (stamp && tid == 0) stamp[kRouted] = global_ns();
        // (after a failed wait the rest of the kernel still runs through its barriers, with the
        // abort flag up, so that both blocks of a pair meet at the same cluster barriers)
        if (!*abort_flag) {
            // Slots in ascending token order (the reference hands them out in atomicAdd arrival
            // order, moe/gate.cuh:689-718): base slot of every expert for a tile of 128 tokens = sum of
            // the earlier tiles' histograms, then each token's rank inside the tile; the sum over all
            // tiles is the expert's count, published with one count flag per expert to its owner rank.
            int* base = ctl->poff_s;                                // [E]
            int* part = ctl->own_s;                                 // [256]
            int (*wcount)[256] = reinterpret_cast<int (*)[256]>(ctl->stage_s);  // [8][256]
            const int n_tiles = a.S / BM;
            int ep = 1;
            while (ep < a.E) ep <<= 1;
            // base[e] = tokens the tiles before `upto` sent to expert e: 256 / ep threads per expert
            // share the tiles, each with sixteen loads in flight at a time (the histograms sit in
            // L2, and one load after the other would cost a round trip per tile)
            auto sum_tiles_before = [&](int upto) {
                const int groups = 256 / ep;
                const int e = tid % ep, grp = tid / ep;
                int run = 0;
                if (tid < 256 && e < a.E) {
                    for (int t0 = grp; t0 < upto; t0 += 16 * groups) {
                        int v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int t = t0 + j * groups;
                            v[j] = t < upto ? __ldcg(a.tile_hist + (size_t)t * a.E + e) : 0;
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) run += v[j];
                    }
                }
                if (tid < 256) part[tid] = run;
                __syncthreads();
                if (tid < a.E) {
                    int sum = 0;
                    for (int gi = 0; gi < groups; ++gi) sum += part[gi * ep + tid];
                    base[tid] = sum;
                }
                __syncthreads();
            };
            // totals of every expert: unclamped count for this rank, clamped count to the owner
            auto publish_counts = [&](int last_tile_too) {
                for (int e = tid; e < a.E; e += kThreads) {
                    int total = base[e];
                    if (last_tile_too) total += __ldcg(a.tile_hist + (size_t)(n_tiles - 1) * a.E + e);
                    a.counts[e] = (unsigned)total;
                    const int owner = e / a.nLx, le = e - owner * a.nLx;
                    st_release_sys(reinterpret_cast<unsigned long long*>(a.peers.arena[owner] + a.lay.cflag) +
                                       ((size_t)a.rank * a.nLx + le),
                                   make_flag(a.epoch, (unsigned)min(total, a.EC)));
                }
            };
            // When the last block pair routed no tile it has nothing to do here: its second block
            // adds up ALL tiles and publishes the counts, off the path of the blocks that write
            // slots.  Otherwise the block of the last tile does it on top of its own work.
            const bool spare = n_rt < n_clusters;
            if (spare && blockIdx.x == gridDim.x - 1) {
                sum_tiles_before(n_tiles);
                publish_counts(0);
            }
            for (int rt = cluster_id; rt < n_rt; rt += n_clusters) {
                const int tile = rt * 2 + (int)cta_rank;
                if (tile >= n_tiles) break;  // block-uniform
                const int tok0 = tile * BM;
                for (int i = tid; i < 8 * 256; i += kThreads) (&wcount[0][0])[i] = 0;
                sum_tiles_before(tile);
                if (stamp && tid == 0) stamp[kSlotBase] = global_ns();
                if (!spare && tile == n_tiles - 1) publish_counts(1);
                const int n_own = min(BM, a.S - tok0) * a.K;
                for (int i0 = 0; i0 < n_own; i0 += 256) {
                    const int i = i0 + tid;
                    const bool worker = tid < 256;
                    int e = -1, before = 0;
                    bool lead = false;
                    if (worker) {
                        e = i < n_own ? __ldcg(a.topk + (size_t)tok0 * a.K + i) : -1;
                        const unsigned peers = __match_any_sync(0xffffffffu, e);
                        before = __popc(peers & ((1u << lane) - 1u));
                        lead = e >= 0 && before == 0;
                        if (lead) wcount[warp][e] = __popc(peers);
                    }
                    __syncthreads();
                    if (worker && e >= 0) {
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
                    if (lead) {
                        atomicAdd(&base[e], wcount[warp][e]);
                        wcount[warp][e] = 0;
                    }
                    __syncthreads();
                }
            }
        }
        if (stamp && tid == 0) stamp[kSlotsDone] = global_ns();
        grid_barrier(1);
        if (stamp && tid == 0) stamp[kSlotted] = global_ns();
    }
    if (a.route_only) {
        // The router alone (the separate-launch arrangement uses this kernel as its router: one
        // launch instead of gate, near-tie, histogram and slot kernels).  Same teardown as below.
        tc_fence_before();
        __syncthreads();
        cluster_sync_all();
        if (warp == 2) {
            tc_fence_after();
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(ctl->tmem_base),
                         "r"(TMEM_COLS)
                         : "memory");
        }
        if (stamp && tid == 0) stamp[kEnd] = global_ns();
        return;
    }

    // ------------------------------------------------------------------ plan (every block, same result)
    // Routed count of every (source, local expert) cell, published by the sources' routers
    // (reference: the first-stage signal carries the count, types.cuh:300-317); then the panel
    // list, local expert by local expert, sources in the order their rows are sent; then the
    // tile order.  Replaces the subscriber's decode of initial packets into 128-byte tasks
    // (os/subscriber.cuh:56-185, os/packet.cuh:304-398) and the scheduler's worst-case task bound
    // (os/os.cuh:104-105).
    const int cells = a.world * a.nLx;
    const int NT1 = (a.I + BN - 1) / BN, NT2 = (a.H + BN - 1) / BN;
    const bool transport = warp >= 8;
    // barrier among the eight planning warps (the transport warps are already moving rows)
    auto planners_sync = [&]() { asm volatile("bar.sync 2, 256;" ::: "memory"); };
    {
        for (int c = tid; c < kMaxCells; c += kThreads) ctl->ready_s[c] = 0;
        for (int c = tid; c < kMaxPanels; c += kThreads) ctl->pair_ready_s[c] = 0;
        // sending order of this rank's rows: local expert index first, owners rotated so that at
        // any moment the source ranks write to different owners
        for (int i = tid; i < a.E; i += kThreads) {
            const int le = i / a.world, owner = (a.rank + 1 + i % a.world) % a.world;
            ctl->own_s[i] = (int)min(__ldcg(a.counts + owner * a.nLx + le), (unsigned)a.EC);
        }
        __syncthreads();
        if (warp == 0) {
            // dispatch units before every expert, in sending order
            const int total = warp_prefix([&](int i) { return (ctl->own_s[i] + a.unit_rows - 1) / a.unit_rows; },
                                          ctl->prefix_s, a.E, lane);
            if (lane == 0) ctl->total_units = (unsigned)total;
        }
        __syncthreads();
    }
    if (transport) {
        // The transport warps know all they need (what this rank sends where) and start moving rows
        // while the other warps wait for the counts of the other ranks and build the tile plan.
        // They sign the cluster barrier that ends the plan now and collect it before the teardown.
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    } else {
        const unsigned long long* cflag =
            reinterpret_cast<const unsigned long long*>(a.peers.arena[a.rank] + a.lay.cflag);
        // (relaxed polls: the count travels inside the flag word itself, nothing else is read on
        // the strength of it, and an acquiring load costs a fence that waits for this SM's stores in
        // flight -- the transport warps are already streaming rows to the peers)
        for (int c = tid; c < cells; c += 256) {
            unsigned long long v = 0;
            const long long t0 = clock64();
            for (;;) {
                v = ld_relaxed_sys(cflag + c);
                if ((uint32_t)(v >> 32) == a.epoch) break;
                if (clock64() - t0 > budget) {
                    give_up(KLEOS_AT_PLAN_WAIT, c);
                    v = 0;
                    break;
                }
                __nanosleep(64);
            }
            ctl->cnt_s[c] = (int)min((unsigned)(v & 0xffffffffu), (unsigned)a.pEC);
        }
        planners_sync();
        if (warp == 1) {
            // panels before every cell, cells in plan order o = le * world + j
            const int n_panels = warp_prefix(
                [&](int o) {
                    const int le = o / a.world, j = o - le * a.world;
                    return (ctl->cnt_s[((a.rank + 1 + j) % a.world) * a.nLx + le] + kTileM - 1) / kTileM;
                },
                ctl->poff_s, cells, lane);
            __syncwarp();
            for (int le = lane; le <= a.nLx; le += 32) ctl->le_start[le] = le < a.nLx ? ctl->poff_s[le * a.world] : n_panels;
            __syncwarp();
            // lag of the tile order: enough segments between a GEMM1 segment and its GEMM2 segment
            // to cover two and a half times the tiles in flight (a tile is published up to one tile
            // time after it is finished)
            int pairs = 0;
            for (int le = lane; le < a.nLx; le += 32)
                pairs += (ctl->le_start[le + 1] - ctl->le_start[le] + 1) >> 1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) pairs += __shfl_xor_sync(0xffffffffu, pairs, o);
            const int t1 = max(1, pairs * NT1 / a.nLx), t2 = max(1, pairs * NT2 / a.nLx);
            const int in_flight = (int)gridDim.x >> 1;
            const int lag = min(a.nLx, max(1, (2 * in_flight + in_flight / 2 + t2 + t1 + t2 - 1) / (t1 + t2)));
            const int n_tiles = warp_prefix(
                [&](int sg) {
                    int phase, le;
                    segment_of(sg, a.nLx, lag, &phase, &le);
                    const int np = ctl->le_start[le + 1] - ctl->le_start[le];
                    return ((np + 1) >> 1) * (phase ? NT2 : NT1);
                },
                ctl->seg_prefix, 2 * a.nLx, lane);
            if (lane == 0) {
                ctl->lag = lag;
                ctl->total_panels = n_panels;
                ctl->total_tiles = n_tiles;
            }
        }
        planners_sync();
        for (int o = tid; o < cells; o += 256) {
            const int le = o / a.world, j = o - le * a.world;
            const int src = (a.rank + 1 + j) % a.world;
            const int c = src * a.nLx + le;
            const int cnt = ctl->cnt_s[c];
            int n = ctl->poff_s[o];
            for (int r = 0; r < cnt && n < kMaxPanels; r += kTileM)  // the host never plans beyond the table
                ctl->panel_s[n++] = make_uint2((unsigned)(c * a.pEC + r),
                                               (unsigned)min(kTileM, cnt - r) | ((unsigned)le << 8) |
                                                   ((unsigned)src << 16));
        }
        if (blockIdx.x == 0) {
            // cells this rank sends nothing to: nothing will complete them, so their data flags
            // go out now (reference os/packet.cuh:240-259)
            for (int i = tid; i < a.E; i += 256)
                if (ctl->own_s[i] == 0) {
                    const int le = i / a.world, owner = (a.rank + 1 + i % a.world) % a.world;
                    st_release_sys(reinterpret_cast<unsigned long long*>(a.peers.arena[owner] + a.lay.xflag) +
                                       ((size_t)a.rank * a.nLx + le),
                                   make_flag(a.epoch, 0u));
                }
            // a rank whose experts received nothing still tells every source that it is done
            if (ctl->total_panels == 0 && tid < a.world && !a.suppress)
                st_release_sys(reinterpret_cast<unsigned long long*>(a.peers.arena[tid] + a.lay.yflag) + a.rank,
                               make_flag(a.epoch, 1u));
        }
        tc_fence_before();
        planners_sync();
        cluster_sync_all();  // both blocks' barriers exist before anything remote touches them
        tc_fence_after();
    }
    const uint32_t tmem_base = ctl->tmem_base;
    const int total_tiles = ctl->total_tiles;
    // Parity of every pipeline barrier at the start of the tile stream, one bit per barrier: the
    // routing phase used barrier s ceil((route_slices - s) / 6) times before.  Producer and issuer
    // each keep their own copy and flip bit s whenever they have used stage s, so the inner
    // loops carry no divisions (they run in ONE thread each, whose instruction latencies add up
    // to the time per stage).
    uint32_t parity0 = 0;
#pragma unroll
    for (int sg = 0; sg < kSlices; ++sg)
        parity0 |= (((route_slices + (uint32_t)(kSlices - 1 - sg)) / (uint32_t)kSlices) & 1u) << sg;
    if (stamp && tid == 0) stamp[kPlanned] = global_ns();

    // The leader's producer claims tiles from the rank's task queue (claim) and hands every claimed
    // index (or -1: no more work) to the roles of both blocks through an eight-entry ring (hand_out).  The ring
    // needs no "empty" signal: the producer is at most one tile ahead of the MMA issuer (six
    // K slices of shared memory), the issuer at most two tiles ahead of the read-back warps (two
    // accumulators), and every role copies its entry into registers before it does anything
    // else, so at most four entries are live at any time.
    unsigned static_claims = 0;
    auto claim = [&]() -> int {  // leader's producer thread only: next tile of the rank's queue, or -1
        if (*abort_flag) return -1;  // (the subscriber mirrors the rank's abort word into this flag)
        if (a.debug & 2) {
            // tuning switch: static split of the same tile order (pair c takes tiles c, c + pairs, ...)
            const unsigned c = (blockIdx.x >> 1) + static_claims++ * (gridDim.x >> 1);
            return c < (unsigned)total_tiles ? (int)c : -1;
        }
        const unsigned c = atomicAdd(&ctr->tile_next, 1u);
        return c < (unsigned)total_tiles ? (int)c : -1;
    };
    auto hand_out = [&](uint32_t i, int t) {  // ... and its publication to the roles of both blocks
        const int slot = i % kRing;
        ctl->task_s[slot] = t;
        st_cluster_u32(map_to_cta(smem_u32(&ctl->task_s[slot]), 1), (uint32_t)t);
        mbar_arrive(&ctl->task_full[slot]);
        mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->task_full[slot]), 1));
    };
    auto take = [&](uint32_t i, int where) -> int {  // every other role
        const int slot = i % kRing;
        const uint32_t parity = (i / kRing) & 1u;
        if (!mbar_try_wait_cluster(&ctl->task_full[slot], parity)) {
            const long long t0 = clock64();
            uint32_t polls = 0;
            while (!mbar_try_wait_cluster(&ctl->task_full[slot], parity)) {
                __nanosleep(40);
                if ((++polls & 31u) == 0) {
                    if (*abort_flag) return -1;
                    if (clock64() - t0 > budget) {
                        give_up(where, -2 - (int)i);
                        return -1;
                    }
                }
            }
        }
        return *reinterpret_cast<volatile int*>(&ctl->task_s[slot]);
    };

    // The combine, run by the transport warps once their rows are dispatched and by the read-back
    // warps once the tile stream has ended.
    auto run_combine = [&]() {
        // Tokens are visited in passes: the experts of one rank finish in the order of their local
        // index, so a token's rows are all back once the LAST of its experts (by local index) has
        // returned; pass q takes the tokens whose last expert falls into the q-th part of that
        // order.  An item is (pass, block of eight tokens): the first eight lanes each load one
        // token's choices, slots, gate probabilities and mCw; the warp then takes the block's
        // tokens of this pass one by one, waits (bounded) for the return flags of the token's
        // panels and gathers the rows (reference: the subscriber decodes returned tiles into
        // combine tasks, os/subscriber.cuh:187-332; the sum itself processor.cuh:110-168).
        constexpr int KMAX = KT > 0 ? KT : kMaxTopK;
        const int passes = min(a.nLx, kMaxPasses);
        const int nblk = (a.S + kCombineBlock - 1) / kCombineBlock;
        const unsigned total_items = (unsigned)(passes * nblk);
        const int K = KT > 0 ? KT : a.K;
        const int TCM = a.pEC / kTileM;
        const unsigned long long* ypflag =
            reinterpret_cast<const unsigned long long*>(a.peers.arena[a.rank] + a.lay.ypflag);
        const TE* ycell = reinterpret_cast<const TE*>(a.peers.arena[a.rank] + a.lay.ycell);
        const TE* probs = static_cast<const TE*>(a.probs);
        const int chunks = a.H / (16 / (int)sizeof(TE));
        for (;;) {
            unsigned item = 0;
            if (lane == 0) item = (*abort_flag) ? 0xffffffffu : atomicAdd(&ctr->item_next, 1u);
            item = __shfl_sync(0xffffffffu, item, 0);
            if (item >= total_items) break;
            const int q = (int)item / nblk, b = (int)item - q * nblk;
            const int t_mine = b * kCombineBlock + lane;
            int cls = -1;  // pass in which this lane's token is handled
            int e_m[KMAX], sl_m[KMAX];
            float p_m[KMAX], w_m = 1.f;
#pragma unroll
            for (int j = 0; j < KMAX; ++j) {
                e_m[j] = 0;
                sl_m[j] = kDropped;
                p_m[j] = 0.f;
            }
            if (lane < kCombineBlock && t_mine < a.S) {
                cls = 0;
#pragma unroll
                for (int j = 0; j < KMAX; ++j)
                    if (j < K) {
                        e_m[j] = __ldcg(a.topk + (size_t)t_mine * K + j);
                        sl_m[j] = __ldcg(a.slots + (size_t)t_mine * K + j);
                        if (sl_m[j] != kDropped) cls = max(cls, (e_m[j] % a.nLx) * passes / a.nLx);
                    }
                if (cls == q) {
                    w_m = __ldcg(a.mcw + t_mine);
#pragma unroll
                    for (int j = 0; j < KMAX; ++j)
                        if (j < K) p_m[j] = ld_cg_elem(probs + (size_t)t_mine * a.PX + e_m[j]);
                }
            }
            unsigned todo = __ballot_sync(0xffffffffu, cls == q);
            while (todo) {
                const int src_lane = __ffs(todo) - 1;
                todo &= todo - 1;
                const int t = b * kCombineBlock + src_lane;
                const TE* yrow[KMAX];
                float p[KMAX];
                bool failed = false;
#pragma unroll
                for (int j = 0; j < KMAX; ++j) {
                    const int e = __shfl_sync(0xffffffffu, e_m[j], src_lane);
                    const int sl = __shfl_sync(0xffffffffu, sl_m[j], src_lane);
                    p[j] = __shfl_sync(0xffffffffu, p_m[j], src_lane);
                    yrow[j] = nullptr;
                    if (j < K && sl != kDropped) {
                        yrow[j] = ycell + ((size_t)e * a.pEC + sl) * a.H;
                        if (lane == j) {
                            // a flag another warp of this block has already seen up needs no poll
                            const int f = e * TCM + sl / kTileM;
                            volatile unsigned* word = &ctl->seen_s[f >> 5];
                            if (!((*word >> (f & 31)) & 1u)) {
                                unsigned long long v;
                                if (!wait_flag(ypflag + f, a.epoch, budget, &v)) {
                                    give_up(KLEOS_AT_COMBINE_WAIT, e);
                                    failed = true;
                                } else {
                                    asm volatile("fence.acq_rel.cta;" ::: "memory");
                                    atomicOr(const_cast<unsigned*>(word), 1u << (f & 31));
                                }
                            } else {
                                asm volatile("fence.acq_rel.cta;" ::: "memory");
                            }
                        }
                    }
                }
                const float w = __shfl_sync(0xffffffffu, w_m, src_lane);
                __syncwarp();  // the polling lanes' acquires order every lane's row loads behind the flags
                failed = __any_sync(0xffffffffu, failed) || *abort_flag;
                if (failed) {
                    todo = 0;
                    break;
                }
                combine_row<TE, KT>(yrow, p, w, static_cast<TE*>(a.out) + (size_t)t * a.H, chunks, lane, K);
            }
        }
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both blocks)
        if (lane == 0) {
            asm volatile("fence.proxy.async;" ::: "memory");
            uint32_t par = parity0;
            int s = 0;
            // The leader claims one tile ahead: the round trip of the claim for tile i+1 runs under
            // the loads of tile i.  (Claims stay in order, so the tile a block waits for is still
            // either running or held by a block whose current tile has a smaller index.)  A few
            // K slices into tile i both producers look at tile i+1 and, if it depends on a flag this
            // block has not seen yet, ask the subscriber warp to watch that flag: an acquiring poll
            // of a flag in global memory costs microseconds, which the subscriber spends while the
            // producer keeps loading.
            int ahead = leader ? claim() : -1;
            if (leader) hand_out(0, ahead);
            const long long c_begin = clock64();
            long long w_empty = 0, w_ready = 0;
            const long long w_fence = 0;
            uint32_t req_seq = 0;
            int asked_for = -1;  // tile whose dependency the subscriber has been asked to watch
            int peeked = -1;     // tile already decoded during the tile before it
            Tile peeked_tile{};
            // what tile t waits for: kind 0 = data flag of a cell, kind 1 = GEMM1 counter of a pair
            auto dependency = [&](const Tile& x, int* kind, int* id) -> bool {
                if (x.phase == 0) {
                    const PanelEntry px = panel_of(ctl, x.panel0 + ((int)cta_rank < x.n_left ? (int)cta_rank : 0));
                    *kind = 0;
                    *id = px.src * a.nLx + px.le;
                    return !*reinterpret_cast<volatile unsigned char*>(&ctl->ready_s[*id]);
                }
                *kind = 1;
                *id = x.panel0;
                return !*reinterpret_cast<volatile unsigned char*>(&ctl->pair_ready_s[*id]);
            };
            auto ask = [&](int t_for, int kind, int id) {
                ++req_seq;
                asked_for = t_for;
                *reinterpret_cast<volatile unsigned*>(&ctl->sub_req) = (req_seq << 16) | ((unsigned)kind << 15) | (unsigned)id;
            };
            for (uint32_t i = 0;; ++i) {
                int t;
                if (leader) {
                    t = *abort_flag ? -1 : ahead;  // handed out already (tile 0 above, later ones below)
                    if (t >= 0) ahead = claim();
                } else {
                    t = take(i, KLEOS_AT_GEMM_PRODUCER);
                }
                if (t < 0) break;
                const Tile ti = t == peeked ? peeked_tile : decode_tile(ctl, t, a.nLx);
                // the block without a panel of its own re-reads the first one and discards
                const int my_panel = ti.panel0 + ((int)cta_rank < ti.n_left ? (int)cta_rank : 0);
                const PanelEntry p = panel_of(ctl, my_panel);
                const int N = ti.phase ? a.H : a.I, Kd = ti.phase ? a.I : a.H;
                const int KS = Kd / BK, KB = (KS + SUB - 1) / SUB;
                const int brow = ti.le * N + ti.nt * BN + (int)cta_rank * (BN / 2);
                const CUtensorMap* ma = ti.phase ? &map_y1 : &map_x;
                const CUtensorMap* mb = ti.phase ? &map_w2 : &map_w1;
                bool ok = true;
                const long long c_ready = stall ? clock64() : 0;
                {
                    // GEMM1: rows of the panel's cell may still be on their way from the source rank
                    // (reference: the subscriber polls the first-stage flag, os/subscriber.cuh:107);
                    // GEMM2: starts when all GEMM1 tiles of the panel pair are stored (reference: tQS
                    // counter and notifyNext, processor.cuh:717-729)
                    int kind, id;
                    if (dependency(ti, &kind, &id)) {
                        if (asked_for != t) ask(t, kind, id);
                        volatile unsigned char* memo = kind ? &ctl->pair_ready_s[id] : &ctl->ready_s[id];
                        const long long t0 = clock64();
                        while (!*memo) {
                            __nanosleep(32);
                            if (*abort_flag) {
                                ok = false;
                                break;
                            }
                            if (clock64() - t0 > 2 * budget) {  // the subscriber gives up first
                                give_up(kind ? KLEOS_AT_GEMM_PRODUCER : KLEOS_AT_PLAN_WAIT, 4000 + id);
                                ok = false;
                                break;
                            }
                        }
                        asm volatile("fence.acq_rel.cta;" ::: "memory");
                    }
                    if (stall) w_ready += clock64() - c_ready;
                }
                if (!ok) continue;  // the next claim returns -1 (abort is up) and ends every role
                for (int kb = 0; kb < KB; ++kb) {
                    const uint32_t ph = (par >> s) & 1u;
                    if (!timed_wait(&ctl->empty[s], ph ^ 1, &w_empty)) {
                        if (!*abort_flag) give_up(KLEOS_AT_GEMM_PRODUCER, t);
                        break;
                    }
                    const int nsub = min(SUB, KS - kb * SUB);
                    if (leader) mbar_expect_tx(&ctl->full[s], 2 * nsub * SLICE_BYTES);
                    const uint32_t full_leader = map_to_cta(smem_u32(&ctl->full[s]), 0);
                    uint8_t* sa = tiles + s * STAGE_BYTES;
                    for (int sub = 0; sub < nsub; ++sub) {
                        const int kx = (kb * SUB + sub) * BK;
                        tma_load_2d_pair(sa + sub * SLICE_BYTES, ma, kx, p.row_base, full_leader);
                        tma_load_2d_pair(sa + sub * SLICE_BYTES + A_STAGE_BYTES, mb, kx, brow, full_leader);
                    }
                    if (kb == min(2, KB - 1)) {
                        // look at the next tile: the leader hands its claim out now, the partner reads
                        // it if it is there already
                        int nxt = -1;
                        if (leader) {
                            hand_out(i + 1, ahead);
                            nxt = ahead;
                        } else {
                            const int slot = (i + 1) % kRing;
                            if (mbar_try_wait_cluster(&ctl->task_full[slot], ((i + 1) / kRing) & 1u))
                                nxt = *reinterpret_cast<volatile int*>(&ctl->task_s[slot]);
                        }
                        if (nxt >= 0) {
                            int kind, id;
                            peeked_tile = decode_tile(ctl, nxt, a.nLx);
                            peeked = nxt;
                            if (dependency(peeked_tile, &kind, &id)) ask(nxt, kind, id);
                        }
                    }
                    par ^= 1u << s;
                    s = s + 1 == NST ? 0 : s + 1;
                }
            }
            if (stall) {
                stall[kProdEmpty] = w_empty;
                stall[kProdReady] = w_ready;
                stall[kProdFence] = w_fence;
                stall[kProdTotal] = clock64() - c_begin;
            }
            atomicAdd(&ctl->roles_done, 1);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader only)
        if (lane == 0) {
            if (leader) {
                uint32_t par = parity0;
                int s = 0;
                const long long c_begin = clock64();
                long long w_acc = 0, w_full = 0, w_task = 0;
                for (uint32_t i = 0;; ++i) {
                    const long long c_task = stall ? clock64() : 0;
                    const int t = take(i, KLEOS_AT_GEMM_MMA);
                    if (stall) w_task += clock64() - c_task;
                    if (t < 0) break;
                    const Tile ti = decode_tile(ctl, t, a.nLx);
                    const int KS = (ti.phase ? a.I : a.H) / BK, KB = (KS + SUB - 1) / SUB;
                    const uint32_t tn = route_tiles + i, buf = tn & 1, use = tn >> 1;
                    if (!timed_wait(&ctl->acc_empty[buf], (use & 1) ^ 1, &w_acc)) {
                        if (!*abort_flag) give_up(KLEOS_AT_GEMM_MMA, t);
                        break;
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * BN;
                    bool ok = true;
                    for (int kb = 0; kb < KB; ++kb) {
                        const uint32_t ph = (par >> s) & 1u;
                        if (!timed_wait(&ctl->full[s], ph, &w_full)) {
                            if (!*abort_flag) give_up(KLEOS_AT_GEMM_MMA, t);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t sa = smem_u32(tiles + s * STAGE_BYTES);
                        const int nsub = min(SUB, KS - kb * SUB);
                        for (int sub = 0; sub < nsub; ++sub) {
                            const uint64_t da = make_smem_desc(sa + sub * SLICE_BYTES);
                            const uint64_t db = make_smem_desc(sa + sub * SLICE_BYTES + A_STAGE_BYTES);
#pragma unroll
                            for (int k = 0; k < BK / UMMA_K; ++k)
                                umma_bf16_pair(d_tmem, da + 2 * k, db + 2 * k, kInstrDesc,
                                               (kb | sub | k) != 0 ? 1u : 0u);
                        }
                        const uint32_t e_local = smem_u32(&ctl->empty[s]);
                        umma_commit_pair(map_to_cta(e_local, 0));
                        umma_commit_pair(map_to_cta(e_local, 1));
                        par ^= 1u << s;
                        s = s + 1 == NST ? 0 : s + 1;
                    }
                    if (!ok) break;
                    const uint32_t f_local = smem_u32(&ctl->acc_full[buf]);
                    umma_commit_pair(map_to_cta(f_local, 0));
                    umma_commit_pair(map_to_cta(f_local, 1));
                }
                if (stall) {
                    stall[kMmaAcc] = w_acc;
                    stall[kMmaFull] = w_full;
                    stall[kMmaTask] = w_task;
                    stall[kMmaTotal] = clock64() - c_begin;
                }
            }
            atomicAdd(&ctl->roles_done, 1);
        }
        __syncwarp();
    } else if (warp == 3) {
        // ------------------------------------------------------------ subscriber
        // Watches, on behalf of this block's producer, the one flag the producer's next tile depends
        // on (the data flag of a dispatched cell, or the GEMM1 counter of a panel pair) and notes
        // in shared memory when it has been seen (reference: the subscriber warps poll the flags
        // and turn arrivals into tasks, os/subscriber.cuh:56-185).  Also mirrors the rank's abort
        // word into this block while any role is still working.
        if (lane == 0) {
            unsigned seen = 0;
            const unsigned need = 8u * (unsigned)NT1;
            const unsigned long long* xflag =
                reinterpret_cast<const unsigned long long*>(a.peers.arena[a.rank] + a.lay.xflag);
            while (*reinterpret_cast<volatile int*>(&ctl->roles_done) < kRoleWarps) {
                if (ld_relaxed_gpu(&ctr->abort_all)) *abort_flag = 1;
                const unsigned r = *reinterpret_cast<volatile unsigned*>(&ctl->sub_req);
                if ((r >> 16) == seen) {
                    __nanosleep(200);
                    continue;
                }
                seen = r >> 16;
                const int kind = (int)((r >> 15) & 1u), id = (int)(r & 0x7fffu);
                const long long t0 = clock64();
                bool ok = true;
                for (;;) {
                    // relaxed polls; one acquiring load and one proxy fence (the operands are read
                    // through the async proxy) once the flag is up
                    const bool up = kind ? ld_relaxed_gpu(&ctr->pair_done[id]) >= need
                                         : (uint32_t)(ld_relaxed_sys(xflag + id) >> 32) == a.epoch;
                    if (up) {
                        if (kind) (void)ld_acquire_gpu(&ctr->pair_done[id]);
                        else (void)ld_acquire_sys(xflag + id);
                        asm volatile("fence.proxy.async;" ::: "memory");
                        break;
                    }
                    __nanosleep(100);
                    if (*abort_flag || ld_relaxed_gpu(&ctr->abort_all)) {
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    if (clock64() - t0 > budget) {
                        give_up(kind ? KLEOS_AT_GEMM_PRODUCER : KLEOS_AT_PLAN_WAIT, kind ? 3000 + id : 1000 + id);
                        ok = false;
                        break;
                    }
                }
                if (ok) {
                    asm volatile("fence.acq_rel.cta;" ::: "memory");
                    if (kind) *reinterpret_cast<volatile unsigned char*>(&ctl->pair_ready_s[id]) = 1;
                    else *reinterpret_cast<volatile unsigned char*>(&ctl->ready_s[id]) = 1;
                }
            }
        }
        __syncwarp();
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------------------------------------ accumulator read-back (both blocks)
        const int q = warp - 4;
        const uint32_t acc_empty0 = smem_u32(&ctl->acc_empty[0]);
        const int TCM = a.pEC / kTileM;
        // Publication of a finished tile.  The stores of the tile must be visible before its
        // counter moves, which costs a fence that waits for those stores; issued right behind
        // them it would hold this warp for microseconds per tile.  So a tile is published when
        // the warp next has nothing to do (its next accumulator is not ready yet) or, at the
        // latest, just before it reads the next accumulator back: by then the stores have
        // drained and the fence returns at once.
        int pend_phase = 0, pend_panel = -1;
        auto publish = [&]() {
            if (pend_panel < 0) return;
            // The warp's stores are ordered before the counter update by ONE fence of the lane that
            // updates it, after the warp has met (the fence is cumulative over what that lane has
            // observed through the warp barrier): the pattern of a grid-wide barrier, per warp.
            if (pend_phase == 0) {
                // GEMM1: the pair's counter releases its GEMM2 tiles (reference processor.cuh:717-729)
                __syncwarp();
                if (lane == 0) {
                    fence_release_gpu();
                    atomicAdd(&ctr->pair_done[pend_panel], 1u);
                    if (stamp && q == 0) stamp[kLastGemm1] = global_ns();
                }
            } else {
                // GEMM2: one return flag per (expert, 128-row panel), raised by the warp that stores
                // the panel's last piece (reference: one signal per returned tile, processor.cuh:745-769)
                __syncwarp();
                if (lane == 0) {
                    fence_release_sys();
                    const unsigned prev = atomicAdd(&ctr->panel_ret[pend_panel], 1u);
                    if (prev + 1u == 4u * (unsigned)NT2) {
                        const PanelEntry pp = panel_of(ctl, pend_panel);
                        const int cell = pp.src * a.nLx + pp.le;
                        const int r0 = pp.row_base - cell * a.pEC;
                        const size_t e_global = (size_t)a.rank * a.nLx + pp.le;
                        if (!a.suppress)
                            st_release_sys(reinterpret_cast<unsigned long long*>(a.peers.arena[pp.src] + a.lay.ypflag) +
                                               (e_global * TCM + r0 / kTileM),
                                           make_flag(a.epoch, 1u));
                        const unsigned done = atomicAdd(&ctr->panels_returned, 1u);
                        if (done + 1u == (unsigned)ctl->total_panels && !a.suppress) {
                            // everything this rank's experts owed has been returned: tell every
                            // source (they leave the forward only after all owners said so)
                            fence_release_sys();
                            for (int r = 0; r < a.world; ++r)
                                st_release_sys(reinterpret_cast<unsigned long long*>(a.peers.arena[r] + a.lay.yflag) + a.rank,
                                               make_flag(a.epoch, 1u));
                        }
                    }
                }
            }
            pend_panel = -1;
            __syncwarp();
        };
        const bool tally = stall && q == 0 && lane == 0;
        const long long c_begin = clock64();
        long long w_pub = 0, w_acc = 0, w_read = 0;
        for (uint32_t i = 0;; ++i) {
            const int t = take(i, KLEOS_AT_GEMM_EPILOGUE);
            if (t < 0) break;
            const Tile ti = decode_tile(ctl, t, a.nLx);
            const bool have_panel = (int)cta_rank < ti.n_left;
            const int my_panel = ti.panel0 + (have_panel ? (int)cta_rank : 0);
            const PanelEntry p = panel_of(ctl, my_panel);
            const int rows = have_panel ? p.rows : 0;
            const int N = ti.phase ? a.H : a.I;
            const uint32_t tn = route_tiles + i, buf = tn & 1, use = tn >> 1;
            if (*abort_flag) break;
            if (stamp && i == 0 && q == 0 && lane == 0) stamp[kFirstTile] = global_ns();
            {
                // this tile's 256 bias values, one private copy per warp, loaded while the main
                // loop of the tile is still running
                const TE* bias = static_cast<const TE*>(ti.phase ? a.b2 : a.b1);
                using TE2 = typename Pack2<TE>::type;
                const int nb = ti.nt * BN + 8 * lane;
                float* bs = &ctl->bias_s[q][8 * lane];
                if (nb < N) {
                    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(bias + (size_t)ti.le * N + nb));
                    const TE2* h2 = reinterpret_cast<const TE2*>(&raw);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = Pack2<TE>::to_f2(h2[j]);
                        bs[2 * j] = f.x;
                        bs[2 * j + 1] = f.y;
                    }
                }
                __syncwarp();
            }
            long long c0 = tally ? clock64() : 0;
            {
                // (warp-uniform decision: lane 0's view)
                const int ready = __shfl_sync(0xffffffffu, mbar_try_wait(&ctl->acc_full[buf], use & 1) ? 1 : 0, 0);
                if (!ready) publish();  // idle: publish the last tile now
            }
            if (tally) {
                w_pub += clock64() - c0;
                c0 = clock64();
            }
            if (!mbar_wait(&ctl->acc_full[buf], use & 1, budget, abort_flag)) {
                if (!*abort_flag && lane == 0) give_up(KLEOS_AT_GEMM_EPILOGUE, t);
                break;
            }
            if (tally) {
                w_acc += clock64() - c0;
                c0 = clock64();
            }
            publish();
            if (tally) {
                w_pub += clock64() - c0;
                c0 = clock64();
            }
            tc_fence_after();
            const int n0 = ti.nt * BN;
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
            const uint32_t acc_empty_leader = map_to_cta(acc_empty0 + buf * 8u, 0);
            const int rows_w = min(32, rows - q * 32);
            if (rows_w <= 0) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
            } else if (ti.phase == 0) {
                TE* obase = static_cast<TE*>(a.y1) + (size_t)(p.row_base + q * 32) * a.I + n0;
                read_back<TE, kAct>(taddr, ctl->bias_s[q], ctl->stage_s[q], obase, (size_t)a.I, rows_w, n0, N,
                                    lane, acc_empty_leader);
            } else {
                // straight into the SOURCE rank's result cell (reference os/packet.cuh:338-340)
                const int cell = p.src * a.nLx + p.le;
                const int r0 = p.row_base - cell * a.pEC;
                const size_t e_global = (size_t)a.rank * a.nLx + p.le;
                TE* obase = reinterpret_cast<TE*>(a.peers.arena[p.src] + a.lay.ycell) +
                            (e_global * a.pEC + r0 + q * 32) * a.H + n0;
                read_back<TE, 2>(taddr, ctl->bias_s[q], ctl->stage_s[q], obase, (size_t)a.H, rows_w, n0, N,
                                 lane, acc_empty_leader);
            }
            // completion bookkeeping: every read-back warp of the pair counts, with or without rows;
            // it is published later (see publish above)
            pend_phase = ti.phase;
            pend_panel = ti.phase == 0 ? ti.panel0 : (have_panel ? my_panel : -1);
            if (tally) w_read += clock64() - c0;
            if (stamp && q == 0 && lane == 0) stamp[kLastTile] = global_ns();
        }
        if (!*abort_flag) publish();
        if (tally) {
            stall[kBackPublish] = w_pub;
            stall[kBackAcc] = w_acc;
            stall[kBackRead] = w_read;
            stall[kBackTotal] = clock64() - c_begin;
        }
        // no tiles left: help with the combine of the tokens whose rows return last
        run_combine();
        if (lane == 0) atomicAdd(&ctl->roles_done, 1);
        __syncwarp();
    } else if (warp >= 8) {
        // ------------------------------------------------------------ transport (both blocks)
        // (1) dispatch: this rank's routed, unscaled token rows into the owners' cells, row i of a
        // cell = the token that owns slot i (reference os/packet.cuh:147-166).  Units of up to
        // eight consecutive rows of one cell are claimed from a counter in sending order; a unit
        // is published with one system fence and one counter update, and whoever brings a cell's
        // count to its total raises the cell's data flag on the owner (:214-237).
        const unsigned row_chunks = (unsigned)((size_t)a.H * sizeof(TE) / 16);
        const unsigned total_units = ctl->total_units;
        for (;;) {
            unsigned u = 0;
            if (lane == 0) u = (*abort_flag) ? 0xffffffffu : atomicAdd(&ctr->unit_next, 1u);
            u = __shfl_sync(0xffffffffu, u, 0);
            if (u >= total_units) break;
            int lo = 0, hi = a.E;  // last order position with prefix_s[] <= u
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (ctl->prefix_s[mid] <= u) lo = mid; else hi = mid;
            }
            const int le = lo / a.world, owner = (a.rank + 1 + lo % a.world) % a.world;
            const int e = owner * a.nLx + le;
            const int routed = ctl->own_s[lo];
            const int slot0 = (int)(u - ctl->prefix_s[lo]) * a.unit_rows;
            const int nrows = min(a.unit_rows, routed - slot0);
            const int my_tok = lane < nrows ? __ldcg(a.cell_tokens + (size_t)e * a.pEC + slot0 + lane) : 0;
            char* cell = a.peers.arena[owner] + a.lay.xcell +
                         (((size_t)a.rank * a.nLx + le) * a.pEC + slot0) * a.H * sizeof(TE);
            // two rows at a time, eight 16-byte loads per lane and row in flight before the stores
            for (int r = 0; r < nrows; r += 2) {
                const int tok0 = __shfl_sync(0xffffffffu, my_tok, r);
                const int tok1 = __shfl_sync(0xffffffffu, my_tok, min(r + 1, kUnitRows - 1));
                const bool two = r + 1 < nrows;
                const uint4* src0 = reinterpret_cast<const uint4*>(
                    static_cast<const char*>(a.tokens) + (size_t)tok0 * a.H * sizeof(TE));
                const uint4* src1 = reinterpret_cast<const uint4*>(
                    static_cast<const char*>(a.tokens) + (size_t)tok1 * a.H * sizeof(TE));
                uint4* dst0 = reinterpret_cast<uint4*>(cell + (size_t)r * a.H * sizeof(TE));
                uint4* dst1 = reinterpret_cast<uint4*>(cell + (size_t)(r + 1) * a.H * sizeof(TE));
                for (unsigned c0 = lane; c0 < row_chunks; c0 += 256) {
                    uint4 v0[8], v1[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        if (c0 + 32 * k < row_chunks) {
                            v0[k] = __ldg(src0 + c0 + 32 * k);
                            if (two) v1[k] = __ldg(src1 + c0 + 32 * k);
                        }
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        if (c0 + 32 * k < row_chunks) {
                            dst0[c0 + 32 * k] = v0[k];
                            if (two) dst1[c0 + 32 * k] = v1[k];
                        }
                }
            }
            __syncwarp();
            if (lane == 0) {
                fence_release_sys();
                const unsigned prev = atomicAdd(&ctr->cell_done[e], (unsigned)nrows);
                if ((int)prev + nrows == routed) {
                    fence_release_sys();
                    st_release_sys(reinterpret_cast<unsigned long long*>(a.peers.arena[owner] + a.lay.xflag) +
                                       ((size_t)a.rank * a.nLx + le),
                                   make_flag(a.epoch, (unsigned)routed));
                }
            }
        }
        if (stamp && warp == 8 && lane == 0) stamp[kDispatched] = global_ns();
        if (a.debug & 1) {
            // tuning switch: leave the memory system to the tile stream until its last tile is done
            // (the producer, the issuer and the four read-back warps have all signed off)
            const long long t0 = clock64();
            while (*reinterpret_cast<volatile int*>(&ctl->roles_done) < 6 && !*abort_flag && clock64() - t0 < budget)
                __nanosleep(1000);
        }

        run_combine();
        if (stamp && warp == 8 && lane == 0) stamp[kCombined] = global_ns();
        // (3) nobody leaves the forward before every expert rank has finished with this rank's
        // cells and counts: the next forward may then overwrite them (flags carry the epoch, so
        // nothing is ever cleared).  One block waits for the whole rank.
        if (blockIdx.x == 0 && warp == 8 && lane < a.world && !*abort_flag) {
            unsigned long long v;
            const unsigned long long* yf =
                reinterpret_cast<const unsigned long long*>(a.peers.arena[a.rank] + a.lay.yflag) + lane;
            if (!wait_flag(yf, a.epoch, budget, &v)) give_up(KLEOS_AT_COMBINE_WAIT, 2000 + lane);
        }
        __syncwarp();
        if (lane == 0) atomicAdd(&ctl->roles_done, 1);
    }

    // teardown: neither block may leave while its partner can still touch its shared memory,
    // barriers or tensor memory
    if (transport) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // the plan's barrier
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                     : "memory");
    }
    if (stamp && tid == 0) stamp[kEnd] = global_ns();
}

}  // namespace kleos
