// Expert-FFN GEMM with paired blocks (tcgen05 cta_group::2): a cluster of two blocks on
// neighbouring SMs computes a 256 x 256 output tile -- two 128-row panels of the same local
// expert against the same 256 weight rows.  Each block TMA-loads its own panel (A) and only
// HALF of the weight tile (B), so the bytes pulled into an SM per FLOP drop by a third compared
// with one block per 128 x 256 tile.  Shared memory holds six 64-wide K slices per block, used
// as six shallow or three deep pipeline stages (template parameter kSub).  The epilogue stages
// its rows through a swizzled shared-memory tile so that every store instruction writes whole
// 128-byte lines, also when the destination is a peer's cell.  No load is multicast: every block
// fetches exactly the bytes it keeps.
//
// Per block, 256 threads:
//   warp 0      TMA producer (one lane): waits on its own `empty`, loads into its own shared
//               memory, credits the bytes to the LEADER's `full` barrier
//   warp 1      leader only: issues tcgen05.mma.cta_group::2, commits to `empty` and
//               `acc_full` of BOTH blocks
//   warp 2      tensor-memory allocation / release (both blocks, cta_group::2 forms)
//   warps 4..7  epilogue of the block's own 128 accumulator rows; arrives on the LEADER's
//               `acc_empty`
// Work and epilogue semantics follow the reference's tile worker (os/processor/processor.cuh:
// 350-489,706-741).  Every wait is bounded.  This kernel runs one GEMM over a finished panel
// list (the dense single-expert layer, and the routed layer when its phases are launched one
// by one); the persistent kernel in moe_flow.cuh reuses its tile shapes and pipeline.
#pragma once

#include <cuda.h>

#include "gemm_common.cuh"
#include "tc_common.cuh"

namespace kleos {
namespace gemm_tc2 {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int kSlices = 6;                        // 64-wide K slices of shared memory in total
constexpr int A_STAGE_BYTES = BM * BK * 2;        // 16 KiB: one K slice of this block's panel
constexpr int B_STAGE_BYTES = (BN / 2) * BK * 2;  // 16 KiB: one K slice of this block's half weight tile
constexpr int SLICE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int TMEM_COLS = 512;  // two accumulators of 256 fp32 columns
constexpr int SMEM_BYTES = kSlices * SLICE_BYTES + 1024 + 28672;

struct Control {
    unsigned long long full[kSlices];   // used on the leader (one per pipeline stage)
    unsigned long long empty[kSlices];  // one per block
    unsigned long long acc_full[2];    // one per block
    unsigned long long acc_empty[2];   // used on the leader, 8 arrivals (4 warps x 2 blocks)
    uint32_t tmem_base;
    int abort;
    int le_start[257];
    __align__(16) float bias_s[4][256];      // bias of the tile being read back, per epilogue warp
    __align__(16) uint4 stage_s[4][32 * 8];  // per epilogue warp: 32 rows x 128 bytes, swizzled
};

static_assert(sizeof(Control) <= 28672, "control block must fit the shared memory set aside for it");

struct PairTile {
    int panel0, n_panels_left, nt, le;
};

// Tiles ordered by local expert, then N tile, then panel pair.
__device__ __forceinline__ bool decode_pair_tile(int t, const int* le_start, int le_begin,
                                                 int le_end, int NT, PairTile* c) {
    for (int le = le_begin; le < le_end; ++le) {
        const int p0 = le_start[le], np = le_start[le + 1] - p0;
        const int npair = (np + 1) >> 1;
        const int tiles = npair * NT;
        if (t < tiles) {
            const int nt = t / npair, pi = t - nt * npair;
            c->le = le;
            c->nt = nt;
            c->panel0 = p0 + 2 * pi;
            c->n_panels_left = np - 2 * pi;  // 1 when the pair's second panel does not exist
            return true;
        }
        t -= tiles;
    }
    return false;
}

__device__ __forceinline__ int total_pair_tiles(const int* le_start, int le_begin, int le_end,
                                                int NT) {
    int total = 0;
    for (int le = le_begin; le < le_end; ++le) total += ((le_start[le + 1] - le_start[le] + 1) >> 1) * NT;
    return total;
}

}  // namespace gemm_tc2

// kEpi selects the fused epilogue at compile time (0: bias + ReLU, 1: bias + GELU, 2: bias only)
// so the read-back loop stays a short straight-line sequence.
// kSub = 64-wide K slices per pipeline stage: 1 gives six shallow stages (best when the weights
// stream from HBM), 2 gives three deep stages and half the barrier round trips (best when the
// operands come from L2 and the tensor pipe is the limit).
template <typename TE, int kEpi, int kSub>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(256, 1)
ffn_gemm_tc2(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
             GemmArgs g) {
    using namespace tc;
    using namespace gemm_tc2;
    constexpr int SUB = kSub, STAGES = kSlices / kSub, STAGE_BYTES = kSub * SLICE_BYTES;
    constexpr int NST = STAGES;
    constexpr uint32_t kInstrDesc = make_instr_desc_16b(2 * BM, BN, Pack2<TE>::kMmaFormat);
    using TE2 = typename Pack2<TE>::type;
    const long long t_kernel = clock64();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    Control* ctl = reinterpret_cast<Control*>(tiles + kSlices * SLICE_BYTES);
    __shared__ bool last_block;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t cta_rank = cluster_ctarank();
    const bool leader = cta_rank == 0;
    volatile int* abort_flag = &ctl->abort;

    for (int i = tid; i <= g.nLx; i += blockDim.x) ctl->le_start[i] = g.le_start[i];
    if (tid == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], 8);
        }
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&ctl->tmem_base)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both blocks' barriers exist before anything remote touches them
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    if (g.stats && tid == 0) g.stats[blockIdx.x * kStatSlots + 8] = clock64() - t_kernel;
    auto panel_at = [&](int i) -> PanelEntry { return g.panels[i]; };

    const int NT = (g.N + BN - 1) / BN;
    const int total = total_pair_tiles(ctl->le_start, g.le_begin, g.le_end, NT);
    const int KS = g.Kd / BK;                 // 64-wide K slices
    const int KB = (KS + SUB - 1) / SUB;      // pipeline stages per tile
    const int n_clusters = (int)gridDim.x >> 1, cluster_id = blockIdx.x >> 1;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both blocks)
        if (lane == 0) {
            asm volatile("fence.proxy.async;" ::: "memory");
            uint32_t it = 0;
            long long w_empty = 0;
            const long long t_begin = clock64();
            for (int t = cluster_id; t < total && !*abort_flag; t += n_clusters) {
                PairTile pt;
                if (!decode_pair_tile(t, ctl->le_start, g.le_begin, g.le_end, NT, &pt)) break;
                // the block without a panel of its own re-reads the first one and discards
                const int my_panel = pt.panel0 + ((int)cta_rank < pt.n_panels_left ? (int)cta_rank : 0);
                const PanelEntry p = panel_at(my_panel);
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % NST;
                    const uint32_t ph = (it / NST) & 1;
                    if (!mbar_wait_timed(&ctl->empty[s], ph ^ 1, g.wait_cycles, abort_flag, &w_empty)) {
                        report_error(g.status, KLEOS_AT_GEMM_PRODUCER, t, (int)g.epoch);
                        *abort_flag = 1;
                        break;
                    }
                    // the leader announces the bytes of both blocks on its own barrier
                    const int nsub = min(SUB, KS - kb * SUB);
                    if (leader) mbar_expect_tx(&ctl->full[s], 2 * nsub * SLICE_BYTES);
                    const uint32_t full_leader = map_to_cta(smem_u32(&ctl->full[s]), 0);
                    uint8_t* sa = tiles + s * STAGE_BYTES;
                    for (int sub = 0; sub < nsub; ++sub) {
                        const int kx = (kb * SUB + sub) * BK;
                        tma_load_2d_pair(sa + sub * SLICE_BYTES, &map_a, kx, p.row_base, full_leader);
                    }
                }
            }
            if (g.stats) {
                g.stats[blockIdx.x * kStatSlots + 0] = w_empty;
                g.stats[blockIdx.x * kStatSlots + 1] = clock64() - t_begin;
            }
        }
        __syncwarp();
    } else if (warp == 3) {
        // ------------------------------------------------------------ second TMA producer (both blocks)
        // The weight slices are issued by a thread of their own, next to the panel slices of
        // warp 0 (measured: 1.6 % off the launch).  It waits for the same free-stage barrier and
        // its bytes complete on the same full barrier; the byte count announced by warp 0 covers
        // both, and a slice landing before that announcement only makes the barrier's byte
        // count negative for a moment (the phase cannot complete before warp 0 has arrived).
        if (lane == 0) {
            asm volatile("fence.proxy.async;" ::: "memory");
            uint32_t it = 0;
            long long w_unused = 0;
            for (int t = cluster_id; t < total && !*abort_flag; t += n_clusters) {
                PairTile pt;
                if (!decode_pair_tile(t, ctl->le_start, g.le_begin, g.le_end, NT, &pt)) break;
                const int brow = pt.le * g.N + pt.nt * BN + (int)cta_rank * (BN / 2);
                bool ok = true;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % NST;
                    const uint32_t ph = (it / NST) & 1;
                    if (!mbar_wait_timed(&ctl->empty[s], ph ^ 1, g.wait_cycles, abort_flag, &w_unused)) {
                        ok = false;  // the first producer reports the failure
                        break;
                    }
                    const int nsub = min(SUB, KS - kb * SUB);
                    const uint32_t full_leader = map_to_cta(smem_u32(&ctl->full[s]), 0);
                    uint8_t* sa = tiles + s * STAGE_BYTES;
                    for (int sub = 0; sub < nsub; ++sub)
                        tma_load_2d_pair(sa + sub * SLICE_BYTES + A_STAGE_BYTES, &map_b, (kb * SUB + sub) * BK, brow,
                                         full_leader);
                }
                if (!ok) break;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader only)
        if (leader && lane == 0) {
            uint32_t it = 0, tile_n = 0;
            long long w_acc = 0, w_full = 0;
            const long long t_begin = clock64();
            for (int t = cluster_id; t < total && !*abort_flag; t += n_clusters, ++tile_n) {
                const uint32_t buf = tile_n & 1, use = tile_n >> 1;
                if (!mbar_wait_timed(&ctl->acc_empty[buf], (use & 1) ^ 1, g.wait_cycles, abort_flag, &w_acc)) {
                    report_error(g.status, KLEOS_AT_GEMM_MMA, t, (int)g.epoch);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                bool ok = true;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % NST;
                    const uint32_t ph = (it / NST) & 1;
                    if (!mbar_wait_timed(&ctl->full[s], ph, g.wait_cycles, abort_flag, &w_full)) {
                        report_error(g.status, KLEOS_AT_GEMM_MMA, t, (int)g.epoch);
                        *abort_flag = 1;
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
                    // the stage is free in both blocks once these MMAs have read it
                    const uint32_t e_local = smem_u32(&ctl->empty[s]);
                    umma_commit_pair(map_to_cta(e_local, 0));
                    umma_commit_pair(map_to_cta(e_local, 1));
                }
                if (!ok) break;
                const uint32_t f_local = smem_u32(&ctl->acc_full[buf]);
                umma_commit_pair(map_to_cta(f_local, 0));
                umma_commit_pair(map_to_cta(f_local, 1));
            }
            if (g.stats) {
                g.stats[blockIdx.x * kStatSlots + 2] = w_acc;
                g.stats[blockIdx.x * kStatSlots + 3] = w_full;
                g.stats[blockIdx.x * kStatSlots + 4] = clock64() - t_begin;
            }
        }
        __syncwarp();
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------------------------------------ epilogue (both blocks)
        const int q = warp - 4;
        const TE* bias = static_cast<const TE*>(g.bias);
        uint32_t tile_n = 0;
        long long w_accfull = 0, w_tmem = 0;
        const long long t_begin = clock64();
        for (int t = cluster_id; t < total; t += n_clusters, ++tile_n) {
            PairTile pt;
            if (!decode_pair_tile(t, ctl->le_start, g.le_begin, g.le_end, NT, &pt)) break;
            const bool have_panel = (int)cta_rank < pt.n_panels_left;
            const PanelEntry p = panel_at(pt.panel0 + (have_panel ? (int)cta_rank : 0));
            const int rows = have_panel ? p.rows : 0;
            const uint32_t buf = tile_n & 1, use = tile_n >> 1;
            if (*abort_flag) break;
            {
                // stage this tile's 256 bias values in shared memory (one private copy per warp,
                // one 16-byte load per lane) while the main loop of the tile is still running:
                // global loads issued later would queue behind the operand traffic streaming
                // into this SM
                const int nb = pt.nt * BN + 8 * lane;
                float* bs = &ctl->bias_s[q][8 * lane];
                if (nb < g.N) {
                    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(
                        bias + (size_t)pt.le * g.N + nb));
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
            if (!mbar_wait_timed(&ctl->acc_full[buf], use & 1, g.wait_cycles, abort_flag, &w_accfull)) {
                if (lane == 0) report_error(g.status, KLEOS_AT_GEMM_EPILOGUE, t, (int)g.epoch);
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const int n0 = pt.nt * BN;
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
            // this warp's 32 accumulator rows; rows_w of them carry tokens
            const int rows_w = min(32, rows - q * 32);
            if (rows_w <= 0) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->acc_empty[buf]), 0));
                continue;
            }
            TE* obase = out_ptr<TE>(g, p, q * 32, n0);
            uint4* stg = ctl->stage_s[q];
            // Accumulator read-back, two 32-column chunks in flight.  Every 64 columns the warp
            // transposes through a swizzled shared-memory tile so that each store instruction
            // writes four complete 128-byte lines (one row segment per 8 lanes) instead of 32
            // scattered 16-byte pieces: this is what the NVLink path to a peer's cell needs.
            uint32_t r[2][32];
            tmem_ld_32x32(taddr, r[0]);
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                const long long tq = clock64();
                tmem_ld_wait();
                w_tmem += clock64() - tq;
                if (c + 1 < BN / 32) {
                    tmem_ld_32x32(taddr + (c + 1) * 32, r[(c + 1) & 1]);
                } else {
                    // the whole accumulator is in registers: hand it back to the MMA issuer
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->acc_empty[buf]), 0));
                }
                const uint32_t* rc = r[c & 1];
                const float4* bq = reinterpret_cast<const float4*>(&ctl->bias_s[q][c * 32]);
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
                    const int ch = (c & 1) * 4 + j;  // 16-byte chunk inside the 128-byte row segment
                    stg[lane * 8 + (ch ^ (lane & 7))] = make_uint4(
                        packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                }
                if (c & 1) {
                    __syncwarp();
                    const int col0 = (c - 1) * 32;
                    if (n0 + col0 < g.N) {
#pragma unroll
                        for (int it = 0; it < 8; ++it) {
                            const int rr = it * 4 + (lane >> 3), ch = lane & 7;
                            const uint4 v = stg[rr * 8 + (ch ^ (rr & 7))];
                            if (rr < rows_w)
                                *reinterpret_cast<uint4*>(obase + (size_t)rr * g.N + col0 + ch * 8) = v;
                        }
                    }
                    __syncwarp();
                }
            }
        }
        if (g.stats && warp == 4 && lane == 0) {
            g.stats[blockIdx.x * kStatSlots + 5] = w_accfull;
            g.stats[blockIdx.x * kStatSlots + 6] = clock64() - t_begin;
            g.stats[blockIdx.x * kStatSlots + 7] = w_tmem;
        }
    }

    // teardown: neither block may leave while its partner can still touch its shared memory,
    // barriers or tensor memory
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(TMEM_COLS)
                     : "memory");
    }
    if (g.mode == 1) publish_return_flags(g.ret, &last_block);
}

}  // namespace kleos
