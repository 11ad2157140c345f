// Expert-FFN GEMM on the 5th-generation tensor cores (sm_100a): bf16 operands staged in shared
// memory by TMA (128-byte swizzle), tcgen05.mma issued by one thread with the 128x256 fp32
// accumulator in tensor memory, double-buffered so the epilogue of one tile overlaps the main
// loop of the next, epilogue read back with tcgen05.ld.
//
// Replaces the reference's 128x64x8 mma.sync / cp.async block GEMM
// (os/processor/gemm.cuh:58-107, mmaConfig.cuh:28-81) and its fused bias+activation epilogue
// (gemm.cuh:23-50, processor.cuh:350-489).
//
// Persistent grid, one block per SM, 256 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      MMA issuer   (one elected lane)
//   warp 2      tensor-memory allocation / release
//   warps 4..7  epilogue, warp q owns accumulator lanes [32q, 32q+32)
// Every mbarrier wait is bounded; on expiry the block records a status and drains.
#pragma once

#include <cuda.h>

#include "gemm_common.cuh"
#include "tc_common.cuh"

namespace kleos {
namespace gemm_tc {
using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16, STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int TMEM_COLS = 512;              // two 128x256 fp32 accumulators
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 12288 /*control*/;


struct Control {
    unsigned long long full[STAGES];
    unsigned long long empty[STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    uint32_t tmem_base;
    int abort;
    int le_start[257];
    __align__(16) float bias_s[2][4][256];  // bias of the tile being read back: [accumulator][epilogue warp]
};

}  // namespace gemm_tc

// kEpi selects the fused epilogue at compile time (0: bias + ReLU, 1: bias + GELU, 2: bias only)
// so the read-back loop stays a short straight-line sequence.
template <typename TE, int kEpi>
__global__ void __launch_bounds__(256, 1)
ffn_gemm_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            GemmArgs g) {
    using namespace tc;
    using namespace gemm_tc;
    constexpr uint32_t kInstrDesc = make_instr_desc_16b(BM, BN, Pack2<TE>::kMmaFormat);
    using TE2 = typename Pack2<TE>::type;
    extern __shared__ uint8_t smem_raw[];
    // operand stages need 1024-byte alignment for the 128-byte swizzle pattern
    uint8_t* tiles = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    Control* ctl = reinterpret_cast<Control*>(tiles + STAGES * STAGE_BYTES);
    __shared__ bool last_block;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int* abort_flag = &ctl->abort;

    for (int i = tid; i <= g.nLx; i += blockDim.x) ctl->le_start[i] = g.le_start[i];
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], 4);
        }
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&ctl->tmem_base)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    const int NT = (g.N + BN - 1) / BN;
    const int total = (ctl->le_start[g.le_end] - ctl->le_start[g.le_begin]) * NT;
    const int KB = g.Kd / BK;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // dispatched rows and y1 rows were written with ordinary stores (possibly by a
            // peer GPU); order them before this thread's async-proxy reads
            asm volatile("fence.proxy.async;" ::: "memory");
            uint32_t it = 0;
            long long w_empty = 0;
            const long long t_begin = clock64();
            for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x) {
                TileCoord tcd;
                if (!decode_tile(t, ctl->le_start, g.le_begin, g.le_end, NT, &tcd)) break;
                const PanelEntry p = g.panels[tcd.panel];
                const int brow = tcd.le * g.N + tcd.nt * BN;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait_timed(&ctl->empty[s], ph ^ 1, g.wait_cycles, abort_flag, &w_empty)) {
                        report_error(g.status, KLEOS_AT_GEMM_PRODUCER, t, (int)g.epoch);
                        *abort_flag = 1;
                        break;
                    }
                    mbar_expect_tx(&ctl->full[s], STAGE_BYTES);
                    uint8_t* sa = tiles + s * STAGE_BYTES;
                    tma_load_2d(sa, &map_a, kb * BK, p.row_base, &ctl->full[s]);
                    tma_load_2d(sa + A_STAGE_BYTES, &map_b, kb * BK, brow, &ctl->full[s]);
                }
            }
            if (g.stats) {
                g.stats[blockIdx.x * kStatSlots + 0] = w_empty;
                g.stats[blockIdx.x * kStatSlots + 1] = clock64() - t_begin;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, tile_n = 0;
            long long w_acc = 0, w_full = 0;
            const long long t_begin = clock64();
            for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x, ++tile_n) {
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
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait_timed(&ctl->full[s], ph, g.wait_cycles, abort_flag, &w_full)) {
                        report_error(g.status, KLEOS_AT_GEMM_MMA, t, (int)g.epoch);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(tiles + s * STAGE_BYTES);
                    const uint64_t da = make_smem_desc(sa);
                    const uint64_t db = make_smem_desc(sa + A_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // advancing K by 16 bf16 = 32 bytes inside the swizzled row: +2 in the
                        // descriptor's 16-byte address units
                        umma_bf16(d_tmem, da + 2 * k, db + 2 * k, kInstrDesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(&ctl->empty[s]);  // stage is free once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&ctl->acc_full[buf]);
            }
            if (g.stats) {
                g.stats[blockIdx.x * kStatSlots + 2] = w_acc;
                g.stats[blockIdx.x * kStatSlots + 3] = w_full;
                g.stats[blockIdx.x * kStatSlots + 4] = clock64() - t_begin;
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------------------------------------ epilogue
        const int q = warp - 4;
        const int row = q * 32 + lane;
        const TE* bias = static_cast<const TE*>(g.bias);
        uint32_t tile_n = 0;
        long long w_accfull = 0, w_tmem = 0;
        const long long t_begin = clock64();
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++tile_n) {
            TileCoord tcd;
            if (!decode_tile(t, ctl->le_start, g.le_begin, g.le_end, NT, &tcd)) break;
            const PanelEntry p = g.panels[tcd.panel];
            const uint32_t buf = tile_n & 1, use = tile_n >> 1;
            if (*abort_flag) break;
            {
                // stage this tile's 256 bias values in shared memory (one private copy per warp,
                // one 16-byte load per lane) while the main loop of the tile is still running:
                // global loads issued later would queue behind the operand traffic streaming
                // into this SM
                const int nb = tcd.nt * BN + 8 * lane;
                float* bs = &ctl->bias_s[buf][q][8 * lane];
                if (nb < g.N) {
                    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(
                        bias + (size_t)tcd.le * g.N + nb));
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
            const int n0 = tcd.nt * BN;
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
            TE* orow = (row < p.rows) ? out_ptr<TE>(g, p, row, n0) : nullptr;
            // accumulator read-back, two 32-column chunks in flight; bias fetched as 16-byte
            // broadcast loads
            uint32_t r[2][32];
            tmem_ld_32x32(taddr, r[0]);
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                const long long tq = clock64();
                tmem_ld_wait();
                w_tmem += clock64() - tq;
                if (c + 1 < BN / 32) tmem_ld_32x32(taddr + (c + 1) * 32, r[(c + 1) & 1]);
                if (orow != nullptr && n0 + c * 32 < g.N) {
                    const uint32_t* rc = r[c & 1];
                    const float4* bq = reinterpret_cast<const float4*>(&ctl->bias_s[buf][q][c * 32]);
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
                    uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        dst[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2],
                                            packed[4 * j + 3]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
        }
        if (g.stats && warp == 4 && lane == 0) {
            g.stats[blockIdx.x * kStatSlots + 5] = w_accfull;
            g.stats[blockIdx.x * kStatSlots + 6] = clock64() - t_begin;
            g.stats[blockIdx.x * kStatSlots + 7] = w_tmem;
        }
    }

    // teardown: everyone meets, then the allocating warp releases tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(TMEM_COLS)
                     : "memory");
    }
    if (g.mode == 1) publish_return_flags(g.ret, &last_block);
}

}  // namespace kleos
