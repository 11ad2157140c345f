// Expert-FFN GEMM for TF32 layers (torch_dtype 1) on the 5th-generation tensor cores:
// tcgen05.mma kind::tf32 over 4-byte operands staged by TMA (128-byte swizzle, 32 elements per
// row), 128x256 fp32 accumulator in tensor memory, double-buffered, read back with tcgen05.ld.
// Same block roles and bounded waits as the 16-bit GEMM (gemm_tc2.cuh) without the pairing; the differences are the
// operand width (K slices of 32 elements, 8 per instruction), the 4-byte epilogue (bias read as
// fp32 words, results rounded to TF32, each lane storing whole 128-byte lines of its own row)
// and the instruction descriptor.
//
// Replaces the reference's mma.sync m16n8k8 TF32 block GEMM (os/processor/mmaConfig.cuh:73-81,
// os/processor/gemm.cuh:58-107) and its fused bias + activation epilogue (gemm.cuh:23-50).
#pragma once

#include <cuda.h>

#include "gemm_common.cuh"
#include "tc_common.cuh"

namespace kleos {
namespace gemm_tf32 {
using namespace tc;

constexpr int BM = 128, BN = 256, BK = 32, UMMA_K = 8, STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 4;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 4;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int TMEM_COLS = 512;              // two 128x256 fp32 accumulators
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 12288 /*control*/;

constexpr uint32_t kInstrDesc = make_instr_desc_tf32(BM, BN);

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

}  // namespace gemm_tf32

// kEpi: 0 bias + ReLU, 1 bias + GELU, 2 bias only.
template <int kEpi>
__global__ void __launch_bounds__(256, 1)
ffn_gemm_tf32(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
              GemmArgs g) {
    using namespace tc;
    using namespace gemm_tf32;
    using TE = tf32_t;
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
                        // advancing K by 8 elements = 32 bytes inside the swizzled row: +2 in the
                        // descriptor's 16-byte address units
                        umma_tf32(d_tmem, da + 2 * k, db + 2 * k, kInstrDesc, (kb | k) != 0 ? 1u : 0u);
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
        const float* bias = static_cast<const float*>(g.bias);
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
                // two 16-byte loads per lane) while the main loop of the tile is still running
                const int nb = tcd.nt * BN + 8 * lane;
                float4* bs = reinterpret_cast<float4*>(&ctl->bias_s[buf][q][8 * lane]);
                if (nb < g.N) {
                    const float4* src = reinterpret_cast<const float4*>(bias + (size_t)tcd.le * g.N + nb);
                    bs[0] = __ldg(src);
                    bs[1] = __ldg(src + 1);
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
                    uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 bf = bq[j];
                        float v[4] = {__uint_as_float(rc[4 * j]) + bf.x, __uint_as_float(rc[4 * j + 1]) + bf.y,
                                      __uint_as_float(rc[4 * j + 2]) + bf.z, __uint_as_float(rc[4 * j + 3]) + bf.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if constexpr (kEpi == 0) v[i] = fmaxf(v[i], 0.f);
                            else if constexpr (kEpi == 1) v[i] = apply_act(v[i], 1);
                            v[i] = round_tf32(v[i]);
                        }
                        dst[j] = make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]),
                                            __float_as_uint(v[2]), __float_as_uint(v[3]));
                    }
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
