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

namespace kleos {
namespace tc {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16, STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int TMEM_COLS = 512;              // two 128x256 fp32 accumulators
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 2048 /*control*/;

struct Control {
    unsigned long long full[STAGES];
    unsigned long long empty[STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    uint32_t tmem_base;
    int abort;
    int le_start[257];
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the budget ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity,
                                          long long budget, volatile int* abort) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*abort || clock64() - t0 > budget) return false;
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y,
                                            unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y),
        "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128 B apart, groups of
// 8 rows 1024 B apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);   // start address, bits [0,14)
    d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;                      // version
    d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
    return d;
}

// Instruction descriptor: D fp32, A/B bf16, both K-major, M = 128, N = 256.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                (static_cast<uint32_t>(BN >> 3) << 17) |
                                (static_cast<uint32_t>(BM >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(kInstrDesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread = lane = row).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace tc

__global__ void __launch_bounds__(256, 1)
ffn_gemm_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            GemmArgs g) {
    using namespace tc;
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
    const int total = ctl->le_start[g.nLx] * NT;
    const int KB = g.Kd / BK;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // dispatched rows and y1 rows were written with ordinary stores (possibly by a
            // peer GPU); order them before this thread's async-proxy reads
            asm volatile("fence.proxy.async;" ::: "memory");
            uint32_t it = 0;
            for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x) {
                TileCoord tcd;
                if (!decode_tile(t, ctl->le_start, g.nLx, NT, &tcd)) break;
                const PanelEntry p = g.panels[tcd.panel];
                const int brow = tcd.le * g.N + tcd.nt * BN;
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&ctl->empty[s], ph ^ 1, g.wait_cycles, abort_flag)) {
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
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, tile_n = 0;
            for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x, ++tile_n) {
                const uint32_t buf = tile_n & 1, use = tile_n >> 1;
                if (!mbar_wait(&ctl->acc_empty[buf], (use & 1) ^ 1, g.wait_cycles, abort_flag)) {
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
                    if (!mbar_wait(&ctl->full[s], ph, g.wait_cycles, abort_flag)) {
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
                        umma_bf16(d_tmem, da + 2 * k, db + 2 * k, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(&ctl->empty[s]);  // stage is free once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&ctl->acc_full[buf]);
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------------------------------------ epilogue
        const int q = warp - 4;
        const int row = q * 32 + lane;
        const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(g.bias);
        uint32_t tile_n = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++tile_n) {
            TileCoord tcd;
            if (!decode_tile(t, ctl->le_start, g.nLx, NT, &tcd)) break;
            const PanelEntry p = g.panels[tcd.panel];
            const uint32_t buf = tile_n & 1, use = tile_n >> 1;
            if (*abort_flag) break;
            if (!mbar_wait(&ctl->acc_full[buf], use & 1, g.wait_cycles, abort_flag)) {
                if (lane == 0) report_error(g.status, KLEOS_AT_GEMM_EPILOGUE, t, (int)g.epoch);
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const int n0 = tcd.nt * BN;
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
            __nv_bfloat16* orow = (row < p.rows) ? out_ptr<__nv_bfloat16>(g, p, row, n0) : nullptr;
            const __nv_bfloat16* brow = bias + (size_t)tcd.le * g.N + n0;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_ld_wait();
                if (orow != nullptr && n0 + c * 32 < g.N) {
                    uint32_t packed[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float v0 = __uint_as_float(r[2 * j]) + __bfloat162float(brow[c * 32 + 2 * j]);
                        float v1 = __uint_as_float(r[2 * j + 1]) +
                                   __bfloat162float(brow[c * 32 + 2 * j + 1]);
                        if (g.mode == 0) {
                            v0 = apply_act(v0, g.hidden_act);
                            v1 = apply_act(v1, g.hidden_act);
                        }
                        const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
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
