// Router on the tensor cores (bf16 / fp16 / tf32 layers): gate GEMM with the whole padded expert
// dimension as one tcgen05 N extent, softmax + top-k in the accumulator read-back.  A K slice is
// always 128 bytes wide (64 16-bit or 32 4-byte elements, the swizzle span), four instructions
// per slice.
//
// One block per 128 tokens.  The accumulator is 128 lanes x PX fp32 columns of tensor memory,
// so every epilogue thread owns one token's full logit row and no cross-block exchange is
// needed; the reference needs a ring of mailboxes between column-tile blocks once E > 64
// (moe/gate.cuh:93-468).  Selection rules are those of route.cuh / moe/gate.cuh:556-718.
#pragma once

#include "route.cuh"
#include "tc_common.cuh"

namespace kleos {
namespace route_tc {

constexpr int BM = 128, BK = 64, UMMA_K = 16, MAX_STAGES = 6;
constexpr int A_STAGE_BYTES = BM * BK * 2;

template <int PXT>
struct Shape {
    static constexpr int STAGES = PXT <= 64 ? 6 : 4;  // what fits beside the logit tile
    static constexpr int B_STAGE_BYTES = PXT * BK * 2;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr int LDL = PXT + 1;
    static constexpr int LOGIT_BYTES = BM * LDL * 4 + 2 * BM * 4;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + LOGIT_BYTES + 1024 + 256;
};

struct Control {
    unsigned long long full[MAX_STAGES];
    unsigned long long empty[MAX_STAGES];
    unsigned long long acc_full;
    uint32_t tmem_base;
    int abort;
};

}  // namespace route_tc

template <typename TE, int PXT>
__global__ void __launch_bounds__(256, 1)
route_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_wg,
                RouteArgs a, DeviceStatus* status, long long wait_cycles, int epoch) {
    using namespace tc;
    using namespace route_tc;
    using Sh = Shape<PXT>;
    constexpr int STAGES = Sh::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    float* Ls = reinterpret_cast<float*>(tiles + STAGES * Sh::STAGE_BYTES);  // [BM][LDL]
    float* rowmax = Ls + BM * Sh::LDL;
    float* rowden = rowmax + BM;
    Control* ctl = reinterpret_cast<Control*>(rowden + BM);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int* abort_flag = &ctl->abort;
    const int row0 = blockIdx.x * BM;
    constexpr bool kWide = sizeof(TE) == 4;            // tf32: fp32 words
    constexpr int BKE = 128 / (int)sizeof(TE);         // elements per K slice
    const int KB = a.H / BKE;
    uint32_t idesc;
    if constexpr (kWide) idesc = make_instr_desc_tf32(BM, PXT);
    else idesc = make_instr_desc_16b(BM, PXT, Pack2<TE>::kMmaFormat);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        mbar_init(&ctl->acc_full, 1);
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&ctl->tmem_base)), "r"(PXT)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < KB; ++kb) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(&ctl->empty[s], ph ^ 1, wait_cycles, abort_flag)) {
                    report_error(status, KLEOS_AT_GEMM_PRODUCER, blockIdx.x, epoch);
                    *abort_flag = 1;
                    break;
                }
                mbar_expect_tx(&ctl->full[s], Sh::STAGE_BYTES);
                uint8_t* sa = tiles + s * Sh::STAGE_BYTES;
                tma_load_2d(sa, &map_a, kb * BKE, row0, &ctl->full[s]);
                tma_load_2d(sa + A_STAGE_BYTES, &map_wg, kb * BKE, 0, &ctl->full[s]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int kb = 0; kb < KB; ++kb) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(&ctl->full[s], ph, wait_cycles, abort_flag)) {
                    report_error(status, KLEOS_AT_GEMM_MMA, blockIdx.x, epoch);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_u32(tiles + s * Sh::STAGE_BYTES);
                const uint64_t da = make_smem_desc(sa);
                const uint64_t db = make_smem_desc(sa + A_STAGE_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {  // four 32-byte steps per slice
                    if constexpr (kWide) umma_tf32(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    else umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                }
                umma_commit(&ctl->empty[s]);
            }
            if (ok) umma_commit(&ctl->acc_full);
        }
        __syncwarp();
    } else if (warp >= 4) {
        const int q = warp - 4;
        const int r = q * 32 + lane;  // token row inside the tile = accumulator lane
        bool ok = mbar_wait(&ctl->acc_full, 0, wait_cycles, abort_flag);
        if (!ok) {
            if (lane == 0) report_error(status, KLEOS_AT_GEMM_EPILOGUE, blockIdx.x, epoch);
            *abort_flag = 1;
        }
        tc_fence_after();
        if (ok) {
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < PXT / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(taddr + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int e = c * 32 + j;
                    Ls[r * Sh::LDL + e] = __uint_as_float(v[j]) + (e < a.E ? a.bias[e] : 0.f);
                }
            }
            tc_fence_before();
            if (row0 + r < a.S) {
                const RowDecision d = decide_row(Ls + r * Sh::LDL, a.E, a.K,
                                                 a.topk + (size_t)(row0 + r) * a.K,
                                                 a.mcw + row0 + r);
                rowmax[r] = d.max;
                rowden[r] = d.inv_den;
                if (d.margin < a.tie_eps * fmaxf(1.f, fabsf(d.kth))) {
                    const int pos = atomicAdd(a.refine_count, 1);
                    a.refine_list[pos] = row0 + r;
                }
            }
        }
        // the four epilogue warps share the logit tile: meet before the coalesced store
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ok && !*abort_flag) {
            TE* probs = static_cast<TE*>(a.probs);
            const int et = tid - 128;
            // two adjacent probabilities per thread, 4-byte stores (PX == PXT); 256 % PXT == 0,
            // so a thread always visits the same two expert columns
            float cs0 = 0.f, cs1 = 0.f;
            for (int idx = 2 * et; idx < BM * PXT; idx += 256) {
                const int rr = idx / PXT, e = idx % PXT;
                if (row0 + rr >= a.S) break;
                const float m = rowmax[rr], inv = rowden[rr];
                const float p0 = e < a.E ? __expf(Ls[rr * Sh::LDL + e] - m) * inv : 0.f;
                const float p1 = e + 1 < a.E ? __expf(Ls[rr * Sh::LDL + e + 1] - m) * inv : 0.f;
                cs0 += p0;
                cs1 += p1;
                TE* dst = probs + (size_t)(row0 + rr) * PXT + e;
                if constexpr (kWide) {
                    *reinterpret_cast<float2*>(dst) = make_float2(round_tf32(p0), round_tf32(p1));
                } else {
                    *reinterpret_cast<typename Pack2<TE>::type*>(dst) = Pack2<TE>::from_f2(p0, p1);
                }
            }
            // training mode: stash this thread's two column sums of the fp32 probabilities in
            // the operand stages (free once the accumulator is full)
            if (a.col_partial != nullptr) {
                float* cs = reinterpret_cast<float*>(tiles);
                cs[2 * et] = cs0;
                cs[2 * et + 1] = cs1;
            }
        }
        if (a.col_partial != nullptr) {
            // every epilogue thread takes part in the barrier, also after a failed wait
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int et = tid - 128;
            if (ok && !*abort_flag && et < PXT) {
                const float* cs = reinterpret_cast<const float*>(tiles);
                float sum = 0.f;
                for (int k = 0; k < 256 / PXT; ++k) sum += cs[et + k * PXT];  // fixed order
                a.col_partial[(size_t)blockIdx.x * PXT + et] = sum;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(PXT)
                     : "memory");
    }
}

}  // namespace kleos
