// Expert-FFN GEMM on the FP32 pipes: 128x128x16 block tile, 256 threads, 8x8 register tile.
//
// This is the path for torch_dtype 0 (float): the reference also runs float on scalar FMA,
// not on tensor cores (os/processor/mmaConfig.cuh:19-26), and fp32 FMA is what keeps the
// layer output within 1e-5 of the fp64 oracle.  It is also instantiated for bf16 as a
// debugging cross-check of the tensor-core kernel.
#pragma once

#include "gemm_common.cuh"

namespace kleos {

template <typename T>
__global__ void __launch_bounds__(256) ffn_gemm_simt(GemmArgs g) {
    constexpr int BN = 128, BK = 16, LD = 132;  // 128-row panels x 128 columns x 16-deep K steps
    __shared__ __align__(16) float As[BK][LD];
    __shared__ __align__(16) float Bs[BK][LD];
    __shared__ int le_start_s[257];
    __shared__ bool last_block;

    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    for (int i = tid; i <= g.nLx; i += 256) le_start_s[i] = g.le_start[i];
    __syncthreads();
    const int NT = (g.N + BN - 1) / BN;
    const int total = (le_start_s[g.le_end] - le_start_s[g.le_begin]) * NT;
    const T* A = static_cast<const T*>(g.A);
    const T* B = static_cast<const T*>(g.B);
    const T* bias = static_cast<const T*>(g.bias);
    const int lrow = tid >> 1, lk = (tid & 1) * 8;

    for (int t = blockIdx.x; t < total; t += gridDim.x) {
        TileCoord tc;
        if (!decode_tile(t, le_start_s, g.le_begin, g.le_end, NT, &tc)) break;
        const PanelEntry p = g.panels[tc.panel];
        const int n0 = tc.nt * BN;
        const T* arow = A + (size_t)(p.row_base + lrow) * g.Kd;
        const bool brow_ok = (n0 + lrow) < g.N;
        const T* brow = B + ((size_t)tc.le * g.N + n0 + lrow) * g.Kd;

        float acc[8][8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

        // software pipeline: the global loads of K step k+1 are in flight while step k is
        // multiplied out of shared memory
        float av[8], bv[8];
        auto fetch = [&](int k0) {
            // eight consecutive K elements per thread, as 16-byte loads
            constexpr int NV = 8 * sizeof(T) / 16;
            uint4 ra[NV], rb[NV];
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                ra[v] = __ldg(reinterpret_cast<const uint4*>(arow + k0 + lk) + v);
                rb[v] = brow_ok ? __ldg(reinterpret_cast<const uint4*>(brow + k0 + lk) + v)
                                : make_uint4(0u, 0u, 0u, 0u);
            }
            const T* ea = reinterpret_cast<const T*>(ra);
            const T* eb = reinterpret_cast<const T*>(rb);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                av[i] = Elem<T>::to_f(ea[i]);
                bv[i] = Elem<T>::to_f(eb[i]);
            }
        };
        fetch(0);
        for (int k0 = 0; k0 < g.Kd; k0 += BK) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                As[lk + i][lrow] = av[i];
                Bs[lk + i][lrow] = bv[i];
            }
            __syncthreads();
            if (k0 + BK < g.Kd) fetch(k0 + BK);
#pragma unroll
            for (int k = 0; k < BK; ++k) {
                const float4 a0 = *reinterpret_cast<const float4*>(&As[k][ty * 8]);
                const float4 a1 = *reinterpret_cast<const float4*>(&As[k][ty * 8 + 4]);
                const float4 b0 = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
                const float4 b1 = *reinterpret_cast<const float4*>(&Bs[k][64 + tx * 4]);
                const float ar[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const float br[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
            }
            __syncthreads();
        }
        // epilogue: bias, activation (GEMM1), round, store valid rows / columns
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = ty * 8 + i;
            if (r >= p.rows) continue;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
                if (n >= g.N) continue;
                float v = acc[i][j] + Elem<T>::to_f(bias[(size_t)tc.le * g.N + n]);
                if (g.mode == 0) v = apply_act(v, g.hidden_act);
                *out_ptr<T>(g, p, r, n) = Elem<T>::from_f(v);
            }
        }
    }
    if (g.mode == 1) publish_return_flags(g.ret, &last_block);
}

}  // namespace kleos
