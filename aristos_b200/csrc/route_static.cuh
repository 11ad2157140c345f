// kleos_route_static: the router for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a routing
// decision: code running inside a framework's memory-pool callback, a real-time serving loop
// that has pinned its memory budget up front, or a process whose allocator is owned by another
// runtime.  The regular path (kleos_initialize + kleos_forward) allocates its bookkeeping once
// at initialise time; this entry point needs no initialise call at all.  The router's scratch
// (the list of near-tie tokens, their fp64 logits, completion counters, a zero bias) lives in
// the fixed array below, which every GPU that loads the library holds until the process exits.
//
// This file is compiled as part of kleos_api.cu (one translation unit), so the array, the
// cudaGetSymbolAddress call and the launches below all see the same symbol.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>

#include "route.cuh"

namespace {

constexpr int kStaticMaxTokens = 4096;  // S limit
constexpr int kStaticMaxExperts = 64;   // E limit (one 64-wide gate tile)
constexpr int kMaxDevices = 64;

// Layout of the scratch array (byte offsets, all 256-byte aligned).
constexpr size_t kOffCount = 0;                                                // int
constexpr size_t kOffDone = 256;                                               // int[S]
constexpr size_t kOffList = kOffDone + sizeof(int) * kStaticMaxTokens;         // int[S]
constexpr size_t kOffZeroBias = kOffList + sizeof(int) * kStaticMaxTokens;     // float[E], stays 0
constexpr size_t kClearBytes = kOffZeroBias + 256;                             // cleared every call
constexpr size_t kOffLogits = kClearBytes;                                     // double[S*E]
constexpr size_t kScratchBytes =
    kOffLogits + sizeof(double) * kStaticMaxTokens * kStaticMaxExperts;
static_assert(kScratchBytes == 2130432, "the size quoted in kleos_b200.h and in the documentation");

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_route_scratch[kScratchBytes];

unsigned char* g_scratch_ptr[kMaxDevices] = {};

int complain(int code, const char* what) {
    std::fprintf(stderr, "[kleos_b200] kleos_route_static: %s\n", what);
    return code;
}

}  // namespace

extern "C" int kleos_route_static(const void* A, const void* Wg, const float* gate_bias, int S,
                                  int H, int E, int K, int torch_dtype, void* probs,
                                  int32_t* topk, float* mcw, void* stream) {
    using namespace kleos;
    if (!A || !Wg || !probs || !topk || !mcw) return complain(KLEOS_E_ARG, "null device pointer");
    // the near-tie re-evaluation reads rows of A and Wg sixteen bytes at a time
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Wg)) & 15)
        return complain(KLEOS_E_ARG, "A and Wg must be 16-byte aligned");
    if (S < 1 || S > kStaticMaxTokens)
        return complain(KLEOS_E_ARG, "S exceeds the 4096-token limit of the fixed scratch array");
    if (E < 1 || E > kStaticMaxExperts)
        return complain(KLEOS_E_ARG, "E exceeds the 64-expert limit of the fixed scratch array");
    if (K < 1 || K > E || K > kMaxTopK) return complain(KLEOS_E_ARG, "top-k out of range");
    if (H < 64 || H % 64) return complain(KLEOS_E_ARG, "H must be a positive multiple of 64");
    if (torch_dtype != 0 && torch_dtype != 2)
        return complain(KLEOS_E_UNSUPPORTED, "torch_dtype must be 0 (float) or 2 (bf16)");  // fp16: use the layer API

    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return complain(KLEOS_E_CUDA, "no current CUDA device");
    if (!g_scratch_ptr[dev]) {
        // one-time set-up for this device (do the first call outside any stream capture)
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_route_scratch);
        if (e != cudaSuccess || !p) {
            std::fprintf(stderr, "[kleos_b200] cudaGetSymbolAddress failed: %s\n",
                         cudaGetErrorString(e));
            return KLEOS_E_CUDA;
        }
        g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
    }
    unsigned char* scratch = g_scratch_ptr[dev];
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : cudaStreamPerThread;

    // the counter, the completion flags and the zero bias must start at zero; the previous
    // call (or an aborted one) may have left anything there
    if (cudaMemsetAsync(scratch, 0, kClearBytes, st) != cudaSuccess)
        return complain(KLEOS_E_CUDA, "cudaMemsetAsync on the scratch array failed");

    RouteArgs ra{};
    ra.A = A;
    ra.Wg = Wg;
    ra.bias = gate_bias ? gate_bias : reinterpret_cast<const float*>(scratch + kOffZeroBias);
    ra.probs = probs;
    ra.topk = topk;
    ra.mcw = mcw;
    ra.refine_count = reinterpret_cast<int*>(scratch + kOffCount);
    ra.refine_done = reinterpret_cast<int*>(scratch + kOffDone);
    ra.refine_list = reinterpret_cast<int*>(scratch + kOffList);
    ra.refine_logits = reinterpret_cast<double*>(scratch + kOffLogits);
    ra.S = S;
    ra.H = H;
    ra.E = E;
    ra.K = K;
    ra.PX = 64;
    ra.tie_eps = 1e-4f;
    const int grid = (S + 63) / 64;
    if (torch_dtype == 0) {
        route_kernel<float, 64><<<grid, 256, route_smem_bytes<64>(), st>>>(ra);
        refine_kernel<float><<<148, 256, 0, st>>>(ra);
    } else {
        route_kernel<__nv_bfloat16, 64><<<grid, 256, route_smem_bytes<64>(), st>>>(ra);
        refine_kernel<__nv_bfloat16><<<148, 256, 0, st>>>(ra);
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        std::fprintf(stderr, "[kleos_b200] kleos_route_static launch failed: %s\n",
                     cudaGetErrorString(e));
        return KLEOS_E_CUDA;
    }
    return KLEOS_OK;
}
