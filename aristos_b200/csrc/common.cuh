// Shared device helpers: element types, status reporting, bounded waits, system-scope flags.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/kleos_b200.h"

namespace kleos {

constexpr int kTileM = 128;        // rows per expert-cell tile (reference BLOCK_M, types.cuh:38-42)
constexpr int kMaxWorld = 8;       // one NVSwitch node
constexpr int kMaxTopK = 8;
constexpr int kDropped = -1;

// Device-resident status record; first error wins.
struct DeviceStatus {
    int code;
    int where;
    int detail;
    int epoch;
};

__device__ __forceinline__ void report_error(DeviceStatus* st, int where, int detail, int epoch) {
    if (atomicCAS(&st->code, 0, KLEOS_E_DEVICE) == 0) {
        st->where = where;
        st->detail = detail;
        st->epoch = epoch;
        __threadfence();
    }
}

// ---------------------------------------------------------------- element conversion
template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float v) { return v; }
    static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float round(float v) {
        return __bfloat162float(__float2bfloat16_rn(v));
    }
};

template <> struct Elem<__half> {
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
};

// TF32 element (torch_dtype 1): an fp32 word whose low 13 mantissa bits are zero, the storage the
// reference uses for cute::tfloat32_t (types.cuh:128-131).  Rounding is to nearest, ties to even.
struct tf32_t {
    float v;
};
__host__ __device__ __forceinline__ float round_tf32(float x) {
#ifdef __CUDA_ARCH__
    uint32_t u = __float_as_uint(x);
#else
    uint32_t u;
    memcpy(&u, &x, 4);
#endif
    if ((u & 0x7f800000u) != 0x7f800000u) u = (u + 0xfffu + ((u >> 13) & 1u)) & 0xffffe000u;
#ifdef __CUDA_ARCH__
    return __uint_as_float(u);
#else
    float r;
    memcpy(&r, &u, 4);
    return r;
#endif
}
template <> struct Elem<tf32_t> {
    static __device__ __forceinline__ float to_f(tf32_t v) { return v.v; }
    static __device__ __forceinline__ tf32_t from_f(float v) { return tf32_t{round_tf32(v)}; }
    static __device__ __forceinline__ float round(float v) { return round_tf32(v); }
};

// Packed pairs of a 16-bit element type: conversions and single-rounding arithmetic, plus the
// operand-format code of the tcgen05 instruction descriptor (0 = f16, 1 = bf16).
template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
    using type = __nv_bfloat162;
    static constexpr uint32_t kMmaFormat = 1;
    static __device__ __forceinline__ type from_f2(float a, float b) { return __floats2bfloat162_rn(a, b); }
    static __device__ __forceinline__ float2 to_f2(type v) { return __bfloat1622float2(v); }
    static __device__ __forceinline__ type mul(type a, type b) { return __hmul2(a, b); }
    static __device__ __forceinline__ type add(type a, type b) { return __hadd2(a, b); }
};
template <> struct Pack2<__half> {
    using type = __half2;
    static constexpr uint32_t kMmaFormat = 0;
    static __device__ __forceinline__ type from_f2(float a, float b) { return __floats2half2_rn(a, b); }
    static __device__ __forceinline__ float2 to_f2(type v) { return __half22float2(v); }
    static __device__ __forceinline__ type mul(type a, type b) { return __hmul2(a, b); }
    static __device__ __forceinline__ type add(type a, type b) { return __hadd2(a, b); }
};

__device__ __forceinline__ float apply_act(float z, int hidden_act) {
    // 0: ReLU, 1: GELU (erf form), as selected by hidden_act (reference types.cuh:143-159);
    // 2: identity (second GEMM of the dense layer)
    if (hidden_act == 0) return fmaxf(z, 0.f);
    if (hidden_act == 2) return z;
    return 0.5f * z * (1.f + erff(z * 0.70710678118654752f));
}

// ---------------------------------------------------------------- system-scope flags
// A flag word is (epoch << 32) | payload.  Writers store it with release semantics after
// their data stores; readers poll with acquire semantics.  Epochs only grow, so flags never
// need clearing between forwards (the reference cycles a 16-bit sequence number for the same
// purpose, types.cuh:1046-1064).
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long make_flag(uint32_t epoch, uint32_t payload) {
    return (static_cast<unsigned long long>(epoch) << 32) | payload;
}

// Poll until the flag carries `epoch`; gives up after `budget` clock cycles.
__device__ __forceinline__ bool wait_flag(const unsigned long long* flag, uint32_t epoch,
                                          long long budget, unsigned long long* value) {
    const long long t0 = clock64();
    for (;;) {
        const unsigned long long v = ld_acquire_sys(flag);
        if (static_cast<uint32_t>(v >> 32) == epoch) {
            *value = v;
            return true;
        }
        if (clock64() - t0 > budget) return false;
        __nanosleep(64);
    }
}

// 16-byte global accesses.  Loads of data a peer may have written go through L2 (.cg).
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

struct PeerTable {
    char* arena[kMaxWorld];  // base of every rank's symmetric arena as mapped in this process
};

}  // namespace kleos
