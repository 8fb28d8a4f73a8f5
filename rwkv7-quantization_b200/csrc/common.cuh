// Shared device helpers and host-side error plumbing of librwkvq (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/rwkvq.h"

namespace rwkvq {

// ----------------------------------------------------------------------------- host side
extern thread_local char g_err[512];
extern std::atomic<int64_t> g_launches;

int32_t fail(int32_t code, const char* fmt, ...);
int32_t check_launch(const char* what);   // cudaGetLastError() -> status, counts the launch
int sm_count();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define RWKVQ_REQUIRE(cond, code, ...) \
    do {                               \
        if (!(cond)) return ::rwkvq::fail(code, __VA_ARGS__); \
    } while (0)

// ----------------------------------------------------------------------------- device side
__device__ __forceinline__ float div_full(float a, float b) {
    float r;
    asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float div_mode_f32(float a, float b, int mode) {
    return mode == RWKVQ_DIV_FULL ? div_full(a, b) : __fdiv_rn(a, b);
}

template <int DT>
__device__ __forceinline__ float2 cvt2(uint32_t v) {   // two packed 16-bit values -> fp32
    if (DT == RWKVQ_F16) {
        return __half22float2(*reinterpret_cast<const __half2*>(&v));
    } else {
        return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
    }
}
__device__ __forceinline__ float bf16_round(float v) {  // fp32 -> bf16 (RNE) -> fp32
    return __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}
// two fp32 -> two e4m3 bytes (lo in bits 0-7), round-to-nearest-even, saturating.  One hardware instruction
// (written as PTX: the cuda_fp8.h helper may pick its software path, hundreds of instructions per pair).
__device__ __forceinline__ uint32_t e4m3x2(float lo, float hi) {
    unsigned short r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return (uint32_t)r;
}
// two e4m3 bytes (bits 0-15) -> two f16 (exact), low byte in the low half
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_codes) {
    uint32_t r;
    const unsigned short c = (unsigned short)two_codes;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(c));
    return r;
}
__device__ __forceinline__ float clamp448(float v) { return fminf(fmaxf(v, -448.f), 448.f); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// streaming 128-bit weight load: read-only path, do not keep the line in L1
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// atomic max of a non-negative float through its bit pattern
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
    atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}

}  // namespace rwkvq
