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
// wall-time limit of every bounded device-side wait, nanoseconds: 1.5 s unless RWKVQ_WAIT_LIMIT_US (read once) or
// rwkvq_set_wait_limit_us changed it
unsigned long long wait_limit_ns();
// per kernel and device: opt in to `bytes` of dynamic shared memory (once)
int32_t ensure_smem_optin(const void* kern, int bytes, const char* who);
// per (kernel, device, dynamic shared memory size): the opt-in above plus the resident CTAs per SM, looked up once
int32_t kernel_plan(const void* kern, int threads, size_t smem, int optin_bytes, int* per_sm, const char* who);
// programmatic dependent launch unless RWKVQ_PDL=0 (read once)
bool use_pdl();
// The library's per-device status word (device address): kernels whose entry points take no status pointer set it to
// RWKVQ_E_TIMEOUT when a bounded wait gives up; rwkvq_device_status reads it.  Null if the lookup failed.
int* device_status_ptr();

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

// qmax / amax and amax / qmax of the activation scales.  RWKVQ_DIV_TORCH: what torch's GPU kernels compute for
// `scalar / tensor` (reciprocal, then a product) and `tensor / scalar` (product with the rounded reciprocal).
__device__ __forceinline__ float scale_inv(float qmax, float amax, int mode) {
    if (mode == RWKVQ_DIV_TORCH) return __fmul_rn(__frcp_rn(amax), qmax);
    return div_mode_f32(qmax, amax, mode);
}
__device__ __forceinline__ float scale_fwd(float amax, float qmax, int mode) {
    if (mode == RWKVQ_DIV_TORCH) return __fmul_rn(amax, __frcp_rn(qmax));
    return div_mode_f32(amax, qmax, mode);
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

// two floats -> one byte of two e2m1 codes (lo in the low nibble), round-to-nearest-even, saturating
__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
    unsigned short r;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(r) : "f"(hi), "f"(lo));
    return (uint32_t)r;
}
// one byte of two e2m1 codes -> f16 pair (low nibble in the low half), exact
__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(uint32_t byte) {
    uint32_t r;
    const unsigned short b = (unsigned short)(byte & 0xffu);
    asm("{ .reg .b8 t; cvt.u8.u16 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(r) : "h"(b));
    return r;
}
__device__ __forceinline__ float e4m3_to_float(uint32_t code) {
    const uint32_t h2 = e4m3x2_to_f16x2(code & 0xffu);
    return __half2float(__ushort_as_half((unsigned short)(h2 & 0xffffu)));
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

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
    return t;
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait for *p == want (a flag another CTA of the same cooperative launch publishes with st_release_u32).
// The clock costs hundreds of nanoseconds to read, so it is consulted only after a few hundred failed polls.
__device__ __forceinline__ bool wait_flag_eq(const uint32_t* p, uint32_t want, unsigned long long limit_ns) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i) {
        if (ld_acquire_u32(p) == want) return true;
        __nanosleep(64);
    }
    const unsigned long long t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i) {
            if (ld_acquire_u32(p) == want) return true;
            __nanosleep(128);
        }
        if (global_ns() - t0 > limit_ns) return false;
    }
}

// atomic max of a non-negative float through its bit pattern
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
    atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}

}  // namespace rwkvq
