// Shared pieces of the W8A8 (FP8 e4m3 / INT8) kernels: argument block, mma.sync wrappers and the activation
// quantization prologues that fill the shared-memory code tile.
#pragma once
#include "common.cuh"

namespace rwkvq {

constexpr int kWarps = 8;
constexpr int kThr = kWarps * 32;
constexpr int kUnroll = 4;   // any-M kernel: 64-byte units in flight per lane

enum { QT_FP8 = 0, QT_INT8 = 1 };

// Programmatic dependent launch: a kernel may start while its predecessor in the stream drains.  Everything
// before griddep_wait() may only touch data no earlier kernel writes (here: the weights).
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

struct W8Args {
    const void* x[3];         // fused: activations (x_dtype)
    const float* awq[3];      // fused FP8: optional per-channel divisor
    const uint8_t* w[3];
    const float* ws[3];       // weight scale (one fp32 each)
    __half* out[3];
    int32_t* acc[3];          // INT8: optional raw accumulators
    const uint8_t* a_codes;   // pre-quantized mode (any-M mma.sync kernel)
    const float* a_scale;     // pre-quantized: FP8 amax-or-scale [1], INT8 per-row scales [M]
    const uint8_t* codes[3];  // pre-quantized mode of the decode GEMV: activation codes [M, lda] per matrix
    const float* ascale[3];   //   and their scales (FP8: amax-or-scale [1]; INT8: per-row scales [M])
    int64_t ldx, ldw, ldo, ldacc, lda;
    int M, N, K, nmat;
    int div_mode, amax_is_amax;
    uint32_t flags;
    int pitch;                // fused: bytes between rows of the code tile in shared memory
    int lgR;                  // decode GEMV: log2 of the row tiles per round of a CTA (R = 1, 2, 4 or 8); 8/R warps share a tile
    int cpm;                  // decode GEMV: CTAs per matrix (grid = nmat * cpm)
    int tq, trem;             // decode GEMV: row tiles per CTA (quotient, remainder) within a matrix
    unsigned long long* trace;   // profiling aid: [grid][8] timestamps of the CTA's milestones, or null
    float* ffn_amax;             // RELU2: maximum of the relu^2 results (atomic max); AMAX_GIVEN: the amax to quantize with
    int* ffn_count;              // AMAX_GIVEN: CTAs that have read ffn_amax; the last one clears both words for the next pair
    int* status;                 // the library's per-device status word: RWKVQ_E_TIMEOUT if a bounded wait gave up
    unsigned long long wait_ns;  // wall-time limit of the bounded waits
};

// profiling aid, compiled in only with -DRWKVQ_TRACE (the decode kernels run for a few microseconds and every
// instruction between their entry and their first MMA shows in the launch time): thread 0 of a CTA stamps milestone
// `slot` (0..7) with the global timer when a trace buffer is set
__device__ __forceinline__ void w8_mark(const W8Args& a, int slot) {
#ifdef RWKVQ_TRACE
    if (a.trace && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
        a.trace[(size_t)blockIdx.x * 8 + slot] = t;
    }
#else
    (void)a; (void)slot;
#endif
}

template <int QT>
struct Acc { using T = float; };
template <>
struct Acc<QT_INT8> { using T = int32_t; };

__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8(int32_t (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <int QT, typename T>
__device__ __forceinline__ void mma8(T (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if constexpr (QT == QT_FP8) mma_e4m3(c, a0, a1, a2, a3, b0, b1);
    else mma_s8(c, a0, a1, a2, a3, b0, b1);
}

__device__ __forceinline__ float cta_max(float v, float* sh) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = sh[0];
#pragma unroll
    for (int i = 1; i < kWarps; ++i) r = fmaxf(r, sh[i]);
    __syncthreads();
    return r;
}

// ---- fused prologue, FP8: per-call amax then e4m3 codes into shared memory; returns max(amax, 1e-12).
// Up to 4 vectors of 8 activations per thread stay in registers between the two phases (M*K <= 8192, i.e. the
// M = 1 and M = 2 decode cases at K = 4096); larger calls read x a second time (L1/L2 hits).
// ---- per-vector helpers (8 activations = one uint4).  They are written for instruction count: every CTA of the
// decode kernels quantizes the whole activation block itself, so these few lines are executed by all SMs.

// |x| maximum of 8 packed 16-bit values, exact, with packed abs/max (two values per instruction)
template <int DT>
__device__ __forceinline__ float packed_absmax8(const uint4& v) {
    if constexpr (DT == RWKVQ_F16) {
        const __half2* h = reinterpret_cast<const __half2*>(&v);
        const __half2 m = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
        return fmaxf(__low2float(m), __high2float(m));
    } else {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
        const __nv_bfloat162 m = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
        return fmaxf(__low2float(m), __high2float(m));
    }
}

template <int DT>
__device__ __forceinline__ void fp8_vec_amax(const uint4& v, const float* awq, int k, int div_mode, bool after, float& m) {
    if (awq == nullptr && !(DT == RWKVQ_F16 && after)) {      // the common case: max over the raw 16-bit values
        m = fmaxf(m, packed_absmax8<DT>(v));
        return;
    }
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        float2 f = cvt2<DT>(w[q]);
        if (awq) {
            f.x = div_mode_f32(f.x, awq[k + 2 * q], div_mode);
            f.y = div_mode_f32(f.y, awq[k + 2 * q + 1], div_mode);
        }
        if (after) { f.x = bf16_round(f.x); f.y = bf16_round(f.y); }
        m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
}
// codes = e4m3_rn_sat(bf16(x [/ awq]) * inv): the saturating conversion is the clamp to +-448
template <int DT>
__device__ __forceinline__ uint2 fp8_vec_codes(const uint4& v, const float* awq, int k, int div_mode, float inv) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t c[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        float2 f = cvt2<DT>(w[q]);
        if (awq) {
            f.x = div_mode_f32(f.x, awq[k + 2 * q], div_mode);
            f.y = div_mode_f32(f.y, awq[k + 2 * q + 1], div_mode);
        }
        if (DT == RWKVQ_F16 || awq) { f.x = bf16_round(f.x); f.y = bf16_round(f.y); }   // bf16 input is its own rounding
        c[q] = e4m3x2(f.x * inv, f.y * inv);
    }
    return make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
}

// 8 e4m3 codes (uint2) -> the same 8 values as f16 (exact: every e4m3 value is an f16 value)
__device__ __forceinline__ uint4 e4m3x8_to_f16x8(uint2 c) {
    return make_uint4(e4m3x2_to_f16x2(c.x & 0xffffu), e4m3x2_to_f16x2(c.x >> 16), e4m3x2_to_f16x2(c.y & 0xffffu),
                      e4m3x2_to_f16x2(c.y >> 16));
}

// The decode GEMV keeps the quantized FP8 activations as f16 VALUES in shared memory (2 bytes per element): on sm_100
// mma.sync has no fast e4m3 path, so weights are widened to f16 in registers and multiplied with m16n8k16.f16
// (products of two e4m3 values and their fp32 sums are exact).
//
// The prologue runs once per CTA, straight after the dependency release, on cold instruction and data caches, and
// every CTA of a launch reads the same few kilobytes of activations at the same moment.  So it is written for few
// instructions and one read: thread 0 fetches the raw 16-bit rows with bulk copies (global -> shared, completion on
// an mbarrier, independent of the weight ring's cp.async groups) INTO the tile itself -- a raw row and its row of f16
// codes have the same size -- and two short loops (abs-max, then convert in place) work from shared memory.
// `bar` must have been initialised with count 1 and made visible to the CTA.  If the copy has not landed within the
// wait limit the CTA reports RWKVQ_E_TIMEOUT through the status word, gives the copy a second bounded wait (its target
// is the CTA's own shared memory) and stops without touching the tile or writing results.
__device__ __forceinline__ bool w8_bar_wait(uint64_t* bar, unsigned long long limit_ns) {
    const uint32_t b = (uint32_t)__cvta_generic_to_shared(bar);
    auto poll = [&](int n) {
#pragma unroll 1
        for (int i = 0; i < n; ++i) {
            uint32_t ok;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(b) : "memory");
            if (ok) return true;
        }
        return false;
    };
    if (poll(1 << 14)) return true;          // the clock is costly to read: only consulted after many failed polls
    const unsigned long long t0 = global_ns();
    for (;;) {
        if (poll(1 << 10)) return true;
        if (global_ns() - t0 > limit_ns) return false;
    }
}
// CTA-uniform verdict on a staging copy: true = landed for every thread; false = reported, the CTA must return
__device__ __forceinline__ bool w8_staged_or_report(uint64_t* bar, int* status, unsigned long long limit_ns) {
    const bool staged = w8_bar_wait(bar, limit_ns);
    if (__syncthreads_or(!staged)) {
        if (threadIdx.x == 0 && status) atomicExch(status, RWKVQ_E_TIMEOUT);
        if (!staged) w8_bar_wait(bar, limit_ns);
        return false;
    }
    return true;
}

// 128-bit load of activations served from L2 (they were written by an earlier kernel that may still have been running
// when this CTA started under programmatic dependent launch, so a line this SM's L1 kept from before is not trusted)
__device__ __forceinline__ uint4 ldg_l2_16(const void* p) {
    uint4 r;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
}

// Returns max(amax, 1e-12), or a negative value if the staging copy timed out (the CTA must then return).
// The tile holds the codes as f16 values (2 bytes each, no conversion in the K loop).
// GIVEN: the amax comes from a.ffn_amax (published by the kernel that produced x): no abs-max pass, no reduction.
template <int DT, bool WIDE, bool GIVEN = false>
__device__ float quantize_fp8_to_smem(const W8Args& a, int mat, uint8_t* xq, float* sh, uint64_t* bar) {
    const char* x = reinterpret_cast<const char*>(a.x[mat]);
    const float* awq = a.awq[mat];
    const int kv = a.K >> 3;                  // 8-element vectors per row
    const bool after = (a.flags & RWKVQ_FLAG_AMAX_AFTER_BF16) != 0;
    static_assert(WIDE, "the fused prologue fills the f16 tile; e4m3 tiles are filled from pre-quantized codes");
    const int nvec = a.M * kv;
    if (nvec <= 2 * kThr) {
        // one or two vectors per thread (M = 1 at K <= 4096): plain loads kept in registers are a little quicker
        // than the staging copy
        const int i0 = threadIdx.x, i1 = threadIdx.x + kThr;
        int r0 = 0, r1 = 0;
        if (a.M > 1) { r0 = i0 / kv; r1 = i1 / kv; }
        const int k0 = (i0 - r0 * kv) << 3, k1 = (i1 - r1 * kv) << 3;
        uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
        if (i0 < nvec) v0 = *reinterpret_cast<const uint4*>(x + ((int64_t)r0 * a.ldx + k0) * 2);
        if (i1 < nvec) v1 = *reinterpret_cast<const uint4*>(x + ((int64_t)r1 * a.ldx + k1) * 2);
        float amax;
        if constexpr (GIVEN) {
            amax = fmaxf(__ldcg(a.ffn_amax), 1e-12f);
        } else {
            float m = 0.f;
            if (i0 < nvec) fp8_vec_amax<DT>(v0, awq, k0, a.div_mode, after, m);
            if (i1 < nvec) fp8_vec_amax<DT>(v1, awq, k1, a.div_mode, after, m);
            w8_mark(a, 5);
            amax = fmaxf(cta_max(m, sh), 1e-12f);
            w8_mark(a, 6);
        }
        const float inv = div_mode_f32(448.f, amax, a.div_mode);
        if (i0 < nvec) *reinterpret_cast<uint4*>(xq + (size_t)r0 * a.pitch + k0 * 2) = e4m3x8_to_f16x8(fp8_vec_codes<DT>(v0, awq, k0, a.div_mode, inv));
        if (i1 < nvec) *reinterpret_cast<uint4*>(xq + (size_t)r1 * a.pitch + k1 * 2) = e4m3x8_to_f16x8(fp8_vec_codes<DT>(v1, awq, k1, a.div_mode, inv));
        return amax;
    }
    const int64_t ldx2 = a.ldx * 2;
    float m = 0.f;
    {
        // raw rows into the tile by bulk copies (one read of the activations), abs-max and in-place conversion from there.
        // The two loops are deliberately compact (one vector per iteration, not unrolled): they run once per CTA on a
        // cold instruction cache, and inside a sequence of different kernels a four-way unrolled, load-batched version
        // of them measured 2 us SLOWER per launch at M = 1, K = 16384 although it is faster when the same kernel
        // repeats.
        if (threadIdx.x == 0) {
            const uint32_t b = (uint32_t)__cvta_generic_to_shared(bar);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"((uint32_t)(a.M * a.K * 2)) : "memory");
#pragma unroll 1
            for (int r = 0; r < a.M; ++r)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"((uint32_t)__cvta_generic_to_shared(xq + (size_t)r * a.pitch)), "l"(x + (int64_t)r * ldx2),
                               "r"((uint32_t)(a.K * 2)), "r"(b) : "memory");
        }
        float amax = GIVEN ? __ldcg(a.ffn_amax) : 0.f;       // in flight while the copy lands
        if (!w8_staged_or_report(bar, a.status, a.wait_ns)) return -1.f;
        if constexpr (!GIVEN) {
#pragma unroll 1
            for (int r = 0; r < a.M; ++r) {
                const char* src = reinterpret_cast<const char*>(xq + (size_t)r * a.pitch);
#pragma unroll 1
                for (int i = threadIdx.x; i < kv; i += kThr)
                    fp8_vec_amax<DT>(*reinterpret_cast<const uint4*>(src + (size_t)i * 16), awq, i << 3, a.div_mode, after, m);
            }
            w8_mark(a, 5);
            amax = cta_max(m, sh);
            w8_mark(a, 6);
        }
        amax = fmaxf(amax, 1e-12f);
        const float inv = div_mode_f32(448.f, amax, a.div_mode);
#pragma unroll 1
        for (int r = 0; r < a.M; ++r) {
            uint8_t* qr = xq + (size_t)r * a.pitch;
#pragma unroll 1
            for (int i = threadIdx.x; i < kv; i += kThr) {
                const uint2 c = fp8_vec_codes<DT>(*reinterpret_cast<const uint4*>(qr + (size_t)i * 16), awq, i << 3, a.div_mode, inv);
                *reinterpret_cast<uint4*>(qr + (size_t)i * 16) = e4m3x8_to_f16x8(c);
            }
        }
        return amax;
    }
}

// ---- fused prologue, INT8: per-row amax / codes; row scales amax/127 into xs[].
// Few rows (M <= 4): the whole CTA works on one row at a time; more rows: one warp per row.
template <int DT>
__device__ __forceinline__ float int8_vec_amax(const uint4& v, float m) {
    return fmaxf(m, packed_absmax8<DT>(v));
}
// codes = trunc(clamp(x * s, -128, 127)): truncating float->int conversion, then a saturating pack to int8
__device__ __forceinline__ uint32_t pack_s8x4(int a0, int a1, int a2, int a3) {
    uint32_t hi, r;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(a3), "r"(a2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a1), "r"(a0), "r"(hi));
    return r;
}
template <int DT>
__device__ __forceinline__ uint2 int8_vec_codes(const uint4& v, float s) {
    const float2 f0 = cvt2<DT>(v.x), f1 = cvt2<DT>(v.y), f2 = cvt2<DT>(v.z), f3 = cvt2<DT>(v.w);
    return make_uint2(pack_s8x4(__float2int_rz(f0.x * s), __float2int_rz(f0.y * s), __float2int_rz(f1.x * s), __float2int_rz(f1.y * s)),
                      pack_s8x4(__float2int_rz(f2.x * s), __float2int_rz(f2.y * s), __float2int_rz(f3.x * s), __float2int_rz(f3.y * s)));
}

// GIVEN: the rows' maxima come from a.ffn_amax[2 + r] (published by the kernel that produced x, the FFN key projection
// with relu^2 in its epilogue): no abs-max pass; the CTA's threads walk all rows' vectors, eight loads in flight each.
template <int DT, bool GIVEN = false>
__device__ void quantize_int8_to_smem(const W8Args& a, int mat, uint8_t* xq, float* xs, float* sh) {
    const char* x = reinterpret_cast<const char*>(a.x[mat]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if constexpr (GIVEN) {
        const int kv = a.K >> 3, nvec = a.M * kv;
        const uint32_t inv_kv = 0xFFFFFFFFu / (uint32_t)kv + 1u;          // row of a flat vector index without a division
        if ((int)threadIdx.x < a.M) {
            const float m = fmaxf(__ldcg(a.ffn_amax + 2 + threadIdx.x), 1e-12f);
            xs[threadIdx.x] = div_mode_f32(m, 127.f, a.div_mode);
            sh[threadIdx.x] = div_mode_f32(127.f, m, a.div_mode);
        }
        __syncthreads();
#pragma unroll 1
        for (int i0 = threadIdx.x; i0 < nvec; i0 += 8 * kThr) {
            uint4 v[8];
            int rr[8], cc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int idx = min(i0 + j * kThr, nvec - 1);
                rr[j] = (int)__umulhi((uint32_t)idx, inv_kv);
                cc[j] = idx - rr[j] * kv;
                v[j] = ldg_l2_16(x + ((int64_t)rr[j] * a.ldx + (int64_t)cc[j] * 8) * 2);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (i0 + j * kThr < nvec) *reinterpret_cast<uint2*>(xq + (size_t)rr[j] * a.pitch + (size_t)cc[j] * 8) = int8_vec_codes<DT>(v[j], sh[rr[j]]);
        }
        return;
    }
    if (a.M <= 4 && a.K > 2 * kThr * 8 && a.K <= 8 * kThr * 8) {
        // long rows: the whole CTA works on one row at a time and keeps it in registers between amax and codes
        // (one read; measured quicker than two passes above K = 4096, slower below because of its code size)
#pragma unroll 1
        for (int r = 0; r < a.M; ++r) {
            const char* xr = x + (int64_t)r * a.ldx * 2;
            uint4 v[8];
            float m = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int k = (threadIdx.x + j * kThr) * 8;
                if (k < a.K) v[j] = *reinterpret_cast<const uint4*>(xr + k * 2);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if ((int)(threadIdx.x + j * kThr) * 8 < a.K) m = int8_vec_amax<DT>(v[j], m);
            m = fmaxf(cta_max(m, sh), 1e-12f);
            const float s = div_mode_f32(127.f, m, a.div_mode);
            if (threadIdx.x == 0) xs[r] = div_mode_f32(m, 127.f, a.div_mode);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int k = (threadIdx.x + j * kThr) * 8;
                if (k < a.K) *reinterpret_cast<uint2*>(xq + (size_t)r * a.pitch + k) = int8_vec_codes<DT>(v[j], s);
            }
        }
        return;
    }
    if (a.M <= 4) {
        for (int r = 0; r < a.M; ++r) {
            const char* xr = x + (int64_t)r * a.ldx * 2;
            float m = 0.f;
            for (int k = threadIdx.x * 8; k < a.K; k += kThr * 8) m = int8_vec_amax<DT>(*reinterpret_cast<const uint4*>(xr + k * 2), m);
            m = fmaxf(cta_max(m, sh), 1e-12f);
            const float s = div_mode_f32(127.f, m, a.div_mode);
            if (threadIdx.x == 0) xs[r] = div_mode_f32(m, 127.f, a.div_mode);
            for (int k = threadIdx.x * 8; k < a.K; k += kThr * 8)
                *reinterpret_cast<uint2*>(xq + (size_t)r * a.pitch + k) = int8_vec_codes<DT>(*reinterpret_cast<const uint4*>(xr + k * 2), s);
        }
        return;
    }
    // more rows: one warp per row, two passes with 8 loads in flight per lane.  (Calls with many rows are better served
    // by quantizing once, rwkvq_prep_x_int8, and running the projection on the codes: rwkvq_gemm_int8.)
    const int kvl = a.K >> 3;                              // vectors per row
#pragma unroll 1
    for (int r = warp; r < a.M; r += kWarps) {
        const char* xr = x + (int64_t)r * a.ldx * 2;
        uint8_t* qr = xq + (size_t)r * a.pitch;
        float m = 0.f;
#pragma unroll 1
        for (int i0 = lane; i0 < kvl; i0 += 8 * 32) {
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (i0 + 32 * j < kvl) v[j] = ldg_l2_16(xr + (size_t)(i0 + 32 * j) * 16);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (i0 + 32 * j < kvl) m = int8_vec_amax<DT>(v[j], m);
        }
        m = fmaxf(warp_max(m), 1e-12f);
        const float s = div_mode_f32(127.f, m, a.div_mode);
        if (lane == 0) xs[r] = div_mode_f32(m, 127.f, a.div_mode);
#pragma unroll 1
        for (int i0 = lane; i0 < kvl; i0 += 8 * 32) {
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (i0 + 32 * j < kvl) v[j] = ldg_l2_16(xr + (size_t)(i0 + 32 * j) * 16);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (i0 + 32 * j < kvl) *reinterpret_cast<uint2*>(qr + (size_t)(i0 + 32 * j) * 8) = int8_vec_codes<DT>(v[j], s);
        }
    }
}

// The decode GEMV on pre-quantized codes (gemv_w8a8.cu): a.codes / a.ascale / a.w / a.ws / a.out filled for a.nmat
// matrices, M <= 32.  Returns RWKVQ_E_SHAPE without launching when the code tile does not fit shared memory.
bool gemv_codes_fits(int M, int K);
int32_t gemv_codes_run(W8Args a, int qt, cudaStream_t st, const char* who);

}  // namespace rwkvq
