// Weight-only quantized GEMV (fp16 activations, M <= 16 rows) for every stand-alone INT4 / INT8 layout of the
// reference: one warp per output row, 8 weights per lane and step (one 32-bit load of nibbles or one 64-bit load
// of bytes), weights dequantized in registers exactly as the reference kernels spell it, fp32 accumulation,
// warp-shuffle reduction.  This is the general kernel (any group size, affine layouts, padded K); the group-wise
// INT4 decode path of the 7.2B shapes has its own tensor-core kernel in gemv_int4.cu and is cross-checked by this.
#include "common.cuh"

namespace rwkvq {

enum { WA_INT4_TENSOR = 0, WA_INT4_AFFINE = 1, WA_INT4_GROUP = 2, WA_INT8_TENSOR = 3, WA_INT8_AFFINE = 4 };

struct WaArgs {
    const __half* x;        // [M, ldx]
    const uint8_t* w;       // int4: [N, ldw] bytes, two nibbles each (low nibble = even k); int8: [N, ldw]
    const void* scales;     // tensor: fp32[1]; group: [N, K/G] fp32 or fp16
    const float* zeros;     // group: [N, K/G] fp32 or null (zero = -8 * scale)
    const float* mx;        // affine: [K] column offset
    const float* rx;        // affine: [K] column range (stored / 4 or / 16)
    const float* my;        // affine: [N] row offset
    const float* ry;        // affine: [N] row range
    __half* out;            // [M, ldo]
    int64_t ldx, ldw, ldo;
    int M, N, K, group, scale_f16;
};

constexpr int kWaMaxM = 16;

template <int FMT>
__global__ void __launch_bounds__(256) wa16_rowdot_kernel(const WaArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= a.N) return;
    constexpr bool kInt4 = FMT <= WA_INT4_GROUP;
    const uint8_t* wrow = a.w + (int64_t)n * a.ldw;
    float acc[kWaMaxM];
#pragma unroll
    for (int m = 0; m < kWaMaxM; ++m) acc[m] = 0.f;

    float tscale = 0.f, ryv = 0.f, myv = 0.f;
    if (FMT == WA_INT4_TENSOR || FMT == WA_INT8_TENSOR) tscale = reinterpret_cast<const float*>(a.scales)[0];
    if (FMT == WA_INT4_AFFINE || FMT == WA_INT8_AFFINE) { ryv = a.ry[n]; myv = a.my[n]; }
    const int ngroups = FMT == WA_INT4_GROUP ? a.K / a.group : 0;

    for (int k0 = lane * 8; k0 < a.K; k0 += 256) {
        float wv[8];
        if constexpr (kInt4) {
            const uint32_t p = *reinterpret_cast<const uint32_t*>(wrow + (k0 >> 1));
#pragma unroll
            for (int j = 0; j < 8; ++j) wv[j] = (float)((p >> (4 * j)) & 0xFu);
        } else {
            const uint2 p = *reinterpret_cast<const uint2*>(wrow + k0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t b = ((j < 4 ? p.x : p.y) >> (8 * (j & 3))) & 0xFFu;
                wv[j] = FMT == WA_INT8_TENSOR ? (float)(int8_t)b : (float)b;
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int k = k0 + j;
            if (FMT == WA_INT4_TENSOR) {
                wv[j] = (wv[j] > 7.f ? wv[j] - 16.f : wv[j]) * tscale;
            } else if (FMT == WA_INT8_TENSOR) {
                wv[j] = wv[j] * tscale;
            } else if (FMT == WA_INT4_GROUP) {
                const int gi = n * ngroups + k / a.group;
                const float s = a.scale_f16 ? __half2float(reinterpret_cast<const __half*>(a.scales)[gi])
                                            : reinterpret_cast<const float*>(a.scales)[gi];
                const float z = a.zeros ? a.zeros[gi] : -8.f * s;
                wv[j] = wv[j] * s + z;
            } else if (FMT == WA_INT4_AFFINE) {
                wv[j] = (wv[j] + 0.5f) * ryv * a.rx[k] * 16.0f + myv + a.mx[k];
            } else {
                wv[j] = (wv[j] + 0.5f) * ryv * a.rx[k] * 256.0f + myv + a.mx[k];
            }
        }
#pragma unroll
        for (int m = 0; m < kWaMaxM; ++m) {
            if (m < a.M) {
                const uint4 xv = *reinterpret_cast<const uint4*>(a.x + (int64_t)m * a.ldx + k0);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = cvt2<RWKVQ_F16>(xw[q]);
                    acc[m] = fmaf(f.x, wv[2 * q], acc[m]);
                    acc[m] = fmaf(f.y, wv[2 * q + 1], acc[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < kWaMaxM; ++m) {
        if (m < a.M) {
            const float v = warp_sum(acc[m]);
            if (lane == 0) a.out[(int64_t)m * a.ldo + n] = __float2half_rn(v);
        }
    }
}

static int32_t run_wa16(const WaArgs& a, int fmt, cudaStream_t st, const char* who) {
    RWKVQ_REQUIRE(a.x && a.w && a.out, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(a.M >= 0 && a.N >= 0 && a.K >= 0, RWKVQ_E_SHAPE, "%s: negative size", who);
    RWKVQ_REQUIRE(a.M <= kWaMaxM, RWKVQ_E_SHAPE, "%s: M=%d > %d rows", who, a.M, kWaMaxM);
    RWKVQ_REQUIRE(a.K % 8 == 0, RWKVQ_E_SHAPE, "%s: K=%d must be a multiple of 8", who, a.K);
    const bool int4 = fmt <= WA_INT4_GROUP;
    RWKVQ_REQUIRE(a.ldw >= (int4 ? a.K / 2 : a.K) && a.ldw % (int4 ? 4 : 8) == 0, RWKVQ_E_ALIGN, "%s: ldw=%lld", who, (long long)a.ldw);
    RWKVQ_REQUIRE(((uintptr_t)a.w & 7) == 0 && aligned16(a.x) && a.ldx % 8 == 0 && a.ldx >= a.K, RWKVQ_E_ALIGN,
                  "%s: weights need 8-byte, activations 16-byte aligned rows", who);
    RWKVQ_REQUIRE(a.ldo >= a.N, RWKVQ_E_SHAPE, "%s: ldo < N", who);
    if (fmt == WA_INT4_TENSOR || fmt == WA_INT8_TENSOR) RWKVQ_REQUIRE(a.scales != nullptr, RWKVQ_E_BADARG, "%s: null scale", who);
    if (fmt == WA_INT4_GROUP)
        RWKVQ_REQUIRE(a.scales && a.group > 0 && a.K % a.group == 0, RWKVQ_E_SHAPE, "%s: group size %d must divide K=%d", who, a.group, a.K);
    if (fmt == WA_INT4_AFFINE || fmt == WA_INT8_AFFINE)
        RWKVQ_REQUIRE(a.mx && a.rx && a.my && a.ry, RWKVQ_E_BADARG, "%s: null affine vector", who);
    if (a.M == 0 || a.N == 0) return RWKVQ_OK;
    const dim3 grid((unsigned)((a.N + 7) / 8));
    switch (fmt) {
        case WA_INT4_TENSOR: wa16_rowdot_kernel<WA_INT4_TENSOR><<<grid, 256, 0, st>>>(a); break;
        case WA_INT4_AFFINE: wa16_rowdot_kernel<WA_INT4_AFFINE><<<grid, 256, 0, st>>>(a); break;
        case WA_INT4_GROUP: wa16_rowdot_kernel<WA_INT4_GROUP><<<grid, 256, 0, st>>>(a); break;
        case WA_INT8_TENSOR: wa16_rowdot_kernel<WA_INT8_TENSOR><<<grid, 256, 0, st>>>(a); break;
        default: wa16_rowdot_kernel<WA_INT8_AFFINE><<<grid, 256, 0, st>>>(a); break;
    }
    return check_launch(who);
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

int32_t rwkvq_gemv_int4_tensor(const void* x_f16, int64_t ldx, const uint8_t* packed, int64_t ldw, const float* scale,
                               void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, void* stream) {
    WaArgs a{};
    a.x = (const __half*)x_f16; a.w = packed; a.scales = scale; a.out = (__half*)out_f16;
    a.ldx = ldx; a.ldw = ldw; a.ldo = ldo; a.M = (int)M; a.N = (int)N; a.K = (int)K;
    return run_wa16(a, WA_INT4_TENSOR, (cudaStream_t)stream, "gemv_int4_tensor");
}

int32_t rwkvq_gemv_int4_affine(const void* x_f16, int64_t ldx, const uint8_t* packed, int64_t ldw, const float* mx,
                               const float* rx, const float* my, const float* ry, void* out_f16, int64_t ldo, int64_t M,
                               int64_t N, int64_t K, void* stream) {
    WaArgs a{};
    a.x = (const __half*)x_f16; a.w = packed; a.mx = mx; a.rx = rx; a.my = my; a.ry = ry; a.out = (__half*)out_f16;
    a.ldx = ldx; a.ldw = ldw; a.ldo = ldo; a.M = (int)M; a.N = (int)N; a.K = (int)K;
    return run_wa16(a, WA_INT4_AFFINE, (cudaStream_t)stream, "gemv_int4_affine");
}

int32_t rwkvq_gemv_int4_group_generic(const void* x_f16, int64_t ldx, const uint8_t* packed, int64_t ldw, const void* scales,
                                      const float* zeros, int32_t scale_is_f16, int32_t group, void* out_f16, int64_t ldo,
                                      int64_t M, int64_t N, int64_t K, void* stream) {
    WaArgs a{};
    a.x = (const __half*)x_f16; a.w = packed; a.scales = scales; a.zeros = zeros; a.out = (__half*)out_f16;
    a.scale_f16 = scale_is_f16; a.group = group;
    a.ldx = ldx; a.ldw = ldw; a.ldo = ldo; a.M = (int)M; a.N = (int)N; a.K = (int)K;
    return run_wa16(a, WA_INT4_GROUP, (cudaStream_t)stream, "gemv_int4_group_generic");
}

int32_t rwkvq_gemv_int8_w8a16(const void* x_f16, int64_t ldx, const int8_t* w, int64_t ldw, const float* scale,
                              void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, void* stream) {
    WaArgs a{};
    a.x = (const __half*)x_f16; a.w = (const uint8_t*)w; a.scales = scale; a.out = (__half*)out_f16;
    a.ldx = ldx; a.ldw = ldw; a.ldo = ldo; a.M = (int)M; a.N = (int)N; a.K = (int)K;
    return run_wa16(a, WA_INT8_TENSOR, (cudaStream_t)stream, "gemv_int8_w8a16");
}

int32_t rwkvq_gemv_int8_affine(const void* x_f16, int64_t ldx, const uint8_t* w_u8, int64_t ldw, const float* mx,
                               const float* rx, const float* my, const float* ry, void* out_f16, int64_t ldo, int64_t M,
                               int64_t N, int64_t K, void* stream) {
    WaArgs a{};
    a.x = (const __half*)x_f16; a.w = w_u8; a.mx = mx; a.rx = rx; a.my = my; a.ry = ry; a.out = (__half*)out_f16;
    a.ldx = ldx; a.ldw = ldw; a.ldo = ldo; a.M = (int)M; a.N = (int)N; a.K = (int)K;
    return run_wa16(a, WA_INT8_AFFINE, (cudaStream_t)stream, "gemv_int8_affine");
}

}  // extern "C"
