// W8A8 projections for small M (decode): FP8 e4m3 x e4m3 and INT8 x INT8, single matrix or r/k/v in one launch.
//
// The kernel is HBM-bound: the weight matrix [N,K] (one byte per element) is read exactly once with 128-bit
// streaming loads straight into registers, and those registers ARE the B fragments of mma.sync.m16n8k32
// (8 weight rows x 32 k per instruction): lane (g = lane/4, t = lane%4) loads the 16 bytes W[n0+g][k0+16t ..+15]
// and feeds them to two MMAs.  An MMA sums over its 32 k-slots, so the slots may be filled in any order as long
// as A and B agree; the A fragment (quantized activations, 16 token rows) is read with the same permutation
// from shared memory (fused mode) or from a code matrix in global memory (pre-quantized mode).
//
// A CTA is 8 warps working on the same 8 weight rows, each warp on every 8th 64-byte column unit (split-K inside
// the CTA, fixed-order reduction through shared memory, so results are run-to-run identical).  CTAs are persistent:
// each takes a contiguous range of the (matrix, row-tile) list, so the activation quantization of the prologue is
// done once per CTA and matrix, not once per tile.
//
// Fused prologue (what prep_x / prep3_x / prep_x_int8 + the in-kernel quantization of the reference do):
//   FP8 : amax over the whole [M,K] call, inv = 448/max(amax,1e-12), code = e4m3(clamp(bf16(x)*inv)),
//         result scale (amax/448)*w_scale.
//   INT8: per row amax, s = 127/amax, code = trunc(clamp(x*s,-128,127)), row scale amax/127.
#include "common.cuh"

namespace rwkvq {

constexpr int kWarps = 8;
constexpr int kThr = kWarps * 32;
constexpr int kUnroll = 4;

enum { QT_FP8 = 0, QT_INT8 = 1 };

struct W8Args {
    const void* x[3];         // fused: activations (x_dtype)
    const float* awq[3];      // fused FP8: optional per-channel divisor
    const uint8_t* w[3];
    const float* ws[3];       // weight scale (one fp32 each)
    __half* out[3];
    int32_t* acc[3];          // INT8: optional raw accumulators
    const uint8_t* a_codes;   // pre-quantized mode
    const float* a_scale;     // pre-quantized: FP8 amax-or-scale [1], INT8 per-row scales [M]
    int64_t ldx, ldw, ldo, ldacc, lda;
    int M, N, K, nmat;
    int div_mode, amax_is_amax;
    uint32_t flags;
    int pitch;                // fused: bytes between rows of the code tile in shared memory
};

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

// ---- fused prologue, FP8: per-call amax then e4m3 codes into shared memory; returns max(amax, 1e-12)
template <int DT>
__device__ float quantize_fp8_to_smem(const W8Args& a, int mat, uint8_t* xq, float* sh) {
    const char* x = reinterpret_cast<const char*>(a.x[mat]);
    const float* awq = a.awq[mat];
    const int kv = a.K >> 3;                  // 8-element vectors per row
    const int nvec = a.M * kv;
    const bool after = (a.flags & RWKVQ_FLAG_AMAX_AFTER_BF16) != 0;
    float m = 0.f;
    for (int i = threadIdx.x; i < nvec; i += kThr) {
        const int r = i / kv, k = (i - r * kv) << 3;
        const uint4 v = *reinterpret_cast<const uint4*>(x + ((int64_t)r * a.ldx + k) * 2);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float2 f = cvt2<DT>(w[q]);
            if (awq) {
                f.x = div_mode_f32(f.x, awq[k + 2 * q], a.div_mode);
                f.y = div_mode_f32(f.y, awq[k + 2 * q + 1], a.div_mode);
            }
            if (after) { f.x = bf16_round(f.x); f.y = bf16_round(f.y); }
            m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
    }
    const float amax = fmaxf(cta_max(m, sh), 1e-12f);
    const float inv = div_mode_f32(448.f, amax, a.div_mode);
    for (int i = threadIdx.x; i < nvec; i += kThr) {
        const int r = i / kv, k = (i - r * kv) << 3;
        const uint4 v = *reinterpret_cast<const uint4*>(x + ((int64_t)r * a.ldx + k) * 2);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t c[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float2 f = cvt2<DT>(w[q]);
            if (awq) {
                f.x = div_mode_f32(f.x, awq[k + 2 * q], a.div_mode);
                f.y = div_mode_f32(f.y, awq[k + 2 * q + 1], a.div_mode);
            }
            c[q] = e4m3x2(clamp448(bf16_round(f.x) * inv), clamp448(bf16_round(f.y) * inv));
        }
        *reinterpret_cast<uint2*>(xq + (size_t)r * a.pitch + k) = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
    }
    return amax;
}

// ---- fused prologue, INT8: per-row amax / codes; row scales amax/127 into xs[]
template <int DT>
__device__ void quantize_int8_to_smem(const W8Args& a, int mat, uint8_t* xq, float* xs) {
    const char* x = reinterpret_cast<const char*>(a.x[mat]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < a.M; r += kWarps) {
        const char* xr = x + (int64_t)r * a.ldx * 2;
        float m = 0.f;
        for (int k = lane * 8; k < a.K; k += 256) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + k * 2);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = cvt2<DT>(w[q]);
                m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
        }
        m = fmaxf(warp_max(m), 1e-12f);
        const float s = div_mode_f32(127.f, m, a.div_mode);
        if (lane == 0) xs[r] = div_mode_f32(m, 127.f, a.div_mode);
        for (int k = lane * 8; k < a.K; k += 256) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + k * 2);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t c[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = cvt2<DT>(w[q]);
                const uint32_t lo = (uint32_t)__float2int_rz(fminf(fmaxf(f.x * s, -128.f), 127.f)) & 0xffu;
                const uint32_t hi = (uint32_t)__float2int_rz(fminf(fmaxf(f.y * s, -128.f), 127.f)) & 0xffu;
                c[q] = lo | (hi << 8);
            }
            *reinterpret_cast<uint2*>(xq + (size_t)r * a.pitch + k) = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
        }
    }
}

template <int QT, int DT, int MT, bool FUSED>
__global__ void __launch_bounds__(kThr, FUSED ? 3 : 2) gemv_w8a8_kernel(const W8Args a) {
    using T = typename Acc<QT>::T;
    extern __shared__ __align__(16) uint8_t smem[];
    // layout: red[kWarps][MT*4][32] | xs[32] | sh[8] | xq[M][pitch]
    T* red = reinterpret_cast<T*>(smem);
    float* xs = reinterpret_cast<float*>(smem + kWarps * MT * 4 * 32 * 4);
    float* sh = xs + 32;
    uint8_t* xq = reinterpret_cast<uint8_t*>(sh + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ntile = (a.N + 7) >> 3;
    const int64_t total = (int64_t)a.nmat * ntile;
    const int64_t tb = total * blockIdx.x / gridDim.x, te = total * (blockIdx.x + 1) / gridDim.x;
    const int m0 = FUSED ? 0 : blockIdx.y * (16 * MT);
    const int units = (a.K + 63) >> 6;

    int cur_mat = -1;
    float out_scale = 0.f;   // FP8: (amax/448)*w_scale
    float wscale = 0.f;      // INT8: w_scale
    for (int64_t tile = tb; tile < te; ++tile) {
        const int mat = (int)(tile / ntile);
        const int n0 = (int)(tile - (int64_t)mat * ntile) << 3;
        if (mat != cur_mat) {
            cur_mat = mat;
            if constexpr (FUSED) {
                __syncthreads();   // nobody still reads the previous matrix's codes
                if constexpr (QT == QT_FP8) {
                    const float amax = quantize_fp8_to_smem<DT>(a, mat, xq, sh);
                    out_scale = div_mode_f32(amax, 448.f, a.div_mode) * a.ws[mat][0];
                } else {
                    quantize_int8_to_smem<DT>(a, mat, xq, xs);
                    wscale = a.ws[mat][0];
                }
                __syncthreads();
            } else {
                if constexpr (QT == QT_FP8) {
                    const float am = a.a_scale[0];
                    const float s = a.amax_is_amax ? div_mode_f32(fmaxf(am, 1e-12f), 448.f, a.div_mode) : am;
                    out_scale = s * a.ws[mat][0];
                } else {
                    wscale = a.ws[mat][0];
                }
            }
        }
        const int nrow = min(n0 + g, a.N - 1);
        const uint8_t* wrow = a.w[mat] + (int64_t)nrow * a.ldw + 16 * t;

        T c[MT][4];
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) c[i][j] = 0;

        for (int u0 = warp; u0 < units; u0 += kWarps * kUnroll) {
            uint4 wv[kUnroll];
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int k = ((u0 + j * kWarps) << 6) + 16 * t;
                wv[j] = (k < a.K) ? ldg_stream(wrow + ((u0 + j * kWarps) << 6)) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                const int k = ((u0 + j * kWarps) << 6) + 16 * t;
                const bool kin = k < a.K;
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    const int r0 = m0 + i * 16 + g, r1 = r0 + 8;
                    uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0;
                    if constexpr (FUSED) {
                        if (kin && r0 < a.M) a0 = *reinterpret_cast<const uint4*>(xq + (size_t)r0 * a.pitch + k);
                        if (kin && r1 < a.M) a1 = *reinterpret_cast<const uint4*>(xq + (size_t)r1 * a.pitch + k);
                    } else {
                        if (kin && r0 < a.M) a0 = __ldg(reinterpret_cast<const uint4*>(a.a_codes + (int64_t)r0 * a.lda + k));
                        if (kin && r1 < a.M) a1 = __ldg(reinterpret_cast<const uint4*>(a.a_codes + (int64_t)r1 * a.lda + k));
                    }
                    mma8<QT>(c[i], a0.x, a1.x, a0.y, a1.y, wv[j].x, wv[j].y);
                    mma8<QT>(c[i], a0.z, a1.z, a0.w, a1.w, wv[j].z, wv[j].w);
                }
            }
        }

        // split-K reduction across the 8 warps, fixed order
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) red[(warp * MT * 4 + i * 4 + j) * 32 + lane] = c[i][j];
        __syncthreads();
        if (threadIdx.x < MT * 128) {
            const int ij = threadIdx.x >> 5, l = threadIdx.x & 31;      // ij = i*4 + j
            T s = 0;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += red[(w * MT * 4 + ij) * 32 + l];
            const int i = ij >> 2, j = ij & 3;
            const int m = m0 + i * 16 + (l >> 2) + ((j & 2) ? 8 : 0);
            const int n = n0 + 2 * (l & 3) + (j & 1);
            if (m < a.M && n < a.N) {
                float v;
                if constexpr (QT == QT_FP8) {
                    v = s * out_scale;
                } else {
                    if (a.acc[mat]) a.acc[mat][(int64_t)m * a.ldacc + n] = s;
                    const float rs = FUSED ? xs[m] : a.a_scale[m];
                    v = (float)s * (rs * wscale);
                }
                if (a.flags & RWKVQ_FLAG_OUT_VIA_BF16) v = bf16_round(v);
                a.out[mat][(int64_t)m * a.ldo + n] = __float2half_rn(v);
            }
        }
        __syncthreads();
    }
}

static size_t smem_bytes(int MT, int M, int pitch, bool fused) {
    return (size_t)kWarps * MT * 4 * 32 * 4 + 32 * 4 + 8 * 4 + (fused ? (size_t)M * pitch : 0);
}

constexpr size_t kFusedSmemMax = 200 * 1024;

template <int QT, int DT, int MT, bool FUSED>
static int32_t launch_one(const W8Args& a, dim3 grid, size_t smem, cudaStream_t st) {
    auto kern = gemv_w8a8_kernel<QT, DT, MT, FUSED>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFusedSmemMax);
        if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "gemv_w8a8: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    kern<<<grid, kThr, smem, st>>>(a);
    return check_launch("gemv_w8a8");
}

template <int QT, bool FUSED>
static int32_t dispatch(const W8Args& a, int x_dtype, dim3 grid, int MT, size_t smem, cudaStream_t st) {
    if (x_dtype == RWKVQ_F16) {
        return MT == 1 ? launch_one<QT, RWKVQ_F16, 1, FUSED>(a, grid, smem, st) : launch_one<QT, RWKVQ_F16, 2, FUSED>(a, grid, smem, st);
    }
    return MT == 1 ? launch_one<QT, RWKVQ_BF16, 1, FUSED>(a, grid, smem, st) : launch_one<QT, RWKVQ_BF16, 2, FUSED>(a, grid, smem, st);
}

static int32_t check_common(const W8Args& a, const char* who) {
    RWKVQ_REQUIRE(a.M >= 0 && a.N >= 0 && a.K >= 0, RWKVQ_E_SHAPE, "%s: negative size", who);
    RWKVQ_REQUIRE(a.K % 16 == 0, RWKVQ_E_SHAPE, "%s: K=%d must be a multiple of 16", who, a.K);
    RWKVQ_REQUIRE(a.ldw >= a.K && a.ldw % 16 == 0, RWKVQ_E_ALIGN, "%s: ldw=%lld must be >= K and a multiple of 16", who, (long long)a.ldw);
    RWKVQ_REQUIRE(a.ldo >= a.N, RWKVQ_E_SHAPE, "%s: ldo=%lld < N", who, (long long)a.ldo);
    RWKVQ_REQUIRE(a.div_mode == RWKVQ_DIV_IEEE || a.div_mode == RWKVQ_DIV_FULL, RWKVQ_E_BADARG, "%s: div_mode %d", who, a.div_mode);
    for (int i = 0; i < a.nmat; ++i) {
        RWKVQ_REQUIRE(a.w[i] && a.ws[i] && a.out[i], RWKVQ_E_BADARG, "%s: null weight/scale/out pointer (matrix %d)", who, i);
        RWKVQ_REQUIRE(aligned16(a.w[i]), RWKVQ_E_ALIGN, "%s: weight pointer not 16-byte aligned", who);
    }
    return RWKVQ_OK;
}

template <int QT>
static int32_t run_fused(W8Args a, int x_dtype, cudaStream_t st, const char* who) {
    int32_t rc = check_common(a, who);
    if (rc) return rc;
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, x_dtype);
    RWKVQ_REQUIRE(a.M <= 32, RWKVQ_E_SHAPE, "%s: M=%d > 32 (use the GEMM entry points)", who, a.M);
    RWKVQ_REQUIRE(a.ldx >= a.K && a.ldx % 8 == 0, RWKVQ_E_ALIGN, "%s: ldx=%lld must be >= K and a multiple of 8", who, (long long)a.ldx);
    for (int i = 0; i < a.nmat; ++i) {
        RWKVQ_REQUIRE(a.x[i], RWKVQ_E_BADARG, "%s: null activation pointer", who);
        RWKVQ_REQUIRE(aligned16(a.x[i]), RWKVQ_E_ALIGN, "%s: activation pointer not 16-byte aligned", who);
    }
    if (a.M == 0 || a.N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(a.K > 0, RWKVQ_E_SHAPE, "%s: K=0", who);
    const int MT = a.M <= 16 ? 1 : 2;
    a.pitch = ((a.K + 127) / 128) * 128 + 64;
    const size_t smem = smem_bytes(MT, a.M, a.pitch, true);
    RWKVQ_REQUIRE(smem <= kFusedSmemMax, RWKVQ_E_SHAPE, "%s: M*K = %d*%d does not fit the fused kernel's shared memory", who, a.M, a.K);
    const int64_t tiles = (int64_t)a.nmat * ((a.N + 7) / 8);
    const int per_sm = smem <= 72 * 1024 ? 3 : (smem <= 110 * 1024 ? 2 : 1);
    const int64_t grid = std::min<int64_t>(tiles, (int64_t)sm_count() * per_sm);
    return dispatch<QT, true>(a, x_dtype, dim3((unsigned)grid), MT, smem, st);
}

template <int QT>
static int32_t run_codes(W8Args a, cudaStream_t st, const char* who) {
    int32_t rc = check_common(a, who);
    if (rc) return rc;
    RWKVQ_REQUIRE(a.a_codes && a.a_scale, RWKVQ_E_BADARG, "%s: null activation codes / scale", who);
    RWKVQ_REQUIRE(aligned16(a.a_codes) && a.lda % 16 == 0 && a.lda >= a.K, RWKVQ_E_ALIGN, "%s: activation codes need 16-byte aligned rows", who);
    if (a.M == 0 || a.N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(a.K > 0, RWKVQ_E_SHAPE, "%s: K=0", who);
    const int MT = a.M <= 16 ? 1 : 2;
    const int mblocks = (a.M + 16 * MT - 1) / (16 * MT);
    RWKVQ_REQUIRE(mblocks <= 65535, RWKVQ_E_SHAPE, "%s: M=%d too large for this kernel", who, a.M);
    const int64_t tiles = (int64_t)a.nmat * ((a.N + 7) / 8);
    const int64_t grid = std::min<int64_t>(tiles, std::max<int64_t>(1, (int64_t)sm_count() * 2 / std::min(mblocks, 8)));
    return dispatch<QT, false>(a, RWKVQ_BF16, dim3((unsigned)grid, (unsigned)mblocks), MT, smem_bytes(MT, 0, 0, false), st);
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

int32_t rwkvq_gemv_fp8(const void* x, int32_t x_dtype, const float* awq, const uint8_t* w, int64_t ldw, const float* w_scale,
                       void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode,
                       uint32_t flags, void* stream) {
    W8Args a{};
    a.x[0] = x; a.awq[0] = awq; a.w[0] = w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldw = ldw; a.ldo = ldo;
    a.div_mode = div_mode; a.flags = flags;
    return run_fused<QT_FP8>(a, x_dtype, (cudaStream_t)stream, "gemv_fp8");
}

int32_t rwkvq_gemv_fp8_rkv(const void* xr, const void* xk, const void* xv, int32_t x_dtype, const float* awq_r,
                           const float* awq_k, const uint8_t* wr, const uint8_t* wk, const uint8_t* wv, int64_t ldw,
                           const float* sr, const float* sk, const float* sv, void* out_r, void* out_k, void* out_v,
                           int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode, uint32_t flags,
                           void* stream) {
    W8Args a{};
    a.x[0] = xr; a.x[1] = xk; a.x[2] = xv;
    a.awq[0] = awq_r; a.awq[1] = awq_k;
    a.w[0] = wr; a.w[1] = wk; a.w[2] = wv;
    a.ws[0] = sr; a.ws[1] = sk; a.ws[2] = sv;
    a.out[0] = (__half*)out_r; a.out[1] = (__half*)out_k; a.out[2] = (__half*)out_v;
    a.nmat = 3; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldw = ldw; a.ldo = ldo;
    a.div_mode = div_mode; a.flags = flags;
    return run_fused<QT_FP8>(a, x_dtype, (cudaStream_t)stream, "gemv_fp8_rkv");
}

int32_t rwkvq_gemv_int8(const void* x, int32_t x_dtype, const int8_t* w, int64_t ldw, const float* w_scale, void* out_f16,
                        int64_t ldo, int32_t* acc_out, int64_t ldacc, int64_t M, int64_t N, int64_t K, int64_t ldx,
                        int32_t div_mode, uint32_t flags, void* stream) {
    W8Args a{};
    a.x[0] = x; a.w[0] = (const uint8_t*)w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16; a.acc[0] = acc_out;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldw = ldw; a.ldo = ldo; a.ldacc = ldacc;
    a.div_mode = div_mode; a.flags = flags;
    RWKVQ_REQUIRE(acc_out == nullptr || ldacc >= N, RWKVQ_E_SHAPE, "gemv_int8: ldacc < N");
    return run_fused<QT_INT8>(a, x_dtype, (cudaStream_t)stream, "gemv_int8");
}

int32_t rwkvq_gemv_int8_rkv(const void* xr, const void* xk, const void* xv, int32_t x_dtype, const int8_t* wr,
                            const int8_t* wk, const int8_t* wv, int64_t ldw, const float* sr, const float* sk,
                            const float* sv, void* out_r, void* out_k, void* out_v, int64_t ldo, int64_t M, int64_t N,
                            int64_t K, int64_t ldx, int32_t div_mode, uint32_t flags, void* stream) {
    W8Args a{};
    a.x[0] = xr; a.x[1] = xk; a.x[2] = xv;
    a.w[0] = (const uint8_t*)wr; a.w[1] = (const uint8_t*)wk; a.w[2] = (const uint8_t*)wv;
    const bool shared = (flags & RWKVQ_FLAG_INT8_SHARED_WSCALE) != 0;
    a.ws[0] = sr; a.ws[1] = shared ? sr : sk; a.ws[2] = shared ? sr : sv;
    a.out[0] = (__half*)out_r; a.out[1] = (__half*)out_k; a.out[2] = (__half*)out_v;
    a.nmat = 3; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldw = ldw; a.ldo = ldo;
    a.div_mode = div_mode; a.flags = flags;
    return run_fused<QT_INT8>(a, x_dtype, (cudaStream_t)stream, "gemv_int8_rkv");
}

// mma.sync route for pre-quantized codes at any M (bit-exact INT8 accumulators; the route the small-M GEMM
// dispatch takes between the fused decode kernel and the tensor-memory prefill kernel).
int32_t rwkvq_gemm_fp8_mma(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax, const uint8_t* w,
                           int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                           int32_t div_mode, uint32_t flags, void* stream) {
    W8Args a{};
    a.a_codes = a_codes; a.lda = lda; a.a_scale = amax; a.amax_is_amax = amax_is_amax;
    a.w[0] = w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldw = ldw; a.ldo = ldo; a.div_mode = div_mode; a.flags = flags;
    return run_codes<QT_FP8>(a, (cudaStream_t)stream, "gemm_fp8_mma");
}

int32_t rwkvq_gemm_int8_mma(const int8_t* a_codes, int64_t lda, const float* a_scales, const int8_t* w, int64_t ldw,
                            const float* w_scale, void* out_f16, int64_t ldo, int32_t* acc_out, int64_t ldacc, int64_t M,
                            int64_t N, int64_t K, uint32_t flags, void* stream) {
    W8Args a{};
    a.a_codes = (const uint8_t*)a_codes; a.lda = lda; a.a_scale = a_scales;
    a.w[0] = (const uint8_t*)w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16; a.acc[0] = acc_out; a.ldacc = ldacc;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldw = ldw; a.ldo = ldo; a.div_mode = RWKVQ_DIV_IEEE; a.flags = flags;
    RWKVQ_REQUIRE(acc_out == nullptr || ldacc >= N, RWKVQ_E_SHAPE, "gemm_int8_mma: ldacc < N");
    return run_codes<QT_INT8>(a, (cudaStream_t)stream, "gemm_int8_mma");
}

}  // extern "C"
