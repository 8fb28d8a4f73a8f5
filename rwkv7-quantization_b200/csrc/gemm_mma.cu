// W8A8 GEMM on pre-quantized activation codes for ANY M with mma.sync.m16n8k32 (e4m3 or s8): the weight rows are
// streamed from global memory straight into B fragments, the activation codes are read as A fragments from the
// [M,K] code matrix (L1/L2 resident for small M).  Exact int32 accumulation for INT8.  This kernel serves the rows
// between the decode GEMV (M <= 32, codes in shared memory) and the tensor-memory GEMM, and is the bit-exact
// cross-check of both.
#include "w8a8.cuh"

namespace rwkvq {

template <int QT, int MT>
__global__ void __launch_bounds__(kThr, 2) gemm_mma_kernel(const W8Args a) {
    using T = typename Acc<QT>::T;
    __shared__ T red[kWarps * MT * 4 * 32];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ntile = (a.N + 7) >> 3;
    const int64_t tb = (int64_t)ntile * blockIdx.x / gridDim.x, te = (int64_t)ntile * (blockIdx.x + 1) / gridDim.x;
    const int m0 = blockIdx.y * (16 * MT);
    const int units = (a.K + 63) >> 6;

    const bool per_row = (a.flags & RWKVQ_FLAG_WSCALE_PER_ROW) != 0;     // one weight scale per output row n
    float act_scale = 0.f, wscale = a.ws[0][0];
    if constexpr (QT == QT_FP8) {
        const float am = a.a_scale[0];
        act_scale = a.amax_is_amax ? div_mode_f32(fmaxf(am, 1e-12f), 448.f, a.div_mode) : am;
    }
    for (int64_t tile = tb; tile < te; ++tile) {
        const int n0 = (int)tile << 3;
        const int nrow = min(n0 + g, a.N - 1);
        const uint8_t* wrow = a.w[0] + (int64_t)nrow * a.ldw + 16 * t;
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
                    if (kin && r0 < a.M) a0 = __ldg(reinterpret_cast<const uint4*>(a.a_codes + (int64_t)r0 * a.lda + k));
                    if (kin && r1 < a.M) a1 = __ldg(reinterpret_cast<const uint4*>(a.a_codes + (int64_t)r1 * a.lda + k));
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
            const int ij = threadIdx.x >> 5, l = threadIdx.x & 31;
            T s = 0;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += red[(w * MT * 4 + ij) * 32 + l];
            const int i = ij >> 2, j = ij & 3;
            const int m = m0 + i * 16 + (l >> 2) + ((j & 2) ? 8 : 0);
            const int n = n0 + 2 * (l & 3) + (j & 1);
            if (m < a.M && n < a.N) {
                float v;
                const float wsn = per_row ? a.ws[0][n] : wscale;
                if constexpr (QT == QT_FP8) {
                    v = s * (act_scale * wsn);
                } else {
                    if (a.acc[0]) a.acc[0][(int64_t)m * a.ldacc + n] = s;
                    v = (float)s * (a.a_scale[m] * wsn);
                }
                if (a.flags & RWKVQ_FLAG_OUT_VIA_BF16) v = bf16_round(v);
                a.out[0][(int64_t)m * a.ldo + n] = __float2half_rn(v);
            }
        }
        __syncthreads();
    }
}

template <int QT>
static int32_t run_codes(W8Args a, cudaStream_t st, const char* who) {
    RWKVQ_REQUIRE(a.M >= 0 && a.N >= 0 && a.K >= 0, RWKVQ_E_SHAPE, "%s: negative size", who);
    RWKVQ_REQUIRE(a.K % 16 == 0, RWKVQ_E_SHAPE, "%s: K=%d must be a multiple of 16", who, a.K);
    RWKVQ_REQUIRE(a.w[0] && a.ws[0] && a.out[0] && a.a_codes && a.a_scale, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(aligned16(a.w[0]) && a.ldw % 16 == 0 && a.ldw >= a.K, RWKVQ_E_ALIGN, "%s: weight rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(aligned16(a.a_codes) && a.lda % 16 == 0 && a.lda >= a.K, RWKVQ_E_ALIGN, "%s: activation code rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(a.ldo >= a.N, RWKVQ_E_SHAPE, "%s: ldo=%lld < N", who, (long long)a.ldo);
    if (a.M == 0 || a.N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(a.K > 0, RWKVQ_E_SHAPE, "%s: K=0", who);
    const int MT = a.M <= 16 ? 1 : 2;
    const int mblocks = (a.M + 16 * MT - 1) / (16 * MT);
    RWKVQ_REQUIRE(mblocks <= 65535, RWKVQ_E_SHAPE, "%s: M=%d too large for this kernel", who, a.M);
    const int64_t tiles = (a.N + 7) / 8;
    const int64_t gx = std::min<int64_t>(tiles, std::max<int64_t>(1, (int64_t)sm_count() * 2 / std::min(mblocks, 8)));
    dim3 grid((unsigned)gx, (unsigned)mblocks);
    if (MT == 1) gemm_mma_kernel<QT, 1><<<grid, kThr, 0, st>>>(a);
    else gemm_mma_kernel<QT, 2><<<grid, kThr, 0, st>>>(a);
    return check_launch(who);
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

// Few rows whose code tile fits shared memory go to the weight-streaming decode GEMV (gemv_w8a8.cu, activation codes
// copied once per CTA); everything else to the any-M kernel above.
static bool decode_route(int64_t M, int64_t K) { return M <= 32 && gemv_codes_fits((int)M, (int)K); }

int32_t rwkvq_gemm_fp8(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax, const uint8_t* w,
                           int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                           int32_t div_mode, uint32_t flags, void* stream) {
    if (decode_route(M, K))
        return rwkvq_gemm_fp8_rkv(a_codes, nullptr, nullptr, lda, amax, amax_is_amax, w, nullptr, nullptr, ldw, w_scale, nullptr, nullptr,
                                  out_f16, nullptr, nullptr, ldo, M, N, K, div_mode, flags, stream);
    W8Args a{};
    a.a_codes = a_codes; a.lda = lda; a.a_scale = amax; a.amax_is_amax = amax_is_amax;
    a.w[0] = w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldw = ldw; a.ldo = ldo; a.div_mode = div_mode; a.flags = flags;
    RWKVQ_REQUIRE(div_mode == RWKVQ_DIV_IEEE || div_mode == RWKVQ_DIV_FULL, RWKVQ_E_BADARG, "gemm_fp8: div_mode %d", div_mode);
    return run_codes<QT_FP8>(a, (cudaStream_t)stream, "gemm_fp8");
}

int32_t rwkvq_gemm_int8(const int8_t* a_codes, int64_t lda, const float* a_scales, const int8_t* w, int64_t ldw,
                            const float* w_scale, void* out_f16, int64_t ldo, int32_t* acc_out, int64_t ldacc, int64_t M,
                            int64_t N, int64_t K, uint32_t flags, void* stream) {
    if (decode_route(M, K)) {
        W8Args a{};
        a.codes[0] = (const uint8_t*)a_codes; a.lda = lda; a.ascale[0] = a_scales;
        a.w[0] = (const uint8_t*)w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16; a.acc[0] = acc_out; a.ldacc = ldacc;
        a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldw = ldw; a.ldo = ldo; a.div_mode = RWKVQ_DIV_IEEE; a.flags = flags;
        RWKVQ_REQUIRE(acc_out == nullptr || ldacc >= N, RWKVQ_E_SHAPE, "gemm_int8: ldacc < N");
        return gemv_codes_run(a, QT_INT8, (cudaStream_t)stream, "gemm_int8");
    }
    W8Args a{};
    a.a_codes = (const uint8_t*)a_codes; a.lda = lda; a.a_scale = a_scales;
    a.w[0] = (const uint8_t*)w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16; a.acc[0] = acc_out; a.ldacc = ldacc;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldw = ldw; a.ldo = ldo; a.div_mode = RWKVQ_DIV_IEEE; a.flags = flags;
    RWKVQ_REQUIRE(acc_out == nullptr || ldacc >= N, RWKVQ_E_SHAPE, "gemm_int8: ldacc < N");
    return run_codes<QT_INT8>(a, (cudaStream_t)stream, "gemm_int8");
}

/* 1 when rwkvq_gemm_fp8 / rwkvq_gemm_int8 (and the _rkv forms) run M rows of K codes on the weight-streaming decode
 * kernel, 0 when they fall to the any-M kernel. */
int32_t rwkvq_gemm_decode_route(int64_t M, int64_t K) { return decode_route(M, K) ? 1 : 0; }

/* r, k, v on codes in one launch (decode GEMV, M <= 32 and the code tile fits); otherwise three launches of the any-M
 * kernel.  Passing only the first matrix (wk == NULL) runs a single projection. */
int32_t rwkvq_gemm_fp8_rkv(const uint8_t* codes_r, const uint8_t* codes_k, const uint8_t* codes_v, int64_t lda, const float* amax3,
                           int32_t amax_is_amax, const uint8_t* wr, const uint8_t* wk, const uint8_t* wv, int64_t ldw, const float* sr,
                           const float* sk, const float* sv, void* out_r, void* out_k, void* out_v, int64_t ldo, int64_t M, int64_t N,
                           int64_t K, int32_t div_mode, uint32_t flags, void* stream) {
    RWKVQ_REQUIRE(amax3 != nullptr, RWKVQ_E_BADARG, "gemm_fp8_rkv: null amax");
    const int nmat = wk ? 3 : 1;
    if (!decode_route(M, K)) {
        const uint8_t* c[3] = {codes_r, codes_k, codes_v};
        const uint8_t* w[3] = {wr, wk, wv};
        const float* s[3] = {sr, sk, sv};
        void* o[3] = {out_r, out_k, out_v};
        for (int i = 0; i < nmat; ++i) {
            W8Args a{};
            a.a_codes = c[i]; a.lda = lda; a.a_scale = amax3 + i; a.amax_is_amax = amax_is_amax;
            a.w[0] = w[i]; a.ws[0] = s[i]; a.out[0] = (__half*)o[i];
            a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldw = ldw; a.ldo = ldo; a.div_mode = div_mode; a.flags = flags;
            RWKVQ_REQUIRE(div_mode == RWKVQ_DIV_IEEE || div_mode == RWKVQ_DIV_FULL, RWKVQ_E_BADARG, "gemm_fp8_rkv: div_mode %d", div_mode);
            const int32_t rc = run_codes<QT_FP8>(a, (cudaStream_t)stream, "gemm_fp8_rkv");
            if (rc != RWKVQ_OK) return rc;
        }
        return RWKVQ_OK;
    }
    W8Args a{};
    a.codes[0] = codes_r; a.codes[1] = codes_k; a.codes[2] = codes_v; a.lda = lda;
    a.ascale[0] = amax3; a.ascale[1] = amax3 + 1; a.ascale[2] = amax3 + 2; a.amax_is_amax = amax_is_amax;
    a.w[0] = wr; a.w[1] = wk; a.w[2] = wv; a.ws[0] = sr; a.ws[1] = sk; a.ws[2] = sv;
    a.out[0] = (__half*)out_r; a.out[1] = (__half*)out_k; a.out[2] = (__half*)out_v;
    a.nmat = nmat; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldw = ldw; a.ldo = ldo; a.div_mode = div_mode; a.flags = flags;
    return gemv_codes_run(a, QT_FP8, (cudaStream_t)stream, "gemm_fp8_rkv");
}

int32_t rwkvq_gemm_int8_rkv(const int8_t* codes_r, const int8_t* codes_k, const int8_t* codes_v, int64_t lda, const float* scales_r,
                            const float* scales_k, const float* scales_v, const int8_t* wr, const int8_t* wk, const int8_t* wv,
                            int64_t ldw, const float* sr, const float* sk, const float* sv, void* out_r, void* out_k, void* out_v,
                            int64_t ldo, int64_t M, int64_t N, int64_t K, uint32_t flags, void* stream) {
    const bool shared = (flags & RWKVQ_FLAG_INT8_SHARED_WSCALE) != 0;
    const float* s[3] = {sr, shared ? sr : sk, shared ? sr : sv};
    if (!decode_route(M, K)) {
        const int8_t* c[3] = {codes_r, codes_k, codes_v};
        const float* xs[3] = {scales_r, scales_k, scales_v};
        const int8_t* w[3] = {wr, wk, wv};
        void* o[3] = {out_r, out_k, out_v};
        for (int i = 0; i < 3; ++i) {
            W8Args a{};
            a.a_codes = (const uint8_t*)c[i]; a.lda = lda; a.a_scale = xs[i];
            a.w[0] = (const uint8_t*)w[i]; a.ws[0] = s[i]; a.out[0] = (__half*)o[i];
            a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldw = ldw; a.ldo = ldo; a.div_mode = RWKVQ_DIV_IEEE; a.flags = flags;
            const int32_t rc = run_codes<QT_INT8>(a, (cudaStream_t)stream, "gemm_int8_rkv");
            if (rc != RWKVQ_OK) return rc;
        }
        return RWKVQ_OK;
    }
    W8Args a{};
    a.codes[0] = (const uint8_t*)codes_r; a.codes[1] = (const uint8_t*)codes_k; a.codes[2] = (const uint8_t*)codes_v; a.lda = lda;
    a.ascale[0] = scales_r; a.ascale[1] = scales_k; a.ascale[2] = scales_v;
    a.w[0] = (const uint8_t*)wr; a.w[1] = (const uint8_t*)wk; a.w[2] = (const uint8_t*)wv; a.ws[0] = s[0]; a.ws[1] = s[1]; a.ws[2] = s[2];
    a.out[0] = (__half*)out_r; a.out[1] = (__half*)out_k; a.out[2] = (__half*)out_v;
    a.nmat = 3; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldw = ldw; a.ldo = ldo; a.div_mode = RWKVQ_DIV_IEEE; a.flags = flags;
    return gemv_codes_run(a, QT_INT8, (cudaStream_t)stream, "gemm_int8_rkv");
}

}  // extern "C"
