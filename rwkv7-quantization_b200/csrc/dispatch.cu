// Public GEMM entry points on pre-quantized codes: pick the kernel by M.
#include "common.cuh"

extern "C" {
int32_t rwkvq_gemm_fp8_mma(const uint8_t*, int64_t, const float*, int32_t, const uint8_t*, int64_t, const float*, void*, int64_t,
                           int64_t, int64_t, int64_t, int32_t, uint32_t, void*);
int32_t rwkvq_gemm_int8_mma(const int8_t*, int64_t, const float*, const int8_t*, int64_t, const float*, void*, int64_t, int32_t*,
                            int64_t, int64_t, int64_t, int64_t, uint32_t, void*);

int32_t rwkvq_gemm_fp8(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax, const uint8_t* w,
                       int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                       int32_t div_mode, uint32_t flags, void* stream) {
    return rwkvq_gemm_fp8_mma(a_codes, lda, amax, amax_is_amax, w, ldw, w_scale, out_f16, ldo, M, N, K, div_mode, flags, stream);
}

int32_t rwkvq_gemm_int8(const int8_t* a_codes, int64_t lda, const float* a_scales, const int8_t* w, int64_t ldw,
                        const float* w_scale, void* out_f16, int64_t ldo, int32_t* acc_out, int64_t ldacc, int64_t M,
                        int64_t N, int64_t K, uint32_t flags, void* stream) {
    return rwkvq_gemm_int8_mma(a_codes, lda, a_scales, w, ldw, w_scale, out_f16, ldo, acc_out, ldacc, M, N, K, flags, stream);
}
}
