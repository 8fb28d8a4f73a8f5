// Host-side helpers shared by the tensor-memory kernels: the driver's tensor-map encoder (looked up through the
// runtime, so the library does not link libcuda) and the tile map every operand uses.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace rwkvq {

// caller-provided workspace of the tensor-memory kernels: arrival counters, the status word, then partial sums
constexpr int64_t kWsCounterInts = 1024;                       // arrival counters (row tiles of all matrices)
constexpr int64_t kWsHeaderBytes = (kWsCounterInts + 16) * 4;  // counters + status word, then the partial sums

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// byte matrix [rows, row_bytes] with `ld` bytes between rows, tiles of box_rows x 128 bytes, 128-byte swizzle, zero fill
inline int32_t make_map(CUtensorMap* m, const void* ptr, int64_t rows, int64_t row_bytes, int64_t ld, int box_rows, const char* who) {
    EncodeTiledFn fn = encode_fn();
    RWKVQ_REQUIRE(fn != nullptr, RWKVQ_E_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", who);
    RWKVQ_REQUIRE(aligned16(ptr) && ld % 16 == 0 && ld >= row_bytes, RWKVQ_E_ALIGN, "%s: TMA needs a 16-byte aligned base and row pitch", who);
    const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld};
    const cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RWKVQ_REQUIRE(r == CUDA_SUCCESS, RWKVQ_E_LAUNCH, "%s: cuTensorMapEncodeTiled failed (%d)", who, (int)r);
    return RWKVQ_OK;
}

// W8A8 GEMM on CTA pairs (gemm_tc2.cu): eligibility (many tokens, enough 256 x 256 tiles to fill the pairs, not switched
// off with RWKVQ_TC2=0) and the launch.  kind: tc::KIND_F8 / tc::KIND_I8.
bool tc2_eligible(int kind, int64_t M, int64_t N, int64_t K, int nmat);
int32_t run_tc2(int kind, const void* codes, int64_t lda, const float* a_scale, int amax_is_amax, const void* w, int64_t ldw, const float* ws,
                __half* out, int64_t ldo, int32_t* acc, int64_t ldacc, int M, int N, int K, int div_mode, uint32_t flags, float* ffn_amax,
                int* status, cudaStream_t st, const char* who);

}  // namespace rwkvq
