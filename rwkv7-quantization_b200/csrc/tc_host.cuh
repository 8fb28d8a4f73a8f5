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

// A GEMM fused with the all-gather of a column-split projection (result wanted on every rank): its epilogue stores each
// result vector not only to this rank's buffer but, with plain peer stores over NVLink, to the same place in the buffer
// of every other rank, so the gather travels while the tensor cores work on the next tiles.  Peer stores want long
// contiguous runs (32-byte row fragments were measured 2 x slower than a pull kernel), so an epilogue warp turns its
// 32 rows x 64 columns around in a shared-memory staging area and stores 128-byte row segments, four rows per
// instruction.  A CTA that has stored its last tile fences at system scope and counts itself; the last CTA of the grid
// publishes `epoch` in this rank's slot of every peer's flag array (system-scope release).  The receivers only wait for
// the flags (rwkvq_peer_wait).  No TMA touches peer memory.
constexpr int kTcMaxPush = 7;
constexpr uint32_t kTcStgRow = 144;                         // staging row: 64 fp16 + 16 bytes (rows start in different banks)
constexpr uint32_t kTcStgWarp = 32 * kTcStgRow;             // 32 rows per epilogue warp
constexpr size_t kTcStgBytes = 4 * (size_t)kTcStgWarp;      // four epilogue warps
struct TcPush {
    __half* out[kTcMaxPush];       // this rank's column range in each peer's [M, ldo] buffer
    uint32_t* flag[kTcMaxPush];    // this rank's slot in each peer's flag array
    int* counter;                  // CTAs done, zero between launches (a spare word of the workspace header)
    int n;                         // peers (0: no push)
    uint32_t epoch;
};
constexpr int64_t kWsPushCounter = kWsCounterInts + 8;

// fills `push` from the caller's arrays; the peers' buffers must be aligned like `out`
inline int32_t make_push(TcPush* push, void* workspace, int64_t workspace_bytes, const void* out, void* const* peer_out, void* const* peer_flag,
                         int32_t npeers, uint32_t epoch, const char* who) {
    RWKVQ_REQUIRE(npeers >= 0 && npeers <= kTcMaxPush && (npeers == 0 || (peer_out && peer_flag)), RWKVQ_E_BADARG, "%s: %d peers (0..%d)", who, npeers, kTcMaxPush);
    RWKVQ_REQUIRE(workspace != nullptr && workspace_bytes >= kWsHeaderBytes, RWKVQ_E_WORKSPACE, "%s: needs the workspace", who);
    *push = TcPush{};
    push->n = npeers;
    push->epoch = epoch;
    push->counter = reinterpret_cast<int*>(workspace) + kWsPushCounter;
    for (int i = 0; i < npeers; ++i) {
        RWKVQ_REQUIRE(peer_out[i] && peer_flag[i] && ((uintptr_t)peer_flag[i] & 3) == 0, RWKVQ_E_BADARG, "%s: peer %d", who, i);
        RWKVQ_REQUIRE(((uintptr_t)peer_out[i] & 15) == ((uintptr_t)out & 15), RWKVQ_E_ALIGN, "%s: peer buffer %d is aligned differently from out", who, i);
        push->out[i] = reinterpret_cast<__half*>(peer_out[i]);
        push->flag[i] = reinterpret_cast<uint32_t*>(peer_flag[i]);
    }
    return RWKVQ_OK;
}

#ifdef __CUDACC__
// one thread per CTA, after every epilogue thread of the CTA has fenced and arrived
__device__ __forceinline__ void push_signal(const TcPush& p) {
    __threadfence_system();
    if (atomicAdd(p.counter, 1) == (int)gridDim.x - 1) {            // every CTA's tiles are stored on every rank
        *p.counter = 0;
        __threadfence_system();
        for (int i = 0; i < p.n; ++i) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flag[i]), "r"(p.epoch) : "memory");
    }
}
// the coalesced half of the staged epilogue: 32 rows x 64 columns from `stg` to this rank's buffer and the peers'
__device__ __forceinline__ void push_store_rows(const TcPush& p, const uint8_t* stg, __half* out, int64_t ldo, int row0, int col0, int M, int N,
                                                bool vec8, int lane) {
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int row = it * 4 + (lane >> 3), ch = lane & 7;
        const int mm = row0 + row, n0 = col0 + ch * 8;
        const uint4 v = *reinterpret_cast<const uint4*>(stg + row * kTcStgRow + ch * 16);
        if (mm < M && n0 < N) {
            const int64_t off = (int64_t)mm * ldo + n0;
            if (vec8) {
                *reinterpret_cast<uint4*>(out + off) = v;
                for (int i = 0; i < p.n; ++i) *reinterpret_cast<uint4*>(p.out[i] + off) = v;
            } else {
                const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (n0 + j < N) {
                        const __half e = __ushort_as_half((unsigned short)((w4[j >> 1] >> ((j & 1) * 16)) & 0xffff));
                        out[off + j] = e;
                        for (int i = 0; i < p.n; ++i) p.out[i][off + j] = e;
                    }
            }
        }
    }
}
#endif

// W8A8 GEMM on CTA pairs (gemm_tc2.cu): eligibility (many tokens, enough 256 x 256 tiles to fill the pairs, not switched
// off with RWKVQ_TC2=0) and the launch.  kind: tc::KIND_F8 / tc::KIND_I8.
bool tc2_eligible(int kind, int64_t M, int64_t N, int64_t K, int nmat);
int32_t run_tc2(int kind, const void* codes, int64_t lda, const float* a_scale, int amax_is_amax, const void* w, int64_t ldw, const float* ws,
                __half* out, int64_t ldo, int32_t* acc, int64_t ldacc, int M, int N, int K, int div_mode, uint32_t flags, float* ffn_amax,
                int* status, cudaStream_t st, const char* who);

// NVFP4 GEMM for few tokens (up to 256) on the cluster split-K kernel of gemm_tc.cu (gemm_tcs.cuh): weights = the
// 128-row operand, K split across a thread-block cluster, partial sums through distributed shared memory.
bool tcs_nvfp4_eligible(int64_t M, int64_t N, int64_t K);
int32_t run_tcs_nvfp4(const uint8_t* a_codes, int64_t lda, const uint8_t* a_scales_blocked, const float* a_pts, const uint8_t* w_codes,
                      int64_t ldw, const uint8_t* w_scales_blocked, const float* w_tscale, __half* out, int64_t ldo, int64_t M, int64_t N,
                      int64_t K, int* status, cudaStream_t st, const char* who);

}  // namespace rwkvq
