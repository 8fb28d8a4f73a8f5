// NVFP4 (W4A4) projection of many tokens on the block-scaled tensor-core path:
//     TMA -> shared memory -> tcgen05.mma.kind::mxf4nvf4.block_scale.block16 -> tensor memory -> fp16 rows.
//
// Operands.  A = activation codes [M, K/2] (two e2m1 per byte, even k in the low nibble), B = weight codes
// [N, K/2]; both K-major, fetched as 128-byte rows (256 values of k) with the 128-byte swizzle, so one ring stage
// feeds four MMAs of K = 64.  Every 16 consecutive k of a row share one e4m3 scale factor.  The tensor core
// reads the scale factors from tensor memory, 4 bytes (= one K-64 step) per row, rows r, r+32, r+64, r+96 side
// by side in 4 columns of lane r % 32; `tcgen05.cp.32x128b.warpx4` copies exactly one such 512-byte chunk
// (128 rows x 4 scales, byte offset (r % 32) * 16 + (r / 32) * 4 + kblock) from shared to tensor memory.
// The chunks are therefore kept in global memory in that order ("blocked" scales, produced once per weight by
// rwkvq_nvfp4_pack_scales and per call for the activations): the scales of one stage and one 128-row tile are
// 2048 contiguous bytes, fetched by one bulk copy onto the same mbarrier as the code tiles.
//
// One persistent CTA per SM: warp 0 = producer (one lane), warp 1 = MMA issuer (one lane) and owner of the
// tensor-memory allocation, warps 2-5 = epilogue (one lane quarter each).  Tile 128 tokens x BN weight rows;
// BN = 128 keeps two accumulators in tensor memory so the epilogue of a tile overlaps the MMAs of the next,
// BN = 256 keeps one.  Every mbarrier wait is bounded; a timeout is reported through the status word.
//
// The format is described in the reference's reports (iterations/phase1_nvfp4_exploration/reports/
// 03_fused_kernel_en.md:22-34, 11_fused_gemm_ops_en.md:20-26); the reference ships no code for it.
#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "tc_common.cuh"
#include "tc_host.cuh"
#include "w8a8.cuh"

namespace rwkvq {
using namespace tc;

constexpr int kNfThreads = 192;
constexpr int kNfMaxStages = 8;
constexpr uint32_t kNfRowBytes = 128;                       // packed codes of one row per stage (256 values of k)
constexpr uint32_t kNfABytes = kNfTileM * kNfRowBytes;      // 16 KiB
constexpr uint32_t kNfSfCol = 256;                          // first tensor-memory column of the scale factors
constexpr uint32_t kNfTmemCols = 512;
constexpr size_t kNfSmemBudget = 225 * 1024;

struct NfMaps {
    CUtensorMap a, w;
};

// PUSH instantiation: the GEMM carries the all-gather of a column-split projection (TcPush in tc_host.cuh).
struct NfArgs {
    TcPush push;
    const uint8_t* sfa;      // blocked activation scales
    const uint8_t* sfw;      // blocked weight scales
    const float* a_pts;
    const float* w_pts;
    __half* out;
    int64_t ldo;
    int M, N, K;
    int mtiles, ntiles, kstages, stages;
    int* status;
    unsigned long long wait_ns;   // wall-time limit of every mbarrier wait
};

struct NfShared {
    uint64_t full[kNfMaxStages], empty[kNfMaxStages], tfull[2], tempty[2], done;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void nf_abort(NfShared& s, const NfArgs& a) {
    s.abort_flag = 1;
    if (a.status) atomicExch(a.status, RWKVQ_E_TIMEOUT);
}

template <int BN, bool PUSH = false>
__global__ void __launch_bounds__(kNfThreads, 1) gemm_tc_nvfp4_kernel(const __grid_constant__ NfMaps maps, const NfArgs a) {
    constexpr int NACC = BN == 128 ? 2 : 1;
    constexpr int NH = BN / 128;                                   // 128-row scale tiles of the B operand
    constexpr uint32_t kBBytes = BN * kNfRowBytes;
    constexpr uint32_t kStage = kNfABytes + kBBytes + kNfSfStage * (1 + NH);
    extern __shared__ uint8_t smem_raw[];
    __shared__ NfShared s;
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    griddep_launch_dependents();
    if (threadIdx.x == 0) {
        for (int i = 0; i < a.stages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.tfull[i], 1);
            mbar_init(&s.tempty[i], 4);
        }
        mbar_init(&s.done, 4);
        s.abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tmap(&maps.a);
        prefetch_tmap(&maps.w);
    }
    if (warp == 1) tmem_alloc(&s.tmem_base, kNfTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = s.tmem_base;
    const volatile int* abort_flag = &s.abort_flag;
    const int tiles = a.mtiles * a.ntiles;
    const int64_t k64 = a.K >> 6;

    if (warp == 0) {
        // ============================== producer ==============================
        if (lane == 0) {
            // first pass over the ring: the weights and their scales do not depend on the kernels in front, so they are
            // requested BEFORE the dependency wait of programmatic dependent launch
            uint32_t npre = 0;
            for (; npre < (uint32_t)a.stages; ++npre) {
                const int t = blockIdx.x + (int)(npre / (uint32_t)a.kstages) * (int)gridDim.x, kc = (int)(npre % (uint32_t)a.kstages);
                if (t >= tiles) break;
                const int nt = t / a.mtiles;
                uint8_t* dst = ring + (size_t)npre * kStage;
                mbar_expect_tx(&s.full[npre], kStage);
                tma_load_2d(dst + kNfABytes, &maps.w, kc * (int)kNfRowBytes, nt * BN, &s.full[npre]);
                uint8_t* sf = dst + kNfABytes + kBBytes;
#pragma unroll
                for (int h = 0; h < NH; ++h)
                    bulk_load_1d(sf + kNfSfStage * (1 + h), a.sfw + ((int64_t)(nt * NH + h) * k64 + kc * 4) * kNfSfChunk, kNfSfStage, &s.full[npre]);
            }
            griddep_wait();                     // activation codes and scales come from the previous kernels
            uint32_t n = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const int mt = t % a.mtiles, nt = t / a.mtiles;
                for (int kc = 0; kc < a.kstages; ++kc, ++n) {
                    const int st = n % a.stages;
                    uint8_t* dst = ring + (size_t)st * kStage;
                    uint8_t* sf = dst + kNfABytes + kBBytes;
                    if (n >= npre) {
                        if (!mbar_wait(&s.empty[st], ((n / a.stages) & 1) ^ 1, abort_flag, a.wait_ns)) { nf_abort(s, a); ok = false; break; }
                        mbar_expect_tx(&s.full[st], kStage);
                        tma_load_2d(dst + kNfABytes, &maps.w, kc * (int)kNfRowBytes, nt * BN, &s.full[st]);
#pragma unroll
                        for (int h = 0; h < NH; ++h)
                            bulk_load_1d(sf + kNfSfStage * (1 + h), a.sfw + ((int64_t)(nt * NH + h) * k64 + kc * 4) * kNfSfChunk,
                                         kNfSfStage, &s.full[st]);
                    }
                    tma_load_2d(dst, &maps.a, kc * (int)kNfRowBytes, mt * kNfTileM, &s.full[st]);
                    bulk_load_1d(sf, a.sfa + ((int64_t)mt * k64 + kc * 4) * kNfSfChunk, kNfSfStage, &s.full[st]);
                }
            }
            if (!ok) {   // give copies already in flight a bounded time to land before the CTA's memory is released
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 2000000ull) {}
            }
        }
    } else if (warp == 1) {
        // ============================== MMA issuer ==============================
        if (lane == 0) {
            const uint32_t idesc = nvfp4_idesc(BN);
            uint32_t n = 0, pc = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++pc) {
                const int buf = pc % NACC;
                if (!mbar_wait(&s.tempty[buf], ((pc / NACC) & 1) ^ 1, abort_flag, a.wait_ns)) { nf_abort(s, a); break; }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + (uint32_t)(buf * BN);
                for (int kc = 0; kc < a.kstages; ++kc, ++n) {
                    const int st = n % a.stages;
                    if (!mbar_wait(&s.full[st], (n / a.stages) & 1, abort_flag, a.wait_ns)) { nf_abort(s, a); ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(ring + (size_t)st * kStage);
                    const uint32_t ssf = sa + kNfABytes + kBBytes;
                    // scale factors of this stage: two alternating column sets, so a copy never lands in columns
                    // the previous stage's MMAs may still be reading
                    const uint32_t tsfa = tmem_base + kNfSfCol + (n & 1) * 64;
                    const uint32_t tsfb = tsfa + 16;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        tc_cp_sf(tsfa + k * 4, sf_desc(ssf + k * kNfSfChunk));
#pragma unroll
                        for (int h = 0; h < NH; ++h)
                            tc_cp_sf(tsfb + k * (4 * NH) + h * 4, sf_desc(ssf + kNfSfStage * (1 + h) + k * kNfSfChunk));
                    }
                    const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sa + kNfABytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc_mma_nvfp4(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, tsfa + k * 4, tsfb + k * (4 * NH),
                                     (kc > 0 || k > 0) ? 1u : 0u);
                    tc_commit(&s.empty[st]);            // the stage may be refilled once these MMAs have read it
                }
                if (ok) tc_commit(&s.tfull[buf]);
            }
        }
    } else {
        // ============================== epilogue ==============================
        griddep_wait();
        const int q = warp & 3;                         // tensor-memory lane quarter this warp may read
        const float scale = a.a_pts[0] * a.w_pts[0];
        const bool vec_ok = (a.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.out) & 15) == 0);
        uint32_t pc = 0;
        for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++pc) {
            const int mt = t % a.mtiles, nt = t / a.mtiles;
            const int buf = pc % NACC;
            if (!mbar_wait(&s.tfull[buf], (pc / NACC) & 1, abort_flag, a.wait_ns)) { nf_abort(s, a); break; }
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(q * 32) << 16);
            const int m = mt * kNfTileM + q * 32 + lane;
            if constexpr (PUSH) {
                // the warp turns its 32 rows x 64 columns around in shared memory and stores whole 128-byte row segments
                uint8_t* stg = ring + (size_t)a.stages * kStage + (size_t)(warp - 2) * kTcStgWarp;
                const bool vec8 = vec_ok && a.N % 8 == 0;
                for (int c0 = 0; c0 < BN; c0 += 64) {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        uint32_t r[16];
                        tmem_ld16(taddr + c0 + cc * 16, r);
                        tmem_ld_wait();
                        uint32_t h[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const __half2 hh = __floats2half2_rn(__uint_as_float(r[2 * j]) * scale, __uint_as_float(r[2 * j + 1]) * scale);
                            h[j] = *reinterpret_cast<const uint32_t*>(&hh);
                        }
                        uint4* d = reinterpret_cast<uint4*>(stg + lane * kTcStgRow + cc * 32);
                        d[0] = make_uint4(h[0], h[1], h[2], h[3]);
                        d[1] = make_uint4(h[4], h[5], h[6], h[7]);
                    }
                    __syncwarp();
                    push_store_rows(a.push, stg, a.out, a.ldo, mt * kNfTileM + q * 32, nt * BN + c0, a.M, a.N, vec8, lane);
                    __syncwarp();
                }
            } else {
#pragma unroll 2
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(taddr + c0, r);
                tmem_ld_wait();
                const int n0 = nt * BN + c0;
                if (m < a.M && n0 < a.N) {
                    uint32_t h[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const __half2 hh = __floats2half2_rn(__uint_as_float(r[2 * j]) * scale, __uint_as_float(r[2 * j + 1]) * scale);
                        h[j] = *reinterpret_cast<const uint32_t*>(&hh);
                    }
                    __half* o = a.out + (int64_t)m * a.ldo + n0;
                    if (vec_ok && n0 + 16 <= a.N) {
                        reinterpret_cast<uint4*>(o)[0] = make_uint4(h[0], h[1], h[2], h[3]);
                        reinterpret_cast<uint4*>(o)[1] = make_uint4(h[4], h[5], h[6], h[7]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (n0 + j < a.N) o[j] = __ushort_as_half((unsigned short)((h[j >> 1] >> ((j & 1) * 16)) & 0xffff));
                    }
                }
            }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.tempty[buf]);
        }
        if constexpr (PUSH) __threadfence_system();      // this thread's peer stores are ordered before its arrival below
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.done);
    }

    __syncwarp();            // single-lane roles: the other lanes wait here for their lane 0
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        // the accumulators are released only after every epilogue warp has read its last one
        if (!mbar_wait(&s.done, 0, abort_flag, a.wait_ns)) nf_abort(s, a);
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kNfTmemCols);
        if constexpr (PUSH) {
            if (lane == 0) push_signal(a.push);
        }
    }
}

// row-major scales [rows, K/16] -> blocked chunks [ceil(rows/256)*2][K/64][512]; one thread per 4-byte word
__global__ void __launch_bounds__(256) nvfp4_pack_scales_kernel(const uint8_t* __restrict__ sf, int64_t ld, int64_t rows, int64_t k64,
                                                                int64_t words, uint32_t* __restrict__ out) {
    const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= words) return;
    const int64_t chunk = w >> 7;
    const int inner = (int)(w & 127);
    const int64_t tile = chunk / k64, kq = chunk - tile * k64;
    const int64_t row = tile * 128 + (inner & 3) * 32 + (inner >> 2);
    out[w] = row < rows ? *reinterpret_cast<const uint32_t*>(sf + row * ld + kq * 4) : 0u;
}

template <int BN, bool PUSH = false>
static int32_t launch_nvfp4(const NfMaps& maps, NfArgs a, int grid, cudaStream_t st, const char* who) {
    auto kern = gemm_tc_nvfp4_kernel<BN, PUSH>;
    const int32_t rc = ensure_smem_optin(reinterpret_cast<const void*>(kern), (int)kNfSmemBudget, who);   // per device
    if (rc != RWKVQ_OK) return rc;
    const size_t stage = kNfABytes + (size_t)BN * kNfRowBytes + kNfSfStage * (1 + BN / 128);
    const size_t staging = PUSH ? kTcStgBytes : 0;          // the pushing epilogue turns its tiles around in shared memory
    a.stages = (int)std::min<size_t>(kNfMaxStages, (kNfSmemBudget - 1024 - staging) / stage);
    const size_t smem = (size_t)a.stages * stage + staging + 1024;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kNfThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl() ? 1 : 0;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kern, maps, a);
    if (err != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(err));
    }
    return check_launch(who);
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

int64_t rwkvq_nvfp4_blocked_scale_bytes(int64_t rows, int64_t K) {
    if (rows <= 0 || K <= 0) return 0;
    return ((rows + 255) / 256) * 2 * ((K + 63) / 64) * (int64_t)kNfSfChunk;
}

int32_t rwkvq_nvfp4_pack_scales(const uint8_t* block_scales, int64_t lds, int64_t rows, int64_t K, uint8_t* blocked, void* stream) {
    const char* who = "nvfp4_pack_scales";
    RWKVQ_REQUIRE(rows >= 0 && K >= 0 && K % 64 == 0, RWKVQ_E_SHAPE, "%s: K=%lld must be a multiple of 64", who, (long long)K);
    if (rows == 0 || K == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(block_scales && blocked, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(((uintptr_t)block_scales & 3) == 0 && lds % 4 == 0 && lds >= K / 16, RWKVQ_E_ALIGN, "%s: scale rows must be 4-byte aligned", who);
    RWKVQ_REQUIRE(aligned16(blocked), RWKVQ_E_ALIGN, "%s: the blocked buffer must be 16-byte aligned", who);
    const int64_t words = rwkvq_nvfp4_blocked_scale_bytes(rows, K) / 4;
    nvfp4_pack_scales_kernel<<<(unsigned)((words + 255) / 256), 256, 0, (cudaStream_t)stream>>>(block_scales, lds, rows, K / 64, words,
                                                                                                reinterpret_cast<uint32_t*>(blocked));
    return check_launch(who);
}

static int32_t run_tc_nvfp4(const uint8_t* a_codes, int64_t lda, const uint8_t* a_scales_blocked, const float* a_pts,
                            const uint8_t* w_codes, int64_t ldw, const uint8_t* w_scales_blocked, const float* w_tscale,
                            void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace, int64_t workspace_bytes,
                            void* stream, const TcPush* push, const char* who) {
    RWKVQ_REQUIRE(M >= 0 && N >= 0 && K >= 0, RWKVQ_E_SHAPE, "%s: negative size", who);
    RWKVQ_REQUIRE(K % 256 == 0, RWKVQ_E_SHAPE, "%s: K=%lld must be a multiple of 256", who, (long long)K);
    RWKVQ_REQUIRE(ldo >= N, RWKVQ_E_SHAPE, "%s: ldo < N", who);
    if (M == 0 || N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(K > 0, RWKVQ_E_SHAPE, "%s: K=0", who);
    RWKVQ_REQUIRE(a_codes && a_scales_blocked && a_pts && w_codes && w_scales_blocked && w_tscale && out_f16, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(aligned16(a_scales_blocked) && aligned16(w_scales_blocked), RWKVQ_E_ALIGN, "%s: blocked scales must be 16-byte aligned", who);
    RWKVQ_REQUIRE(M < (int64_t(1) << 30) && N < (int64_t(1) << 30) && K < (int64_t(1) << 30), RWKVQ_E_SHAPE, "%s: size too large", who);
    RWKVQ_REQUIRE(workspace == nullptr || (workspace_bytes >= kWsHeaderBytes && aligned16(workspace)), RWKVQ_E_WORKSPACE,
                  "%s: the workspace needs at least %lld bytes, 16-byte aligned", who, (long long)kWsHeaderBytes);
    if (push == nullptr && tcs_nvfp4_eligible(M, N, K))         // few tokens: K split across a thread-block cluster
        return run_tcs_nvfp4(a_codes, lda, a_scales_blocked, a_pts, w_codes, ldw, w_scales_blocked, w_tscale, (__half*)out_f16, ldo, M, N, K,
                             workspace ? reinterpret_cast<int*>(workspace) + kWsCounterInts : nullptr, (cudaStream_t)stream, who);
    const char* bn_env = std::getenv("RWKVQ_NF4_BN");          // read per call: a test switches tiles in one process
    const int forced_bn = bn_env ? std::atoi(bn_env) : 0;
    // 256-row weight tiles halve the activation re-reads per flop but keep one accumulator; they pay once there are
    // enough of them to fill the SMs
    const int64_t tiles256 = ((M + kNfTileM - 1) / kNfTileM) * ((N + 255) / 256);
    const int bn = forced_bn == 128 || forced_bn == 256 ? forced_bn : (tiles256 * 4 >= (int64_t)sm_count() * 3 ? 256 : 128);
    NfArgs a{};
    if (push) a.push = *push;
    a.wait_ns = wait_limit_ns();
    a.sfa = a_scales_blocked; a.sfw = w_scales_blocked; a.a_pts = a_pts; a.w_pts = w_tscale; a.out = (__half*)out_f16; a.ldo = ldo;
    a.M = (int)M; a.N = (int)N; a.K = (int)K;
    a.mtiles = (int)((M + kNfTileM - 1) / kNfTileM);
    a.ntiles = (int)((N + bn - 1) / bn);
    a.kstages = (int)(K / 256);
    a.status = workspace ? reinterpret_cast<int*>(workspace) + kWsCounterInts : nullptr;
    const int64_t tiles = (int64_t)a.mtiles * a.ntiles;
    RWKVQ_REQUIRE(tiles < (int64_t(1) << 30), RWKVQ_E_SHAPE, "%s: too many tiles", who);
    NfMaps maps;
    int32_t rc = make_map(&maps.a, a_codes, M, K / 2, lda, kNfTileM, who);
    if (rc) return rc;
    rc = make_map(&maps.w, w_codes, N, K / 2, ldw, bn, who);
    if (rc) return rc;
    const int grid = (int)std::min<int64_t>(sm_count(), tiles);
    if (push)
        return bn == 128 ? launch_nvfp4<128, true>(maps, a, grid, (cudaStream_t)stream, who) : launch_nvfp4<256, true>(maps, a, grid, (cudaStream_t)stream, who);
    return bn == 128 ? launch_nvfp4<128>(maps, a, grid, (cudaStream_t)stream, who) : launch_nvfp4<256>(maps, a, grid, (cudaStream_t)stream, who);
}

/* 1 if rwkvq_tc_gemm_nvfp4 runs these sizes on the cluster split-K kernel (few tokens), 0 for the tiled form */
int32_t rwkvq_tc_gemm_nvfp4_cluster_route(int64_t M, int64_t N, int64_t K) { return tcs_nvfp4_eligible(M, N, K) ? 1 : 0; }

int32_t rwkvq_tc_gemm_nvfp4(const uint8_t* a_codes, int64_t lda, const uint8_t* a_scales_blocked, const float* a_pts,
                            const uint8_t* w_codes, int64_t ldw, const uint8_t* w_scales_blocked, const float* w_tscale,
                            void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace, int64_t workspace_bytes,
                            void* stream) {
    return run_tc_nvfp4(a_codes, lda, a_scales_blocked, a_pts, w_codes, ldw, w_scales_blocked, w_tscale, out_f16, ldo, M, N, K, workspace,
                        workspace_bytes, stream, nullptr, "tc_gemm_nvfp4");
}

/* rwkvq_tc_gemm_nvfp4 fused with the all-gather of a column-split projection: every result vector is also stored, by
 * peer stores over NVLink, at the same offset behind peer_out[p] (this rank's column range in rank p's [M, ldo] buffer,
 * 16-byte aligned like out_f16), p < npeers <= 7; when the whole grid is done, `epoch` is published at peer_flag[p]
 * (this rank's slot in rank p's flag array; see rwkvq_peer_wait).  The workspace (zeroed once, as for the other
 * tensor-memory entries) is required: it holds the count of finished CTAs.  M > 0 on every rank. */
int32_t rwkvq_tc_gemm_nvfp4_push(const uint8_t* a_codes, int64_t lda, const uint8_t* a_scales_blocked, const float* a_pts,
                                 const uint8_t* w_codes, int64_t ldw, const uint8_t* w_scales_blocked, const float* w_tscale,
                                 void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace, int64_t workspace_bytes,
                                 void* const* peer_out, void* const* peer_flag, int32_t npeers, uint32_t epoch, void* stream) {
    const char* who = "tc_gemm_nvfp4_push";
    RWKVQ_REQUIRE(M > 0 && N > 0, RWKVQ_E_SHAPE, "%s: empty result (the peers would wait for a signal that never comes)", who);
    TcPush push;
    const int32_t rc = make_push(&push, workspace, workspace_bytes, out_f16, peer_out, peer_flag, npeers, epoch, who);
    if (rc != RWKVQ_OK) return rc;
    return run_tc_nvfp4(a_codes, lda, a_scales_blocked, a_pts, w_codes, ldw, w_scales_blocked, w_tscale, out_f16, ldo, M, N, K, workspace,
                        workspace_bytes, stream, &push, who);
}

}  // extern "C"
