// W8A8 GEMM for many tokens on CTA PAIRS: tcgen05.mma.cta_group::2 (two SMs work on one 256 x 256 tile).
//
// Why pairs.  With one CTA per 128 x 256 tile (gemm_tc.cu) every 128-byte step of K needs 48 KB of operands from L2
// per SM for 512 cycles of tensor-core work -- 96 bytes per clock, more than an SM gets from L2, so the tensor pipe
// idles a third of the time.  In a pair each CTA loads its own 128 token rows and only HALF of the 256 weight rows
// (32 KB per step per SM, 64 bytes per clock); the MMA issued by the pair's leader reads both halves of the weight
// tile from the two CTAs' shared memory and accumulates each CTA's 128 x 256 block in that CTA's own tensor memory.
// No multicast is involved: every TMA load lands in the shared memory of the CTA that issued it.
//
// Roles per CTA as in gemm_tc.cu: warp 0 = TMA producer (one lane), warp 1 = tensor-memory owner and -- in the leader
// CTA only -- MMA issuer, warps 2-5 = epilogue.  Barriers: full[] lives in the leader (both producers' bytes are
// counted there: the loads carry .cta_group::2 and name the leader's barrier), empty[] and tfull[] are signalled in both
// CTAs at once by a multicast tcgen05.commit, tempty[] of the leader collects the arrivals of both CTAs' epilogue warps.
// Every wait is bounded; the pair meets at a cluster barrier before the tensor memory is released.
#include <algorithm>
#include <cstdlib>

#include "tc_common.cuh"
#include "tc_host.cuh"
#include "w8a8.cuh"

namespace rwkvq {
using namespace tc;

constexpr int kT2Threads = 320;
constexpr int kT2MaxStages = 6;
constexpr int kT2Chunk = 128;                 // bytes of K per stage
constexpr int kT2Rows = 128;                  // rows of each operand tile per CTA
constexpr uint32_t kT2TileBytes = kT2Rows * kT2Chunk;      // 16 KB
constexpr uint32_t kT2StageBytes = 2 * kT2TileBytes;       // tokens + this CTA's half of the weight tile
constexpr int kT2N = 256;                     // weight rows per pair tile (UMMA N)

struct Tc2Maps {
    CUtensorMap a;      // activation codes [M, K], box 128 rows x 128 bytes
    CUtensorMap w;      // weights [N, K], box 128 rows x 128 bytes
};

struct Tc2Args {
    const float* a_scale;      // FP8 amax-or-scale [1]; INT8 row scales [M]
    const float* ws;           // weight scale: one value, or N with RWKVQ_FLAG_WSCALE_PER_ROW
    __half* out;
    int32_t* acc;              // INT8: optional raw accumulators
    float* ffn_amax;           // RWKVQ_FLAG_RELU2: maximum of the relu^2 results
    int* status;
    unsigned long long wait_ns;
    int64_t ldo, ldacc;
    int M, N, K;
    int kchunks, ptiles, qtiles, stages;      // ptiles: 256-token pair tiles, qtiles: 256-row weight tiles
    int div_mode, amax_is_amax;
    uint32_t flags;
};

struct Tc2Shared {
    uint64_t full[kT2MaxStages], empty[kT2MaxStages], tfull[2], tempty[2], done;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
// address of `local` in the shared memory of CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tiled load into THIS CTA's shared memory whose bytes are counted on the barrier of the pair's leader CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, int x, int y, uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(leader_bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {      // the same warp in both CTAs
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// all MMAs issued so far by this thread have completed -> arrive on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    const unsigned short mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
template <int KIND>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (KIND == KIND_F8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    }
}

__device__ __forceinline__ void t2_abort(Tc2Shared& s, const Tc2Args& a) {
    s.abort_flag = 1;
    if (a.status) atomicExch(a.status, RWKVQ_E_TIMEOUT);
}

template <int KIND>
__global__ void __launch_bounds__(kT2Threads, 1) gemm_tc2_kernel(const __grid_constant__ Tc2Maps maps, const Tc2Args a) {
    using T = typename Acc<KIND == KIND_F8 ? QT_FP8 : QT_INT8>::T;
    extern __shared__ uint8_t smem_raw[];
    __shared__ Tc2Shared s;
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader of the pair
    const int pair = (int)(blockIdx.x >> 1), npairs = (int)(gridDim.x >> 1);
    const int total = a.ptiles * a.qtiles;
    constexpr uint32_t kCols = 512;                   // two 256-column accumulators

    griddep_launch_dependents();
    if (threadIdx.x == 0) {
        for (int i = 0; i < a.stages; ++i) {
            mbar_init(&s.full[i], 1);                 // the leader's expect_tx arrival; both CTAs' bytes
            mbar_init(&s.empty[i], 1);                // one multicast commit per use
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.tfull[i], 1);
            mbar_init(&s.tempty[i], 8);               // four epilogue warps of each CTA (used in the leader only)
        }
        mbar_init(&s.done, 4);
        s.abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tmap(&maps.a);
        prefetch_tmap(&maps.w);
    }
    if (warp == 1) tmem_alloc_pair(&s.tmem_base, kCols);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                               // the peer's barriers exist before anything signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = s.tmem_base;
    const volatile int* abort_flag = &s.abort_flag;

    auto tile_rows = [&](int t, int& mrow, int& nrow) {       // token tiles fastest: the pairs running together share weight tiles
        mrow = (t % a.ptiles) * 256;
        nrow = (t / a.ptiles) * kT2N;
    };

    if (warp == 0) {
        // ============================== TMA producer (both CTAs) ==============================
        if (lane == 0) {
            griddep_wait();                           // the activation codes come from the previous kernel
            uint32_t n = 0;
            bool ok = true;
            for (int t = pair; t < total && ok; t += npairs) {
                int mrow, nrow;
                tile_rows(t, mrow, nrow);
                for (int kc = 0; kc < a.kchunks; ++kc, ++n) {
                    const int st = n % a.stages;
                    if (!mbar_wait(&s.empty[st], ((n / a.stages) & 1) ^ 1, abort_flag, a.wait_ns)) { t2_abort(s, a); ok = false; break; }
                    uint8_t* dst = ring + (size_t)st * kT2StageBytes;
                    if (rank == 0) mbar_expect_tx(&s.full[st], 2 * kT2StageBytes);          // the four tiles of the pair
                    const uint32_t leader_bar = smem_u32(&s.full[st]) & 0xFEFFFFFFu;         // the barrier of the even CTA
                    tma_load_2d_pair(dst, &maps.a, kc * kT2Chunk, mrow + (int)rank * kT2Rows, leader_bar);
                    tma_load_2d_pair(dst + kT2TileBytes, &maps.w, kc * kT2Chunk, nrow + (int)rank * kT2Rows, leader_bar);
                }
            }
            if (!ok) {      // give copies already in flight a bounded time to land before the CTA's memory is released
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 2000000ull) {}
            }
        }
    } else if (warp == 1) {
        // ============================== MMA issuer (leader CTA only) ==============================
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc(KIND, 256, kT2N);
            uint32_t n = 0, pc = 0;
            bool ok = true;
            for (int t = pair; t < total && ok; t += npairs, ++pc) {
                const int buf = pc & 1;
                if (!mbar_wait(&s.tempty[buf], ((pc >> 1) & 1) ^ 1, abort_flag, a.wait_ns)) { t2_abort(s, a); break; }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + (uint32_t)(buf * kT2N);
                for (int kc = 0; kc < a.kchunks; ++kc, ++n) {
                    const int st = n % a.stages;
                    if (!mbar_wait(&s.full[st], (n / a.stages) & 1, abort_flag, a.wait_ns)) { t2_abort(s, a); ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(ring + (size_t)st * kT2StageBytes);
                    const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sa + kT2TileBytes);
#pragma unroll
                    for (int k = 0; k < kT2Chunk / 32; ++k)
                        tc_mma_pair<KIND>(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kc > 0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(&s.empty[st]);          // both CTAs may refill the stage once these MMAs have read it
                }
                if (ok) tc_commit_pair(&s.tfull[buf]);     // both CTAs' epilogues
            }
        }
    } else if (warp < 6) {
        // ============================== epilogue (both CTAs, each its own 128 token rows) ==============================
        griddep_wait();
        const int q = warp & 3;                         // tensor-memory lane quarter this warp may read
        const int row_l = q * 32 + lane;
        const bool per_row = (a.flags & RWKVQ_FLAG_WSCALE_PER_ROW) != 0;
        const bool relu2 = KIND == KIND_F8 && (a.flags & RWKVQ_FLAG_RELU2) != 0;
        const bool hmax_bf16 = (a.flags & RWKVQ_FLAG_AMAX_AFTER_BF16) != 0;
        const float wsc = a.ws[0];
        const uint32_t leader_tempty[2] = {mapa_u32(smem_u32(&s.tempty[0]), 0), mapa_u32(smem_u32(&s.tempty[1]), 0)};
        const bool vec_ok = (a.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.out) & 15) == 0);
        uint32_t pc = 0;
        for (int t = pair; t < total; t += npairs, ++pc) {
            const int buf = pc & 1;
            if (!mbar_wait(&s.tfull[buf], (pc >> 1) & 1, abort_flag, a.wait_ns)) { t2_abort(s, a); break; }
            tc_fence_after_sync();
            int mrow, nrow;
            tile_rows(t, mrow, nrow);
            const int m = mrow + (int)rank * kT2Rows + row_l;
            const uint32_t taddr = tmem_base + (uint32_t)(buf * kT2N) + ((uint32_t)(q * 32) << 16);
            float actscale;
            if constexpr (KIND == KIND_F8) {
                const float am = a.a_scale[0];
                actscale = a.amax_is_amax ? div_mode_f32(fmaxf(am, 1e-12f), 448.f, a.div_mode) : am;
            } else {
                actscale = m < a.M ? a.a_scale[m] : 0.f;
            }
            const float rowscale = actscale * wsc;
            float hmax = 0.f;
            for (int c0 = 0; c0 < kT2N; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(taddr + c0, r);
                tmem_ld_wait();
                const int n0 = nrow + c0;
                if (m < a.M && n0 < a.N) {
                    uint32_t h[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float s0 = rowscale, s1 = rowscale;
                        if (per_row) {
                            s0 = actscale * a.ws[min(n0 + 2 * j, a.N - 1)];
                            s1 = actscale * a.ws[min(n0 + 2 * j + 1, a.N - 1)];
                        }
                        float f0, f1;
                        if constexpr (KIND == KIND_F8) {
                            f0 = __uint_as_float(r[2 * j]) * s0;
                            f1 = __uint_as_float(r[2 * j + 1]) * s1;
                        } else {
                            f0 = (float)(int32_t)r[2 * j] * s0;
                            f1 = (float)(int32_t)r[2 * j + 1] * s1;
                        }
                        if (a.flags & RWKVQ_FLAG_OUT_VIA_BF16) { f0 = bf16_round(f0); f1 = bf16_round(f1); }
                        __half2 hh = __floats2half2_rn(f0, f1);
                        if (relu2) {        // the engine's relu_square on the fp16 result; its maximum goes to the next projection
                            const float2 y = __half22float2(hh);
                            const float v0 = fmaxf(y.x, 0.f), v1 = fmaxf(y.y, 0.f);
                            hh = __floats2half2_rn(v0 * v0, v1 * v1);
                            if (n0 + 2 * j < a.N) {
                                const float2 hv = __half22float2(hh);
                                hmax = fmaxf(hmax, hmax_bf16 ? bf16_round(hv.x) : hv.x);
                                if (n0 + 2 * j + 1 < a.N) hmax = fmaxf(hmax, hmax_bf16 ? bf16_round(hv.y) : hv.y);
                            }
                        }
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
                    if constexpr (KIND == KIND_I8) {
                        if (a.acc) {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (n0 + j < a.N) a.acc[(int64_t)m * a.ldacc + n0 + j] = (int32_t)r[j];
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_tempty[buf]);        // this accumulator may be overwritten
            if (relu2) {
                hmax = warp_max(hmax);
                if (lane == 0 && hmax > 0.f) atomic_max_nonneg(a.ffn_amax, hmax);
            }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.done);
    }

    __syncwarp();            // single-lane roles: the other lanes wait here for their lane 0
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        if (!mbar_wait(&s.done, 0, abort_flag, a.wait_ns)) t2_abort(s, a);     // this CTA's epilogue has read its last accumulator
    }
    cluster_sync_all();      // ... and so has the peer's: the pair's tensor memory (and the leader's barriers) may go
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kCols);
    }
}

// ------------------------------------------------------------------------------------------------ host side
static int t2_grid_pairs() { return std::max(1, sm_count() / 2); }

// Measured on B200 (7.2B shapes, FP8 and INT8): the pair kernel is level with the single-CTA kernel -- +1..3 % from 4096
// tokens on, -2..5 % at 2048 (same number of waves, deeper pipeline to fill) -- so the L2 -> shared-memory traffic it
// halves is not what limits that kernel (under the 1 kW power cap both run at 2.2-2.5 PFLOP/s).  It is therefore used
// from RWKVQ_TC2_MIN_M tokens on (default 4096; RWKVQ_TC2=0 switches it off, RWKVQ_TC2_MIN_M=129 uses it wherever it fits).
bool tc2_eligible(int kind, int64_t M, int64_t N, int64_t K, int nmat) {
    static const int64_t min_m = [] {
        const char* off = std::getenv("RWKVQ_TC2");
        if (off && off[0] == '0') return (int64_t)1 << 62;
        const char* e = std::getenv("RWKVQ_TC2_MIN_M");
        const long long v = e ? std::atoll(e) : 4096;
        return (int64_t)std::max<long long>(v, 129);
    }();
    if (nmat != 1 || M < min_m || N < kT2N || K % 16) return false;
    const int64_t tiles = ((M + 255) / 256) * ((N + kT2N - 1) / kT2N);
    return tiles >= t2_grid_pairs() / 2 && (kind == KIND_F8 || kind == KIND_I8);
}

int32_t run_tc2(int kind, const void* codes, int64_t lda, const float* a_scale, int amax_is_amax, const void* w, int64_t ldw, const float* ws,
                __half* out, int64_t ldo, int32_t* acc, int64_t ldacc, int M, int N, int K, int div_mode, uint32_t flags, float* ffn_amax,
                int* status, cudaStream_t st, const char* who) {
    Tc2Args a{};
    a.a_scale = a_scale; a.ws = ws; a.out = out; a.acc = acc; a.ffn_amax = ffn_amax; a.status = status; a.wait_ns = wait_limit_ns();
    a.ldo = ldo; a.ldacc = ldacc; a.M = M; a.N = N; a.K = K; a.div_mode = div_mode; a.amax_is_amax = amax_is_amax; a.flags = flags;
    a.kchunks = (K + kT2Chunk - 1) / kT2Chunk;
    a.ptiles = (M + 255) / 256;
    a.qtiles = (N + kT2N - 1) / kT2N;
    a.stages = kT2MaxStages;
    const size_t smem = (size_t)a.stages * kT2StageBytes + 1024;
    Tc2Maps maps;
    int32_t rc = make_map(&maps.a, codes, M, K, lda, kT2Rows, who);
    if (rc) return rc;
    rc = make_map(&maps.w, w, N, K, ldw, kT2Rows, who);
    if (rc) return rc;
    const void* kern = kind == KIND_F8 ? (const void*)gemm_tc2_kernel<KIND_F8> : (const void*)gemm_tc2_kernel<KIND_I8>;
    rc = ensure_smem_optin(kern, (int)smem, who);
    if (rc) return rc;
    const int pairs = (int)std::min<int64_t>(t2_grid_pairs(), (int64_t)a.ptiles * a.qtiles);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(kT2Threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl() ? 2 : 1;
    const cudaError_t err = kind == KIND_F8 ? cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<KIND_F8>, maps, a)
                                            : cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<KIND_I8>, maps, a);
    if (err != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(err));
    }
    return check_launch(who);
}

}  // namespace rwkvq
