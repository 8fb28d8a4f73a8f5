// W8A8 projections for small M (decode): FP8 e4m3 x e4m3 and INT8 x INT8, single matrix or r/k/v in one launch.
//
// The kernel is HBM-bound: the weight matrix [N,K] (one byte per element) is read exactly once with 128-bit
// streaming loads straight into registers, and those registers ARE the B fragments of mma.sync.m16n8k32
// (8 weight rows x 32 k per instruction): lane (g = lane/4, t = lane%4) loads the 16 bytes W[n0+g][k0+16t ..+15]
// and feeds them to two MMAs.  An MMA sums over its 32 k-slots, so the slots may be filled in any order as long
// as A and B agree; the A fragment (quantized activations, 16 token rows) is read with the same permutation
// from the code tile in shared memory.
//
// Work split: a CTA is 8 warps working on the same 8 weight rows, each warp on every 8th 64-byte column unit
// (split-K inside the CTA, fixed-order reduction through shared memory, so results are run-to-run identical).
// CTAs are persistent: each takes a contiguous range of the (matrix, row-tile) list, so the activation
// quantization of the prologue is done once per CTA and matrix.
//
// Latency hiding: every lane keeps a ring of D weight loads in flight; a consumed slot is refilled at once with
// the unit D steps ahead, across row-tile boundaries, and the first D loads are issued BEFORE the prologue.
// With programmatic dependent launch the whole prefetch also overlaps the tail of the previous kernel in the
// stream: only the weights (never written by any kernel) are touched before griddepcontrol.wait.
//
// Fused prologue (what prep_x / prep3_x / prep_x_int8 + the in-kernel quantization of the reference do):
//   FP8 : amax over the whole [M,K] call, inv = 448/max(amax,1e-12), code = e4m3(clamp(bf16(x)*inv)),
//         result scale (amax/448)*w_scale.
//   INT8: per row amax, s = 127/amax, code = trunc(clamp(x*s,-128,127)), row scale amax/127.
#include <cstdlib>

#include "w8a8.cuh"

namespace rwkvq {

// ---- asynchronous 16-byte copies global -> shared (bypassing L1): the bytes in flight live in shared memory, not in
// registers, so a CTA keeps S-1 whole chunks (S-1 x D x 4 KB) of weights in flight.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int n = valid ? 16 : 0;                  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One chunk of the K loop: D slots of this thread's staged weights (slot j lies j*4096 bytes further in the stage and
// 512*j bytes further along K) against the activation tile.  All addresses are base pointers plus compile-time
// offsets.  CHECK: K is not a multiple of the chunk span, so every slot is tested against K (staged bytes beyond K
// are zero, the activation loads are skipped).
template <int QT, int MT, int D, bool WIDE, bool CHECK, typename T>
__device__ __forceinline__ void chunk_body(const uint8_t* stage, T (&c)[MT][4], T (&c2)[MT][4], int k0, int K,
                                           const uint8_t* const (&xr)[MT][2]) {
    constexpr int AB = (QT == QT_FP8 && WIDE) ? 2 : 1;        // bytes per activation in the shared-memory tile
#pragma unroll
    for (int j = 0; j < D; ++j) {
        const uint4 wv = *reinterpret_cast<const uint4*>(stage + j * 4096);
        const bool kin = !CHECK || (k0 + j * 512 < K);
        if constexpr (QT == QT_FP8 && WIDE) {
            // widen the 16 weight bytes to f16 pairs; four m16n8k16 MMAs per 16 bytes on two accumulators
            const uint4 w01 = e4m3x8_to_f16x8(make_uint2(wv.x, wv.y)), w23 = e4m3x8_to_f16x8(make_uint2(wv.z, wv.w));
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                uint4 a00 = make_uint4(0, 0, 0, 0), a01 = a00, a10 = a00, a11 = a00;
                if (kin && xr[i][0]) {
                    a00 = *reinterpret_cast<const uint4*>(xr[i][0] + j * 512 * AB);
                    a01 = *reinterpret_cast<const uint4*>(xr[i][0] + j * 512 * AB + 16);
                }
                if (kin && xr[i][1]) {
                    a10 = *reinterpret_cast<const uint4*>(xr[i][1] + j * 512 * AB);
                    a11 = *reinterpret_cast<const uint4*>(xr[i][1] + j * 512 * AB + 16);
                }
                mma_f16(c[i], a00.x, a10.x, a00.y, a10.y, w01.x, w01.y);
                mma_f16(c[i], a00.z, a10.z, a00.w, a10.w, w01.z, w01.w);
                mma_f16(c2[i], a01.x, a11.x, a01.y, a11.y, w23.x, w23.y);
                mma_f16(c2[i], a01.z, a11.z, a01.w, a11.w, w23.z, w23.w);
            }
        } else {
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0;
                if (kin && xr[i][0]) a0 = *reinterpret_cast<const uint4*>(xr[i][0] + j * 512);
                if (kin && xr[i][1]) a1 = *reinterpret_cast<const uint4*>(xr[i][1] + j * 512);
                mma8<QT>(c[i], a0.x, a1.x, a0.y, a1.y, wv.x, wv.y);
                mma8<QT>(c2[i], a0.z, a1.z, a0.w, a1.w, wv.z, wv.w);
            }
        }
    }
}

// WIDE (FP8 only): activations kept as f16 values and weights widened in registers (m16n8k16.f16) instead of
// e4m3 codes multiplied by mma.sync.m16n8k32.e4m3.  S: stages of the shared-memory weight ring.
template <int QT, int DT, int MT, int D, bool WIDE, int S>
__global__ void __launch_bounds__(kThr, 2) gemv_w8a8_kernel(const W8Args a) {
    using T = typename Acc<QT>::T;
    extern __shared__ __align__(16) uint8_t smem[];
    // layout: red[kWarps][MT*4][32] | xs[32] | sh[8] | ring[S][D][256] x 16 B | xq[M][pitch]
    T* red = reinterpret_cast<T*>(smem);
    float* xs = reinterpret_cast<float*>(smem + kWarps * MT * 4 * 32 * 4);
    float* sh = xs + 32;
    uint8_t* ring = reinterpret_cast<uint8_t*>(sh + 8);
    uint8_t* xq = ring + (size_t)S * D * 4096;

    griddep_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ntile = (a.N + 7) >> 3;
    const int total = a.nmat * ntile;
    const int tb = (int)((int64_t)total * blockIdx.x / gridDim.x), te = (int)((int64_t)total * (blockIdx.x + 1) / gridDim.x);
    const int units = (a.K + 63) >> 6;
    const int upw = (units + kWarps - 1) / kWarps;   // 64-byte units per warp and row tile
    const int nchunks = (upw + D - 1) / D;
    const int koff = (warp << 6) + 16 * t;            // this lane's byte offset inside a row for slot 0
    const bool check = (a.K % (D * 512)) != 0;
    uint8_t* my_ring = ring + threadIdx.x * 16;       // this thread's 16 bytes of every slot

    // producer side of the ring: chunk (itile, ich) goes to stage istage; one commit group per chunk
    int itile = tb, ich = 0, istage = 0;
    auto issue = [&]() {
        if (itile < te) {
            const int mat = itile >= 2 * ntile ? 2 : (itile >= ntile ? 1 : 0);
            const int n0 = (itile - mat * ntile) << 3;
            const uint8_t* src = a.w[mat] + (int64_t)min(n0 + g, a.N - 1) * a.ldw + koff + ich * D * 512;
            uint8_t* dst = my_ring + (size_t)istage * D * 4096;
#pragma unroll
            for (int j = 0; j < D; ++j) {
                const bool valid = !check || (koff + (ich * D + j) * 512 < a.K);
                cp_async16(dst + j * 4096, valid ? src + j * 512 : a.w[mat], valid);
            }
            if (++ich == nchunks) { ich = 0; ++itile; }
        }
        cp_async_commit();
        if (++istage == S) istage = 0;
    };
#pragma unroll
    for (int i = 0; i < S - 1; ++i) issue();

    griddep_wait();   // activations may come from the previous kernel; results may overwrite what it read

    int cur_mat = -1, stage = 0;
    float out_scale = 0.f;   // FP8: (amax/448)*w_scale
    float wscale = 0.f;      // INT8: w_scale
    constexpr int AB = (QT == QT_FP8 && WIDE) ? 2 : 1;
    for (int tile = tb; tile < te; ++tile) {
        const int mat = tile >= 2 * ntile ? 2 : (tile >= ntile ? 1 : 0);
        const int n0 = (tile - mat * ntile) << 3;
        if (mat != cur_mat) {
            cur_mat = mat;
            __syncthreads();   // nobody still reads the previous matrix's codes
            if constexpr (QT == QT_FP8) {
                const float amax = quantize_fp8_to_smem<DT, WIDE>(a, mat, xq, sh);
                out_scale = div_mode_f32(amax, 448.f, a.div_mode) * a.ws[mat][0];
            } else {
                quantize_int8_to_smem<DT>(a, mat, xq, xs, sh);
                wscale = a.ws[mat][0];
            }
            __syncthreads();
        }
        T c[MT][4], c2[MT][4];
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) c[i][j] = c2[i][j] = 0;
        // this lane's rows of the activation tile (rows g and g+8 of each 16-row block); null = row beyond M
        const uint8_t* xr[MT][2];
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            xr[i][0] = i * 16 + g < a.M ? xq + (size_t)(i * 16 + g) * a.pitch + (size_t)koff * AB : nullptr;
            xr[i][1] = i * 16 + g + 8 < a.M ? xq + (size_t)(i * 16 + g + 8) * a.pitch + (size_t)koff * AB : nullptr;
        }
        for (int ch = 0; ch < nchunks; ++ch) {
            issue();                       // keep S-1 chunks in flight
            cp_async_wait<S - 1>();        // this thread's copies of the current chunk have landed
            const uint8_t* xc[MT][2];
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                xc[i][0] = xr[i][0] ? xr[i][0] + (size_t)ch * D * 512 * AB : nullptr;
                xc[i][1] = xr[i][1] ? xr[i][1] + (size_t)ch * D * 512 * AB : nullptr;
            }
            const uint8_t* st = my_ring + (size_t)stage * D * 4096;
            if (check) chunk_body<QT, MT, D, WIDE, true>(st, c, c2, koff + ch * D * 512, a.K, xc);
            else chunk_body<QT, MT, D, WIDE, false>(st, c, c2, koff + ch * D * 512, a.K, xc);
            if (++stage == S) stage = 0;
        }
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) c[i][j] += c2[i][j];      // the two accumulators halve the dependent MMA chains

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
            const int m = i * 16 + (l >> 2) + ((j & 2) ? 8 : 0);
            const int n = n0 + 2 * (l & 3) + (j & 1);
            if (m < a.M && n < a.N) {
                float v;
                if constexpr (QT == QT_FP8) {
                    v = s * out_scale;
                } else {
                    if (a.acc[mat]) a.acc[mat][(int64_t)m * a.ldacc + n] = s;
                    v = (float)s * (xs[m] * wscale);
                }
                if (a.flags & RWKVQ_FLAG_OUT_VIA_BF16) v = bf16_round(v);
                a.out[mat][(int64_t)m * a.ldo + n] = __float2half_rn(v);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
}

static size_t smem_bytes(int MT, int M, int pitch, int D, int S) {
    return (size_t)kWarps * MT * 4 * 32 * 4 + 32 * 4 + 8 * 4 + (size_t)S * D * 4096 + (size_t)M * pitch;
}

constexpr size_t kFusedSmemMax = 200 * 1024;

// FP8 weights are widened to f16 in registers by default: measured on B200, mma.sync.m16n8k32.e4m3 is slower than
// cvt.f16x2.e4m3x2 + m16n8k16.f16 for this HBM-bound loop.  RWKVQ_F8_MMA=native selects the e4m3 instruction.
static bool fp8_wide() {
    static const bool on = [] {
        const char* e = std::getenv("RWKVQ_F8_MMA");
        return !(e && e[0] == 'n');
    }();
    return on;
}

static bool use_pdl() {
    static const bool on = [] {
        const char* e = std::getenv("RWKVQ_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

template <int QT, int DT, int MT, int D, bool WIDE, int S>
static int32_t launch_one(const W8Args& a, int64_t tiles, size_t smem, cudaStream_t st) {
    auto kern = gemv_w8a8_kernel<QT, DT, MT, D, WIDE, S>;
    // per instantiation and device: opt in to large dynamic shared memory and ask how many CTAs fit on an SM
    static thread_local int cfg_dev = -1;
    static thread_local size_t cfg_smem = ~size_t(0);
    static thread_local int per_sm = 1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != cfg_dev || smem != cfg_smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFusedSmemMax);
        if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "gemv_w8a8: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        int n = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kThr, smem);
        if (e != cudaSuccess || n < 1) return fail(RWKVQ_E_LAUNCH, "gemv_w8a8: occupancy query failed (%s)", cudaGetErrorString(e));
        per_sm = n;
        cfg_dev = dev;
        cfg_smem = smem;
    }
    const int64_t grid = std::min<int64_t>(tiles, (int64_t)sm_count() * per_sm);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThr);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl() ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
    if (e != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "gemv_w8a8: %s", cudaGetErrorString(e));
    }
    return check_launch("gemv_w8a8");
}

constexpr size_t kTwoPerSm = 110 * 1024;     // shared memory per CTA that still lets two CTAs share an SM

template <int QT, int DT, int MT, int D, bool WIDE>
static int32_t dispatch_s(const W8Args& a, int64_t tiles, cudaStream_t st) {
    const size_t s3 = smem_bytes(MT, a.M, a.pitch, D, 3), s2 = smem_bytes(MT, a.M, a.pitch, D, 2);
    if (s3 <= kTwoPerSm) return launch_one<QT, DT, MT, D, WIDE, 3>(a, tiles, s3, st);
    RWKVQ_REQUIRE(s2 <= kFusedSmemMax, RWKVQ_E_SHAPE, "gemv_w8a8: M*K = %d*%d does not fit the fused kernel's shared memory", a.M, a.K);
    return launch_one<QT, DT, MT, D, WIDE, 2>(a, tiles, s2, st);
}

template <int QT, int DT>
static int32_t dispatch_mt(const W8Args& a, int64_t tiles, cudaStream_t st) {
    const int units = (a.K + 63) / 64;
    const bool deep = units > 4 * kWarps;          // more than 4 units per warp and tile: chunks of 8 slots
    if (QT == QT_FP8 && fp8_wide()) {
        if (a.M <= 16) return deep ? dispatch_s<QT, DT, 1, 8, true>(a, tiles, st) : dispatch_s<QT, DT, 1, 4, true>(a, tiles, st);
        return deep ? dispatch_s<QT, DT, 2, 8, true>(a, tiles, st) : dispatch_s<QT, DT, 2, 4, true>(a, tiles, st);
    }
    if (a.M <= 16) return deep ? dispatch_s<QT, DT, 1, 8, false>(a, tiles, st) : dispatch_s<QT, DT, 1, 4, false>(a, tiles, st);
    return deep ? dispatch_s<QT, DT, 2, 8, false>(a, tiles, st) : dispatch_s<QT, DT, 2, 4, false>(a, tiles, st);
}

template <int QT>
static int32_t run_fused(W8Args a, int x_dtype, cudaStream_t st, const char* who) {
    RWKVQ_REQUIRE(a.M >= 0 && a.N >= 0 && a.K >= 0, RWKVQ_E_SHAPE, "%s: negative size", who);
    RWKVQ_REQUIRE(a.K % 16 == 0, RWKVQ_E_SHAPE, "%s: K=%d must be a multiple of 16", who, a.K);
    RWKVQ_REQUIRE(a.ldw >= a.K && a.ldw % 16 == 0, RWKVQ_E_ALIGN, "%s: ldw=%lld must be >= K and a multiple of 16", who, (long long)a.ldw);
    RWKVQ_REQUIRE(a.ldo >= a.N, RWKVQ_E_SHAPE, "%s: ldo=%lld < N", who, (long long)a.ldo);
    RWKVQ_REQUIRE(a.div_mode == RWKVQ_DIV_IEEE || a.div_mode == RWKVQ_DIV_FULL, RWKVQ_E_BADARG, "%s: div_mode %d", who, a.div_mode);
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, x_dtype);
    RWKVQ_REQUIRE(a.M <= 32, RWKVQ_E_SHAPE, "%s: M=%d > 32 (use the GEMM entry points)", who, a.M);
    RWKVQ_REQUIRE(a.ldx >= a.K && a.ldx % 8 == 0, RWKVQ_E_ALIGN, "%s: ldx=%lld must be >= K and a multiple of 8", who, (long long)a.ldx);
    for (int i = 0; i < a.nmat; ++i) {
        RWKVQ_REQUIRE(a.w[i] && a.ws[i] && a.out[i] && a.x[i], RWKVQ_E_BADARG, "%s: null pointer (matrix %d)", who, i);
        RWKVQ_REQUIRE(aligned16(a.w[i]) && aligned16(a.x[i]), RWKVQ_E_ALIGN, "%s: weight / activation pointer not 16-byte aligned", who);
    }
    if (a.M == 0 || a.N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(a.K > 0, RWKVQ_E_SHAPE, "%s: K=0", who);
    const int MT = a.M <= 16 ? 1 : 2;
    // shared-memory row pitch of the activation tile: int8 codes (1 B) or f16 values of the e4m3 codes (2 B);
    // the odd 64 / 16 bytes keep the fragment loads of different rows on different banks
    a.pitch = (QT == QT_FP8 && fp8_wide()) ? ((2 * a.K + 127) / 128) * 128 + 16 : ((a.K + 127) / 128) * 128 + 64;
    (void)MT;
    const int64_t tiles = (int64_t)a.nmat * ((a.N + 7) / 8);
    RWKVQ_REQUIRE(tiles < (int64_t(1) << 30), RWKVQ_E_SHAPE, "%s: N too large", who);
    return x_dtype == RWKVQ_F16 ? dispatch_mt<QT, RWKVQ_F16>(a, tiles, st) : dispatch_mt<QT, RWKVQ_BF16>(a, tiles, st);
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

}  // extern "C"
