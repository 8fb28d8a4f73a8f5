// NVFP4 (W4A4, block-scaled): e2m1 values, one e4m3 scale per 16 consecutive K, one fp32 scale per tensor.
//
//   activation quantization (per call):  pts = amax / 2688;  block scale = e4m3(clamp(max|x|_16 * 448 / amax, 2^-6, 448));
//                                        code = e2m1_rn(x * (1/pts) / block_scale)
//   projection:                          out = fp16( (sum_k codeA*bsA * codeB*bsB) * ptsA * ptsW )
//
// The reference repository holds no NVFP4 code any more (only its reports describe the format:
// iterations/phase1_nvfp4_exploration/reports/03_fused_kernel_en.md:22-34, 07_quantization_toolchain_v2_en.md:18-25,
// iterations/phase3_x5_residual_scheme/reports/11_fused_gemm_ops_en.md:20-26), so these kernels follow that text.
//
// Decode GEMV (M <= 16): code * block scale is an exact fp16 value (6 significant bits, magnitude 2^-7 .. 2688), so
// both operands are dequantized to fp16 -- the activations once per CTA into shared memory, the weights in registers
// from the streamed 16-byte loads (cvt.f16x2.e2m1x2 + one HMUL2 per pair) -- and multiplied with mma.sync.m16n8k16
// with fp32 accumulation: every product is exact.  Same work split as the INT4 GEMV: 8 weight rows per CTA, the 8
// warps on alternating 128-k units, register ring of loads across row tiles, fixed-order reduction.
#include <cooperative_groups.h>
#include <atomic>
#include <cstdlib>

#include "w8a8.cuh"

namespace rwkvq {

// ---------------------------------------------------------------------------------------- activation quantization
// one thread per 16-block
template <int DT>
__global__ void __launch_bounds__(256) actq_nvfp4_kernel(const void* x, uint8_t* codes, uint8_t* bscale, float* pts_out,
                                                         const float* amax_p, int64_t M, int64_t K, int64_t ldx, int64_t ldc,
                                                         int64_t lds) {
    const int64_t nblk = K >> 4;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const float amax = fmaxf(*amax_p, 1e-12f);
    const float pts = __fdiv_rn(amax, 2688.f);
    if (i == 0) *pts_out = pts;
    if (i >= M * nblk) return;
    const int64_t r = i / nblk, b = i - r * nblk;
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(x) + (r * ldx + b * 16) * 2);
    const uint4 v0 = p[0], v1 = p[1];
    const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float f[16], m = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        const float2 t = cvt2<DT>(w[q]);
        f[2 * q] = t.x;
        f[2 * q + 1] = t.y;
        m = fmaxf(m, fmaxf(fabsf(t.x), fabsf(t.y)));
    }
    const float sb = fminf(fmaxf(m * __fdiv_rn(448.f, amax), 0.015625f), 448.f);
    const uint32_t sc = e4m3x2(sb, 0.f) & 0xffu;
    const float bs = e4m3_to_float(sc);
    const float inv_pts = __fdiv_rn(1.f, pts);
    uint32_t out[2] = {0u, 0u};
#pragma unroll
    for (int q = 0; q < 8; ++q)
        out[q >> 2] |= e2m1x2(__fdiv_rn(f[2 * q] * inv_pts, bs), __fdiv_rn(f[2 * q + 1] * inv_pts, bs)) << (8 * (q & 3));
    *reinterpret_cast<uint2*>(codes + r * ldc + b * 8) = make_uint2(out[0], out[1]);
    bscale[r * lds + b] = (uint8_t)sc;
}

// ---------------------------------------------------------------------------------------- decode GEMV
struct Nf4Args {
    const uint8_t* a_codes;    // [M, lda] packed activation codes
    const uint8_t* a_bs;       // [M, ldas] e4m3 block scales
    const float* a_pts;        // [1]
    const uint8_t* w;          // [N, ldw] packed weight codes
    const uint8_t* w_bs;       // [N, ldws] e4m3 block scales
    const float* w_ts;         // [1]
    __half* out;               // [M, ldo]
    int64_t lda, ldas, ldw, ldws, ldo;
    int M, N, K, pitch;
};

struct Nf4Slot {
    uint4 w;
    uint32_t sc;               // two e4m3 block scales (this lane's 32 codes = blocks 2t, 2t+1 of the unit)
};

template <int D>
__global__ void __launch_bounds__(kThr, 2) gemv_nvfp4_kernel(const Nf4Args a) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem);                       // [kWarps][4][32]
    uint8_t* xs = smem + kWarps * 4 * 32 * 4;                          // [M][pitch] fp16 values code * block scale
    griddep_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int units = a.K >> 7;
    const int ntile = (a.N + 7) >> 3;
    const int tb = (int)((int64_t)ntile * blockIdx.x / gridDim.x), te = (int)((int64_t)ntile * (blockIdx.x + 1) / gridDim.x);
    const int upw = (units + kWarps - 1) / kWarps, nchunks = (upw + D - 1) / D;

    auto fetch = [&](int tile, int c, int j) -> Nf4Slot {
        Nf4Slot s;
        s.w = make_uint4(0, 0, 0, 0);
        s.sc = 0;
        const int u = warp + (c * D + j) * kWarps;
        if (tile >= te || u >= units) return s;
        const int64_t row = min((tile << 3) + g, a.N - 1);
        s.w = ldg_stream(a.w + row * a.ldw + (u << 6) + 16 * t);
        s.sc = __ldg(reinterpret_cast<const unsigned short*>(a.w_bs + row * a.ldws + (u << 3) + 2 * t));
        return s;
    };
    Nf4Slot ring[D];
#pragma unroll
    for (int j = 0; j < D; ++j) ring[j] = fetch(tb, 0, j);

    griddep_wait();
    // prologue: activations dequantized to fp16 (exact), one thread per 16-block
    for (int i = threadIdx.x; i < a.M * (a.K >> 4); i += kThr) {
        const int r = i / (a.K >> 4), b = i - r * (a.K >> 4);
        const uint2 cw = *reinterpret_cast<const uint2*>(a.a_codes + (int64_t)r * a.lda + b * 8);
        const uint32_t s2 = e4m3x2_to_f16x2(a.a_bs[(int64_t)r * a.ldas + b]);
        const uint32_t ss = __byte_perm(s2, s2, 0x1010);               // (bs, bs)
        uint32_t h[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const uint32_t pair = e2m1x2_to_f16x2(((q < 4 ? cw.x : cw.y) >> (8 * (q & 3))) & 0xffu);
            const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&pair), *reinterpret_cast<const __half2*>(&ss));
            h[q] = *reinterpret_cast<const uint32_t*>(&v);
        }
        uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)r * a.pitch + (size_t)b * 32);
        dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
        dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
    }
    __syncthreads();
    const float out_scale = a.a_pts[0] * a.w_ts[0];

    for (int tile = tb; tile < te; ++tile) {
        const int n0 = tile << 3;
        float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};
        for (int ch = 0; ch < nchunks; ++ch) {
            const bool last = ch + 1 == nchunks;
#pragma unroll
            for (int j = 0; j < D; ++j) {
                const Nf4Slot sl = ring[j];
                ring[j] = fetch(last ? tile + 1 : tile, last ? 0 : ch + 1, j);
                const int u = warp + (ch * D + j) * kWarps;
                if (u < units) {
                    const uint32_t s2 = e4m3x2_to_f16x2(sl.sc);        // (bs of block 2t, bs of block 2t+1)
                    const uint32_t sA = __byte_perm(s2, s2, 0x1010), sB = __byte_perm(s2, s2, 0x3232);
                    const uint32_t wd[4] = {sl.w.x, sl.w.y, sl.w.z, sl.w.w};
                    const size_t koff = ((size_t)u << 8) + (size_t)t * 64;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {                      // word i = 8 codes; words 0,1 = first block, 2,3 = second
                        uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0;
                        if (g < a.M) a0 = *reinterpret_cast<const uint4*>(xs + (size_t)g * a.pitch + koff + i * 16);
                        if (g + 8 < a.M) a1 = *reinterpret_cast<const uint4*>(xs + (size_t)(g + 8) * a.pitch + koff + i * 16);
                        const uint32_t sc = i < 2 ? sA : sB;
                        uint32_t b[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint32_t pair = e2m1x2_to_f16x2((wd[i] >> (8 * q)) & 0xffu);
                            const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&pair), *reinterpret_cast<const __half2*>(&sc));
                            b[q] = *reinterpret_cast<const uint32_t*>(&v);
                        }
                        mma_f16(c, a0.x, a1.x, a0.y, a1.y, b[0], b[1]);
                        mma_f16(c2, a0.z, a1.z, a0.w, a1.w, b[2], b[3]);
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) red[(warp * 4 + j) * 32 + lane] = c[j] + c2[j];
        __syncthreads();
        if (threadIdx.x < 128) {
            const int j = threadIdx.x >> 5, l = threadIdx.x & 31;
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += red[(w * 4 + j) * 32 + l];
            const int m = (l >> 2) + ((j & 2) ? 8 : 0), n = n0 + 2 * (l & 3) + (j & 1);
            if (m < a.M && n < a.N) a.out[(int64_t)m * a.ldo + n] = __float2half_rn(s * out_scale);
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------- fused decode GEMV
// One launch per projection for M <= 16 (K a multiple of 512): the activation quantization of rwkvq_actq_nvfp4 runs in
// the prologue (amax, tensor scale, block scales, codes -- and straight on to the dequantized fp16 values
// code * block scale, which is all the MMA needs), and the weight stream is organised like the INT4 group kernel:
// the WEIGHTS are the 16-row A operand of m16n8k16 (rows g and g+8 of lane (g, t)), up to 8 tokens the B operand;
// a warp owns 16 weight rows over a contiguous K range; a unit is 128 k (64 bytes per row, 8 scale blocks); a chunk is
// 4 units plus the 32 scale bytes of each of the 16 rows, all copied with cp.async into a per-warp ring.  A lane's
// 16 bytes of a row are 32 codes = two scale blocks: 16 cvt.f16x2.e2m1x2 and 16 HMUL2 per row make the A registers
// of 8 MMAs.  Activations of a unit are stored [word][lane] (see the INT4 kernel) so that the B-fragment loads have no
// bank conflicts.  8/R warps share a row tile and add their K parts in warp order.
constexpr int kNfD = 4;
constexpr int kNfStage = kNfD * 1024 + 512;       // bytes per warp and stage: codes of 4 units + scales of 16 rows

__device__ __forceinline__ void nf_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void nf_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct NfFusedArgs {
    const void* x;             // [M, ldx] fp16 / bf16
    const uint8_t* w;          // [N, ldw] packed codes
    const uint8_t* w_bs;       // [N, ldws] e4m3 block scales
    const float* w_ts;         // [1]
    __half* out;               // [M, ldo]
    int64_t ldx, ldw, ldws, ldo;
    int M, N, K, pitch;
    int lgR, tq, trem;
    int* status;                 // the library's per-device status word
    unsigned long long wait_ns;  // wall-time limit of the bounded waits
};

template <int DT, int NT, int S>
__global__ void __launch_bounds__(kThr, 2) gemv_nvfp4_fused_kernel(const NfFusedArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: red[kWarps][NT*4][32] floats | ring[kWarps][S][kNfStage] | sh[8] floats + barrier (128 B) | xs[M][pitch]
    float* red = reinterpret_cast<float*>(smem);
    uint8_t* ring = smem + kWarps * NT * 4 * 32 * 4;
    float* sh = reinterpret_cast<float*>(ring + (size_t)kWarps * S * kNfStage);
    uint64_t* xbar = reinterpret_cast<uint64_t*>(sh + 16);
    uint8_t* xs = reinterpret_cast<uint8_t*>(sh) + 128;

    griddep_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int units = a.K >> 7;
    const int cb = blockIdx.x;
    const int tb = cb * a.tq + min(cb, a.trem), te = tb + a.tq + (cb < a.trem ? 1 : 0);   // this CTA's 16-row tiles
    const int lgR = a.lgR, R = 1 << lgR, lgKS = 3 - lgR, KS = 1 << lgKS;
    const int slot = warp >> lgKS, ks = warp & (KS - 1);
    const int rounds = (te - tb + R - 1) >> lgR;
    const int upw = (((units + KS - 1) >> lgKS) + 3) & ~3;           // units per warp and tile, whole chunks
    const int ub = ks * upw, ue = min(ub + upw, units);
    const int nch = max(ue - ub, 0) >> 2;
    const int my_rounds = (nch > 0 && te - tb > slot) ? ((te - tb - slot + R - 1) >> lgR) : 0;
    uint8_t* my_ring = ring + (size_t)warp * S * kNfStage;
    const uint32_t my_ring_s = (uint32_t)__cvta_generic_to_shared(my_ring);

    // producer: per chunk 8 code copies per lane and one 16-byte piece of the scales (t = 0, 1: row g; t = 2, 3: row g+8)
    int p_round = 0, p_ch = 0, p_stage = 0;
    const uint8_t *p_w0 = a.w, *p_w1 = a.w, *p_sc = a.w_bs;
    auto set_rows = [&](int round) {
        const int n0 = (tb + round * R + slot) << 4;
        const int r0 = min(n0 + g, a.N - 1), r1 = min(n0 + g + 8, a.N - 1);
        p_w0 = a.w + (int64_t)r0 * a.ldw + ub * 64 + 16 * t;
        p_w1 = a.w + (int64_t)r1 * a.ldw + ub * 64 + 16 * t;
        p_sc = a.w_bs + (int64_t)((t & 2) ? r1 : r0) * a.ldws + ub * 8 + 16 * (t & 1);
    };
    if (my_rounds > 0) set_rows(0);
    auto issue = [&]() {
        if (p_round < my_rounds) {
            const uint32_t dst = my_ring_s + p_stage * kNfStage;
#pragma unroll
            for (int j = 0; j < kNfD; ++j) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + j * 1024 + lane * 16), "l"(p_w0 + j * 64) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + j * 1024 + 512 + lane * 16), "l"(p_w1 + j * 64) : "memory");
            }
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + kNfD * 1024 + (((t >> 1) * 8 + g) * 32) + (t & 1) * 16), "l"(p_sc) : "memory");
            p_w0 += kNfD * 64;
            p_w1 += kNfD * 64;
            p_sc += kNfD * 8;
            if (++p_ch == nch) {
                p_ch = 0;
                if (++p_round < my_rounds) set_rows(p_round);
            }
        }
        nf_cp_async_commit();
        if (++p_stage == S) p_stage = 0;
    };
#pragma unroll
    for (int i = 0; i < S - 1; ++i) issue();

    // this lane's token rows of the activation tile (tokens beyond M read row M-1: columns that are never stored)
    const uint8_t* xb0[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) xb0[i] = xs + min(i * 8 + g, a.M - 1) * a.pitch + ub * 256 + t * 16;
    const float w_ts = a.w_ts[0];

    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(xbar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    griddep_wait();

    // ---- prologue: activation quantization, fused.  Raw rows by bulk copy into the tile; amax; then every thread turns
    // 16-blocks into dequantized fp16 values in place.
    float pts;
    {
        if (threadIdx.x == 0) {
            const uint32_t b = (uint32_t)__cvta_generic_to_shared(xbar);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"((uint32_t)(a.M * a.K * 2)) : "memory");
#pragma unroll 1
            for (int r = 0; r < a.M; ++r)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"((uint32_t)__cvta_generic_to_shared(xs + (size_t)r * a.pitch)),
                               "l"(reinterpret_cast<const char*>(a.x) + (int64_t)r * a.ldx * 2), "r"((uint32_t)(a.K * 2)), "r"(b) : "memory");
        }
        if (!w8_staged_or_report(xbar, a.status, a.wait_ns)) {     // reported: drain the weight ring and stop
            nf_cp_async_wait<0>();
            return;
        }
        const int kv = a.K >> 3;
        float m = 0.f;
#pragma unroll 1
        for (int r = 0; r < a.M; ++r) {
            const char* src = reinterpret_cast<const char*>(xs + (size_t)r * a.pitch);
#pragma unroll 1
            for (int i = threadIdx.x; i < kv; i += kThr) m = fmaxf(m, packed_absmax8<DT>(*reinterpret_cast<const uint4*>(src + (size_t)i * 16)));
        }
        const float amax = fmaxf(cta_max(m, sh), 1e-12f);
        pts = __fdiv_rn(amax, 2688.f);
        const float inv_pts = __fdiv_rn(1.f, pts), k448 = __fdiv_rn(448.f, amax);
        const int nb = a.K >> 4;                                   // 16-blocks per row (a multiple of 32)
#pragma unroll 1
        for (int r = 0; r < a.M; ++r) {
            uint8_t* row = xs + (size_t)r * a.pitch;
            const char* src = reinterpret_cast<const char*>(row);
#pragma unroll 1
            for (int b = threadIdx.x; b < nb; b += kThr) {
                const uint4 v0 = *reinterpret_cast<const uint4*>(src + (size_t)b * 32), v1 = *reinterpret_cast<const uint4*>(src + (size_t)b * 32 + 16);
                const uint32_t wv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                float f[16], bm = 0.f;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const float2 p = cvt2<DT>(wv[q]);
                    f[2 * q] = p.x;
                    f[2 * q + 1] = p.y;
                    bm = fmaxf(bm, fmaxf(fabsf(p.x), fabsf(p.y)));
                }
                const float sb = fminf(fmaxf(bm * k448, 0.015625f), 448.f);
                const uint32_t sc = e4m3x2(sb, 0.f) & 0xffu;
                const uint32_t s2 = e4m3x2_to_f16x2(sc);
                const uint32_t ss = __byte_perm(s2, s2, 0x1010);           // (bs, bs) as fp16
                const float bs = __half2float(__ushort_as_half((unsigned short)(s2 & 0xffffu)));
                uint32_t h[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const uint32_t pair = e2m1x2_to_f16x2(e2m1x2(__fdiv_rn(f[2 * q] * inv_pts, bs), __fdiv_rn(f[2 * q + 1] * inv_pts, bs)));
                    const __half2 d = __hmul2(*reinterpret_cast<const __half2*>(&pair), *reinterpret_cast<const __half2*>(&ss));
                    h[q] = *reinterpret_cast<const uint32_t*>(&d);
                }
                // vectors 2b, 2b+1 of the row; inside a unit (16 vectors) vector 4t+i goes to place 4i+t.  In place: the
                // eight blocks of a unit sit in eight neighbouring lanes, all of which have read before any writes.
                __syncwarp();
                const int v = 2 * b, u16 = v & ~15, tt = (v >> 2) & 3, i0 = v & 3;
                *reinterpret_cast<uint4*>(row + (size_t)(u16 | (i0 << 2) | tt) * 16) = make_uint4(h[0], h[1], h[2], h[3]);
                *reinterpret_cast<uint4*>(row + (size_t)(u16 | ((i0 + 1) << 2) | tt) * 16) = make_uint4(h[4], h[5], h[6], h[7]);
            }
        }
        __syncthreads();
    }
    const float out_scale = pts * w_ts;

    int stage = 0;
    for (int r = 0; r < rounds; ++r) {
        float c[NT][4], c2[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) c[i][j] = c2[i][j] = 0.f;
        if (r < my_rounds) {
            const uint8_t* xb[NT];
#pragma unroll
            for (int i = 0; i < NT; ++i) xb[i] = xb0[i];
            for (int ch = 0; ch < nch; ++ch) {
                issue();
                nf_cp_async_wait<S - 1>();
                __syncwarp();                              // the scale bytes are read across lanes
                const uint8_t* st = my_ring + stage * kNfStage;
#pragma unroll
                for (int j = 0; j < kNfD; ++j) {
                    const uint4 wg = *reinterpret_cast<const uint4*>(st + j * 1024 + lane * 16);
                    const uint4 wh = *reinterpret_cast<const uint4*>(st + j * 1024 + 512 + lane * 16);
                    // this lane's two scale blocks of the unit, rows g and g+8, as fp16 pairs (s, s)
                    const uint32_t sg = e4m3x2_to_f16x2(*reinterpret_cast<const unsigned short*>(st + kNfD * 1024 + g * 32 + j * 8 + 2 * t));
                    const uint32_t shh = e4m3x2_to_f16x2(*reinterpret_cast<const unsigned short*>(st + kNfD * 1024 + (8 + g) * 32 + j * 8 + 2 * t));
                    const uint32_t sgv[2] = {__byte_perm(sg, sg, 0x1010), __byte_perm(sg, sg, 0x3232)};
                    const uint32_t shv[2] = {__byte_perm(shh, shh, 0x1010), __byte_perm(shh, shh, 0x3232)};
                    const uint32_t wgw[4] = {wg.x, wg.y, wg.z, wg.w}, whw[4] = {wh.x, wh.y, wh.z, wh.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {          // word q: codes 8q .. 8q+7 of the lane's 32; block q / 2
                        uint32_t ag[4], ah[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t pg = e2m1x2_to_f16x2((wgw[q] >> (8 * e)) & 0xffu), ph = e2m1x2_to_f16x2((whw[q] >> (8 * e)) & 0xffu);
                            const __half2 dg = __hmul2(*reinterpret_cast<const __half2*>(&pg), *reinterpret_cast<const __half2*>(&sgv[q >> 1]));
                            const __half2 dh = __hmul2(*reinterpret_cast<const __half2*>(&ph), *reinterpret_cast<const __half2*>(&shv[q >> 1]));
                            ag[e] = *reinterpret_cast<const uint32_t*>(&dg);
                            ah[e] = *reinterpret_cast<const uint32_t*>(&dh);
                        }
#pragma unroll
                        for (int i = 0; i < NT; ++i) {
                            const uint4 bx = *reinterpret_cast<const uint4*>(xb[i] + j * 256 + q * 64);
                            mma_f16(c[i], ag[0], ah[0], ag[1], ah[1], bx.x, bx.y);
                            mma_f16(c2[i], ag[2], ah[2], ag[3], ah[3], bx.z, bx.w);
                        }
                    }
                }
                __syncwarp();                              // all lanes have read this stage before it is refilled
#pragma unroll
                for (int i = 0; i < NT; ++i) xb[i] += kNfD * 256;
                if (++stage == S) stage = 0;
            }
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) c[i][j] += c2[i][j];
        }
        const int tile = tb + r * R + slot;
        bool store = tile < te;
        if (KS > 1) {
            if (r > 0) __syncthreads();
            if (ks > 0) {
#pragma unroll
                for (int i = 0; i < NT; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) red[((warp * NT + i) * 4 + j) * 32 + lane] = c[i][j];
            }
            __syncthreads();
            store = store && ks == 0;
            if (store) {
                for (int kk = 1; kk < KS; ++kk)
#pragma unroll
                    for (int i = 0; i < NT; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) c[i][j] += red[(((warp + kk) * NT + i) * 4 + j) * 32 + lane];
            }
        }
        if (store) {
            const int n0 = tile << 4;
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int m = i * 8 + 2 * t + (j & 1), n = n0 + g + ((j & 2) ? 8 : 0);
                    if (m < a.M && n < a.N) a.out[(int64_t)m * a.ldo + n] = __float2half_rn(c[i][j] * out_scale);
                }
        }
    }
    nf_cp_async_wait<0>();
}

static size_t nf_fused_smem(int NT, int S, int M, int K) {
    return (size_t)kWarps * NT * 4 * 32 * 4 + (size_t)kWarps * S * kNfStage + 128 + (size_t)M * (2 * K + 16);
}

template <int DT, int NT, int S>
static int32_t launch_nf_fused(NfFusedArgs a, size_t smem, cudaStream_t st) {
    auto kern = gemv_nvfp4_fused_kernel<DT, NT, S>;
    int per_sm = 0;
    const int32_t rc = kernel_plan(reinterpret_cast<const void*>(kern), kThr, smem, 224 * 1024, &per_sm, "gemv_nvfp4_fused");
    if (rc != RWKVQ_OK) return rc;
    cudaError_t e;
    a.status = device_status_ptr();
    a.wait_ns = wait_limit_ns();
    const int64_t tiles = (a.N + 15) / 16;
    const int grid = (int)std::min<int64_t>(tiles, (int64_t)sm_count() * std::min(per_sm, 2));
    a.tq = (int)(tiles / grid);
    a.trem = (int)(tiles % grid);
    const int tpc = (int)((tiles + grid - 1) / grid);
    a.lgR = 0;
    while ((1 << a.lgR) < kWarps && (1 << a.lgR) < tpc) ++a.lgR;
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
    e = cudaLaunchKernelEx(&cfg, kern, a);
    if (e != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "gemv_nvfp4_fused: %s", cudaGetErrorString(e));
    }
    return check_launch("gemv_nvfp4_fused");
}

template <int DT, int NT>
static int32_t dispatch_nf_fused(const NfFusedArgs& a, cudaStream_t st) {
    const size_t s2 = nf_fused_smem(NT, 2, a.M, a.K), s4 = nf_fused_smem(NT, 4, a.M, a.K);
    if (s2 <= 110 * 1024) return launch_nf_fused<DT, NT, 2>(a, s2, st);
    if (s4 <= 224 * 1024) return launch_nf_fused<DT, NT, 4>(a, s4, st);
    RWKVQ_REQUIRE(s2 <= 224 * 1024, RWKVQ_E_SHAPE, "gemv_nvfp4_fused: M*K = %d*%d does not fit shared memory; call with fewer rows", a.M, a.K);
    return launch_nf_fused<DT, NT, 2>(a, s2, st);
}

// ---------------------------------------------------------------------------------------- fused activation quantization
// rwkvq_actq_nvfp4 in ONE cooperative launch (the structure of the fused FP8 quantizer): per-CTA partial maxima, a
// grid-wide rendezvous through a token that is unique per launch, then codes and block scales.  A 16-block is two
// 8-element vectors held by two neighbouring threads, which exchange their maxima with one shuffle.  The block scales
// are written row-major and / or in the blocked order the tensor-core GEMM reads (either pointer may be null).
constexpr int kNfQThreads = 512;

constexpr int kNfQMaxCtas = 512;       // slots[512] | flags[512] | epoch word

struct NfQArgs {
    const void* x;
    uint8_t* codes;
    uint8_t* bs_rows;        // [M, lds] or null
    uint8_t* bs_blocked;     // blocked order or null
    float* pts;
    float* slots;
    uint32_t* flags;
    int* status;
    int64_t ldx, ldc, lds;
    int M, K;
    unsigned long long wait_ns;
};

template <int DT>
__global__ void __launch_bounds__(kNfQThreads, 2) actq_nvfp4_fused_kernel(const NfQArgs a) {
    __shared__ float sh[kNfQThreads / 32];
    __shared__ float s_amax;
    __shared__ int s_fail;
    __shared__ uint32_t s_token;
    const int kv = a.K >> 3, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x;
    // The rendezvous value is the scratch's epoch + 1, read on the device (see actq_fp8_fused_kernel): a captured launch
    // can be replayed, because nothing about it is fixed on the host.
    if (threadIdx.x == 0) {
        s_token = ld_acquire_u32(a.flags + kNfQMaxCtas) + 1u;
        s_fail = 0;
    }
    // ---- pass 1: partial maximum of this CTA's rows, four rows per step
    float m = 0.f;
    for (int r = blockIdx.x; r < a.M; r += 4 * G) {
        for (int i = threadIdx.x; i < kv; i += kNfQThreads) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int rj = min(r + j * G, a.M - 1);
                v[j] = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(a.x) + ((int64_t)rj * a.ldx + (int64_t)i * 8) * 2);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) m = fmaxf(m, packed_absmax8<DT>(v[j]));
        }
    }
    m = warp_max(m);
    if (lane == 0) sh[warp] = m;
    __syncthreads();
    const uint32_t token = s_token;
    if (threadIdx.x == 0) {
        float b = sh[0];
        for (int i = 1; i < kNfQThreads / 32; ++i) b = fmaxf(b, sh[i]);
        a.slots[blockIdx.x] = b;
        __threadfence();
        st_release_u32(a.flags + blockIdx.x, token);
    }
    // ---- rendezvous: thread t waits for CTA t's flag (bounded), then the maxima are combined
    float g = 0.f;
    if ((int)threadIdx.x < G) {
        if (wait_flag_eq(a.flags + threadIdx.x, token, a.wait_ns)) g = __ldcg(a.slots + threadIdx.x);
        else s_fail = 1;
    }
    g = warp_max(g);
    __syncthreads();
    if (lane == 0) sh[warp] = g;
    __syncthreads();
    if (threadIdx.x == 0) {
        float b = sh[0];
        for (int i = 1; i < kNfQThreads / 32; ++i) b = fmaxf(b, sh[i]);
        s_amax = b;
        if (s_fail && a.status) atomicExch(a.status, RWKVQ_E_TIMEOUT);
        if (blockIdx.x == 0 && !s_fail) st_release_u32(a.flags + kNfQMaxCtas, token);   // every CTA has read the old epoch
    }
    __syncthreads();
    if (s_fail) return;
    // ---- pass 2: block scales and codes (the second read of x hits L2)
    const float amax = fmaxf(s_amax, 1e-12f);
    const float pts = __fdiv_rn(amax, 2688.f);
    if (blockIdx.x == 0 && threadIdx.x == 0) *a.pts = pts;
    const float inv_pts = __fdiv_rn(1.f, pts), k448 = __fdiv_rn(448.f, amax);
    const int64_t k64 = a.K >> 6;
    for (int r = blockIdx.x; r < a.M; r += G) {
        for (int i0 = 0; i0 < kv; i0 += kNfQThreads) {           // whole warps: kv is even, a block is lanes 2j, 2j+1
            const int i = i0 + threadIdx.x;
            const bool on = i < kv;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (on) v = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(a.x) + ((int64_t)r * a.ldx + (int64_t)i * 8) * 2);
            const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
            float f[8], bm = 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 p = cvt2<DT>(wv[q]);
                f[2 * q] = p.x;
                f[2 * q + 1] = p.y;
                bm = fmaxf(bm, fmaxf(fabsf(p.x), fabsf(p.y)));
            }
            bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
            const float sb = fminf(fmaxf(bm * k448, 0.015625f), 448.f);
            const uint32_t sc = e4m3x2(sb, 0.f) & 0xffu;
            const float bs = e4m3_to_float(sc);
            uint32_t out = 0;
#pragma unroll
            for (int q = 0; q < 4; ++q) out |= e2m1x2(__fdiv_rn(f[2 * q] * inv_pts, bs), __fdiv_rn(f[2 * q + 1] * inv_pts, bs)) << (8 * q);
            if (on) {
                *reinterpret_cast<uint32_t*>(a.codes + (int64_t)r * a.ldc + (int64_t)i * 4) = out;
                if ((i & 1) == 0) {
                    const int b = i >> 1;
                    if (a.bs_rows) a.bs_rows[(int64_t)r * a.lds + b] = (uint8_t)sc;
                    if (a.bs_blocked)
                        a.bs_blocked[((int64_t)(r >> 7) * k64 + (b >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (b & 3)] = (uint8_t)sc;
                }
            }
        }
    }
}

// Few tokens (the kernel takes up to 16384 vectors; the dispatcher gives it up to 8192: 4 rows of K = 16384, 16 of
// K = 4096): ONE plain launch of a CLUSTER of 1 to 8 CTAs
// of 256 threads, like the small FP8 quantizer: every thread keeps up to 8 vectors in registers between the abs-max
// and the codes (one read of the activations, all loads in flight together), the CTAs exchange their maxima through
// distributed shared memory and one cluster barrier.  No scratch, no second launch for the projection behind it to
// wait for.  CTAs of 256 threads (16 K registers) become resident next to the CTAs of the projection in front; with
// 1024 threads (the whole register file) the cluster had to wait for free SMs and the call was slower than the two
// chained launches below.  Same arithmetic as the other forms: same bits.
constexpr int kNfSmallThreads = 256;
constexpr int kNfSmallKeep = 8;

template <int DT>
__global__ void __launch_bounds__(kNfSmallThreads, 1) actq_nvfp4_small_kernel(const NfQArgs a) {
    __shared__ float sh[kNfSmallThreads / 32];
    __shared__ float s_part[8];           // maxima of the cluster's CTAs (each CTA writes its slot in every CTA)
    __shared__ float s_amax;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    cooperative_groups::cluster_group cl = cooperative_groups::this_cluster();
    const int C = (int)cl.num_blocks(), cr = (int)cl.block_rank();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const char* x = reinterpret_cast<const char*>(a.x);
    const int kv = a.K >> 3, nvec = a.M * kv;
    const uint32_t inv_kv = 0xFFFFFFFFu / (uint32_t)kv + 1u;          // row of a flat vector index without a division
    const int64_t k64 = a.K >> 6;
    asm volatile("griddepcontrol.wait;" ::: "memory");                // the activations may come from the previous kernel
    // the cluster's threads take the vectors round-robin; kv and the step are even, so the two vectors of a 16-block
    // sit in neighbouring lanes at the same j
    const int first = cr * kNfSmallThreads + (int)threadIdx.x, step = C * kNfSmallThreads;
    uint4 v[kNfSmallKeep];
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < kNfSmallKeep; ++j) {
        const int idx = first + j * step;
        v[j] = make_uint4(0, 0, 0, 0);
        if (idx < nvec) {
            const int r = (int)__umulhi((uint32_t)idx, inv_kv), c = idx - r * kv;
            v[j] = *reinterpret_cast<const uint4*>(x + ((int64_t)r * a.ldx + (int64_t)c * 8) * 2);
        }
    }
#pragma unroll
    for (int j = 0; j < kNfSmallKeep; ++j) m = fmaxf(m, packed_absmax8<DT>(v[j]));
    m = warp_max(m);
    if (lane == 0) sh[warp] = m;
    __syncthreads();
    if (warp == 0) {
        const float b = warp_max(lane < kNfSmallThreads / 32 ? sh[lane] : 0.f);
        if (lane < C) *cl.map_shared_rank(&s_part[cr], lane) = b;      // this CTA's maximum into slot cr of CTA `lane`
    }
    cl.sync();                                                          // all slots written (and visible) in every CTA
    if (threadIdx.x == 0) {
        float b = s_part[0];
        for (int i = 1; i < C; ++i) b = fmaxf(b, s_part[i]);
        s_amax = b;
    }
    __syncthreads();
    const float amax = fmaxf(s_amax, 1e-12f);
    const float pts = __fdiv_rn(amax, 2688.f);
    if (cr == 0 && threadIdx.x == 0) *a.pts = pts;
    const float inv_pts = __fdiv_rn(1.f, pts), k448 = __fdiv_rn(448.f, amax);
#pragma unroll
    for (int j = 0; j < kNfSmallKeep; ++j) {
        const int idx = first + j * step;
        if (j * step >= nvec) break;                                   // uniform over the cluster
        const uint32_t wv[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
        float f[8], bm = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 p = cvt2<DT>(wv[q]);
            f[2 * q] = p.x;
            f[2 * q + 1] = p.y;
            bm = fmaxf(bm, fmaxf(fabsf(p.x), fabsf(p.y)));
        }
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
        const float sb = fminf(fmaxf(bm * k448, 0.015625f), 448.f);
        const uint32_t sc = e4m3x2(sb, 0.f) & 0xffu;
        const float bs = e4m3_to_float(sc);
        uint32_t out = 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) out |= e2m1x2(__fdiv_rn(f[2 * q] * inv_pts, bs), __fdiv_rn(f[2 * q + 1] * inv_pts, bs)) << (8 * q);
        if (idx < nvec) {
            const int r = (int)__umulhi((uint32_t)idx, inv_kv), i = idx - r * kv;
            *reinterpret_cast<uint32_t*>(a.codes + (int64_t)r * a.ldc + (int64_t)i * 4) = out;
            if ((i & 1) == 0) {
                const int b = i >> 1;
                if (a.bs_rows) a.bs_rows[(int64_t)r * a.lds + b] = (uint8_t)sc;
                if (a.bs_blocked)
                    a.bs_blocked[((int64_t)(r >> 7) * k64 + (b >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (b & 3)] = (uint8_t)sc;
            }
        }
    }
}

// The same quantization as TWO plain launches chained by programmatic dependent launch, for blocks of up to 2^19
// vectors (few tokens): a cooperative launch costs about 6 us more than a plain one and gives a 16-row block 16 CTAs;
// here the abs-max pass and the code pass each spread the block over two CTAs per SM.  The maximum travels through a
// scratch word (atomic max of the float's bits: the values are non-negative); the last CTA of the code pass clears
// it, so the words are zero again before the next launch on the stream can reach them and a captured graph replays.
// Words: flags[kNfQMaxCtas + 4] = maximum, [+ 7] = CTAs done (the FP8 two-launch quantizer uses the same words of the
// same scratch in the same way).  Same arithmetic as the cooperative kernel: same bits.
constexpr int kNfTwoThreads = 256;
constexpr int64_t kNfTwoMaxVectors = 1 << 19;

// grid rows * cpr: CTA b takes every cpr-th group of kNfTwoThreads vectors of row b / cpr and of every
// (gridDim.x / cpr)-th row after it
template <int DT>
__global__ void __launch_bounds__(kNfTwoThreads) actq_nvfp4_two_amax_kernel(const NfQArgs a, int cpr) {
    __shared__ float sh[kNfTwoThreads / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int kv = a.K >> 3, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = (int)blockIdx.x % cpr, rstep = (int)gridDim.x / cpr, cstep = cpr * kNfTwoThreads;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float m = 0.f;
    for (int r = (int)blockIdx.x / cpr; r < a.M; r += rstep) {
        const char* row = reinterpret_cast<const char*>(a.x) + (int64_t)r * a.ldx * 2;
        for (int c0 = seg * kNfTwoThreads + (int)threadIdx.x; c0 < kv; c0 += 4 * cstep) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c0 + j * cstep < kv) v[j] = *reinterpret_cast<const uint4*>(row + (int64_t)(c0 + j * cstep) * 16);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c0 + j * cstep < kv) m = fmaxf(m, packed_absmax8<DT>(v[j]));
        }
    }
    m = warp_max(m);
    if (lane == 0) sh[warp] = m;
    __syncthreads();
    if (warp == 0) {
        m = warp_max(lane < kNfTwoThreads / 32 ? sh[lane] : 0.f);
        if (lane == 0 && m > 0.f) atomicMax(reinterpret_cast<int*>(a.flags) + kNfQMaxCtas + 4, __float_as_int(m));
    }
}

template <int DT>
__global__ void __launch_bounds__(kNfTwoThreads) actq_nvfp4_two_codes_kernel(const NfQArgs a, int cpr) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int kv = a.K >> 3;
    const int seg = (int)blockIdx.x % cpr, rstep = (int)gridDim.x / cpr, cstep = cpr * kNfTwoThreads;
    int* two = reinterpret_cast<int*>(a.flags) + kNfQMaxCtas + 4;
    const int64_t k64 = a.K >> 6;
    asm volatile("griddepcontrol.wait;" ::: "memory");              // the abs-max pass is complete and visible
    const float amax = fmaxf(__int_as_float(__ldcg(two)), 1e-12f);
    const float pts = __fdiv_rn(amax, 2688.f);
    if (blockIdx.x == 0 && threadIdx.x == 0) *a.pts = pts;
    const float inv_pts = __fdiv_rn(1.f, pts), k448 = __fdiv_rn(448.f, amax);
    for (int r = (int)blockIdx.x / cpr; r < a.M; r += rstep) {
        const char* row = reinterpret_cast<const char*>(a.x) + (int64_t)r * a.ldx * 2;
        // whole warps walk together: kv is even and a 16-block is the vectors of lanes 2j and 2j + 1
        for (int base = seg * kNfTwoThreads; base < kv; base += 4 * cstep) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = base + j * cstep + (int)threadIdx.x;
                v[j] = i < kv ? *reinterpret_cast<const uint4*>(row + (int64_t)i * 16) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (base + j * cstep >= kv) continue;              // uniform over the CTA
                const int i = base + j * cstep + (int)threadIdx.x;
                const uint32_t wv[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
                float f[8], bm = 0.f;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 p = cvt2<DT>(wv[q]);
                    f[2 * q] = p.x;
                    f[2 * q + 1] = p.y;
                    bm = fmaxf(bm, fmaxf(fabsf(p.x), fabsf(p.y)));
                }
                bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
                const float sb = fminf(fmaxf(bm * k448, 0.015625f), 448.f);
                const uint32_t sc = e4m3x2(sb, 0.f) & 0xffu;
                const float bs = e4m3_to_float(sc);
                uint32_t out = 0;
#pragma unroll
                for (int q = 0; q < 4; ++q) out |= e2m1x2(__fdiv_rn(f[2 * q] * inv_pts, bs), __fdiv_rn(f[2 * q + 1] * inv_pts, bs)) << (8 * q);
                if (i < kv) {
                    *reinterpret_cast<uint32_t*>(a.codes + (int64_t)r * a.ldc + (int64_t)i * 4) = out;
                    if ((i & 1) == 0) {
                        const int b = i >> 1;
                        if (a.bs_rows) a.bs_rows[(int64_t)r * a.lds + b] = (uint8_t)sc;
                        if (a.bs_blocked)
                            a.bs_blocked[((int64_t)(r >> 7) * k64 + (b >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (b & 3)] = (uint8_t)sc;
                    }
                }
            }
        }
    }
    __syncthreads();                                    // every thread of this CTA has read the maximum
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(two + 3, 1) == (int)gridDim.x - 1) {
            two[0] = 0;
            __threadfence();
            two[3] = 0;
        }
    }
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

int32_t rwkvq_actq_nvfp4(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes, int64_t ldc,
                         uint8_t* block_scales, int64_t lds, float* pts, float* amax_scratch, void* stream) {
    const char* who = "actq_nvfp4";
    RWKVQ_REQUIRE(x && codes && block_scales && pts && amax_scratch, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, x_dtype);
    RWKVQ_REQUIRE(M >= 0 && K >= 0 && K % 16 == 0, RWKVQ_E_SHAPE, "%s: K=%lld must be a multiple of 16", who, (long long)K);
    RWKVQ_REQUIRE(aligned16(x) && ldx % 8 == 0 && ldx >= K, RWKVQ_E_ALIGN, "%s: activation rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(((uintptr_t)codes & 7) == 0 && ldc % 8 == 0 && ldc >= K / 2 && lds >= K / 16, RWKVQ_E_ALIGN, "%s: code rows must be 8-byte aligned", who);
    int32_t rc = rwkvq_prep_x(x, x_dtype, M, K, ldx, nullptr, nullptr, K, amax_scratch, RWKVQ_DIV_IEEE, stream);
    if (rc) return rc;
    const int64_t nthreads = std::max<int64_t>(1, M * (K / 16));
    const unsigned grid = (unsigned)((nthreads + 255) / 256);
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dtype == RWKVQ_F16) actq_nvfp4_kernel<RWKVQ_F16><<<grid, 256, 0, st>>>(x, codes, block_scales, pts, amax_scratch, M, K, ldx, ldc, lds);
    else actq_nvfp4_kernel<RWKVQ_BF16><<<grid, 256, 0, st>>>(x, codes, block_scales, pts, amax_scratch, M, K, ldx, ldc, lds);
    return check_launch(who);
}

int64_t rwkvq_gemv_nvfp4_smem_bytes(int64_t M, int64_t K) { return kWarps * 4 * 32 * 4 + M * (2 * K + 16); }

int32_t rwkvq_gemv_nvfp4(const uint8_t* a_codes, int64_t lda, const uint8_t* a_block_scales, int64_t ldas, const float* a_pts,
                         const uint8_t* w_codes, int64_t ldw, const uint8_t* w_block_scales, int64_t ldws, const float* w_tscale,
                         void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, void* stream) {
    const char* who = "gemv_nvfp4";
    RWKVQ_REQUIRE(a_codes && a_block_scales && a_pts && w_codes && w_block_scales && w_tscale && out_f16, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(M >= 0 && N >= 0 && K >= 0 && M <= 16, RWKVQ_E_SHAPE, "%s: M=%lld (at most 16 rows per call)", who, (long long)M);
    RWKVQ_REQUIRE(K % 128 == 0, RWKVQ_E_SHAPE, "%s: K=%lld must be a multiple of 128", who, (long long)K);
    RWKVQ_REQUIRE(aligned16(w_codes) && ldw % 16 == 0 && ldw >= K / 2, RWKVQ_E_ALIGN, "%s: weight code rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(((uintptr_t)w_block_scales & 1) == 0 && ldws % 2 == 0 && ldws >= K / 16, RWKVQ_E_ALIGN, "%s: weight scale rows must be 2-byte aligned", who);
    RWKVQ_REQUIRE(((uintptr_t)a_codes & 7) == 0 && lda % 8 == 0 && lda >= K / 2 && ldas >= K / 16, RWKVQ_E_ALIGN, "%s: activation code rows must be 8-byte aligned", who);
    RWKVQ_REQUIRE(ldo >= N, RWKVQ_E_SHAPE, "%s: ldo < N", who);
    if (M == 0 || N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(K > 0, RWKVQ_E_SHAPE, "%s: K=0", who);
    const size_t smem = (size_t)rwkvq_gemv_nvfp4_smem_bytes(M, K);
    RWKVQ_REQUIRE(smem <= 200 * 1024, RWKVQ_E_SHAPE, "%s: M*K = %lld*%lld does not fit shared memory; call with fewer rows", who, (long long)M, (long long)K);
    Nf4Args a{};
    a.a_codes = a_codes; a.a_bs = a_block_scales; a.a_pts = a_pts; a.w = w_codes; a.w_bs = w_block_scales; a.w_ts = w_tscale;
    a.out = (__half*)out_f16; a.lda = lda; a.ldas = ldas; a.ldw = ldw; a.ldws = ldws; a.ldo = ldo;
    a.M = (int)M; a.N = (int)N; a.K = (int)K; a.pitch = (int)(2 * K + 16);
    auto kern = gemv_nvfp4_kernel<4>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    RWKVQ_REQUIRE(e == cudaSuccess, RWKVQ_E_LAUNCH, "%s: cudaFuncSetAttribute: %s", who, cudaGetErrorString(e));
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThr, smem);
    RWKVQ_REQUIRE(e == cudaSuccess && per_sm >= 1, RWKVQ_E_LAUNCH, "%s: occupancy query failed", who);
    const int64_t tiles = (N + 7) / 8;
    const unsigned grid = (unsigned)std::min<int64_t>(tiles, (int64_t)sm_count() * per_sm);
    kern<<<grid, kThr, smem, (cudaStream_t)stream>>>(a);
    return check_launch(who);
}

int64_t rwkvq_gemv_nvfp4_fused_smem_bytes(int64_t M, int64_t K) { return (int64_t)nf_fused_smem(M <= 8 ? 1 : 2, 2, (int)M, (int)K); }

int32_t rwkvq_gemv_nvfp4_fused(const void* x, int32_t x_dtype, int64_t ldx, const uint8_t* w_codes, int64_t ldw,
                               const uint8_t* w_block_scales, int64_t ldws, const float* w_tscale, void* out_f16, int64_t ldo,
                               int64_t M, int64_t N, int64_t K, void* stream) {
    const char* who = "gemv_nvfp4_fused";
    RWKVQ_REQUIRE(x && w_codes && w_block_scales && w_tscale && out_f16, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, x_dtype);
    RWKVQ_REQUIRE(M >= 0 && N >= 0 && K >= 0 && M <= 16, RWKVQ_E_SHAPE, "%s: M=%lld (at most 16 rows per call)", who, (long long)M);
    RWKVQ_REQUIRE(K % 512 == 0, RWKVQ_E_SHAPE, "%s: K=%lld must be a multiple of 512", who, (long long)K);
    RWKVQ_REQUIRE(aligned16(w_codes) && ldw % 16 == 0 && ldw >= K / 2, RWKVQ_E_ALIGN, "%s: weight code rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(aligned16(w_block_scales) && ldws % 16 == 0 && ldws >= K / 16, RWKVQ_E_ALIGN, "%s: weight scale rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(aligned16(x) && ldx % 8 == 0 && ldx >= K, RWKVQ_E_ALIGN, "%s: activation rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(ldo >= N, RWKVQ_E_SHAPE, "%s: ldo < N", who);
    if (M == 0 || N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(K > 0, RWKVQ_E_SHAPE, "%s: K=0", who);
    NfFusedArgs a{};
    a.x = x; a.w = w_codes; a.w_bs = w_block_scales; a.w_ts = w_tscale; a.out = (__half*)out_f16;
    a.ldx = ldx; a.ldw = ldw; a.ldws = ldws; a.ldo = ldo; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.pitch = (int)(2 * K + 16);
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dtype == RWKVQ_F16) return M <= 8 ? dispatch_nf_fused<RWKVQ_F16, 1>(a, st) : dispatch_nf_fused<RWKVQ_F16, 2>(a, st);
    return M <= 8 ? dispatch_nf_fused<RWKVQ_BF16, 1>(a, st) : dispatch_nf_fused<RWKVQ_BF16, 2>(a, st);
}

int64_t rwkvq_actq_nvfp4_fused_scratch_bytes(void) { return (2 * kNfQMaxCtas + 32) * 4; }

int32_t rwkvq_actq_nvfp4_fused(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes, int64_t ldc,
                               uint8_t* block_scales, int64_t lds, uint8_t* block_scales_blocked, float* pts, void* scratch,
                               int64_t scratch_bytes, int32_t* status, void* stream) {
    const char* who = "actq_nvfp4_fused";
    RWKVQ_REQUIRE(x && codes && pts && scratch && (block_scales || block_scales_blocked), RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, x_dtype);
    RWKVQ_REQUIRE(M > 0 && K > 0 && K % 16 == 0 && M < (1 << 30), RWKVQ_E_SHAPE, "%s: M=%lld K=%lld (K must be a multiple of 16)", who, (long long)M, (long long)K);
    RWKVQ_REQUIRE(block_scales_blocked == nullptr || K % 64 == 0, RWKVQ_E_SHAPE, "%s: blocked scales need K %% 64 == 0", who);
    RWKVQ_REQUIRE(aligned16(x) && ldx % 8 == 0 && ldx >= K, RWKVQ_E_ALIGN, "%s: activation rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(((uintptr_t)codes & 3) == 0 && ldc % 4 == 0 && ldc >= K / 2 && (block_scales == nullptr || lds >= K / 16), RWKVQ_E_ALIGN,
                  "%s: code rows must be 4-byte aligned", who);
    RWKVQ_REQUIRE(scratch_bytes >= rwkvq_actq_nvfp4_fused_scratch_bytes() && ((uintptr_t)scratch & 3) == 0, RWKVQ_E_WORKSPACE,
                  "%s: scratch of %lld bytes needed", who, (long long)rwkvq_actq_nvfp4_fused_scratch_bytes());
    NfQArgs a{};
    a.x = x; a.codes = codes; a.bs_rows = block_scales; a.bs_blocked = block_scales_blocked; a.pts = pts;
    a.slots = reinterpret_cast<float*>(scratch); a.flags = reinterpret_cast<uint32_t*>(scratch) + kNfQMaxCtas; a.status = status ? status : device_status_ptr();
    a.ldx = ldx; a.ldc = ldc; a.lds = lds; a.M = (int)M; a.K = (int)K;
    a.wait_ns = wait_limit_ns();
    const char* small_env = std::getenv("RWKVQ_NVFP4_ACTQ_SMALL_MAX");  // read per call: a test switches routes in one process
    // measured: up to 4 vectors per thread of the largest cluster the one launch wins (att, 16 rows: 9.5 against 10.2 us;
    // FFN value, 4 rows: 14.0 against 18.6 us), at 8 per thread the two chained launches are as fast or faster
    const int64_t small_max = small_env ? std::atoll(small_env) : (int64_t)8 * 4 * kNfSmallThreads;
    if (M * (K / 8) <= std::min<int64_t>(small_max, (int64_t)8 * kNfSmallKeep * kNfSmallThreads) && K / 8 < 65536) {
        int cluster = 1;                                 // about 4 vectors per thread
        while (cluster < 8 && M * (K / 8) > (int64_t)cluster * 4 * kNfSmallThreads) cluster <<= 1;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)cluster);
        cfg.blockDim = dim3(kNfSmallThreads);
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)cluster;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = use_pdl() ? 2 : 1;
        const cudaError_t e = x_dtype == RWKVQ_F16 ? cudaLaunchKernelEx(&cfg, actq_nvfp4_small_kernel<RWKVQ_F16>, a)
                                                   : cudaLaunchKernelEx(&cfg, actq_nvfp4_small_kernel<RWKVQ_BF16>, a);
        if (e != cudaSuccess) {
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
        }
        return check_launch(who);
    }
    const char* two_env = std::getenv("RWKVQ_NVFP4_ACTQ_TWO_MAX");      // read per call: a test switches routes in one process
    const int64_t two_max = two_env ? std::atoll(two_env) : kNfTwoMaxVectors;
    if (M * (K / 8) <= two_max) {
        const int kv = (int)(K / 8);
        int cpr = 1;                                     // CTAs per row: about two CTAs per SM in all, 256+ vectors each
        while ((int64_t)M * cpr < 2 * (int64_t)sm_count() && cpr * 2 * kNfTwoThreads <= kv) cpr <<= 1;
        const int rows = (int)std::min<int64_t>(M, std::max<int64_t>(1, 4 * (int64_t)sm_count() / cpr));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)(rows * cpr));
        cfg.blockDim = dim3(kNfTwoThreads);
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = use_pdl() ? 1 : 0;
        cudaError_t e = x_dtype == RWKVQ_F16 ? cudaLaunchKernelEx(&cfg, actq_nvfp4_two_amax_kernel<RWKVQ_F16>, a, cpr)
                                             : cudaLaunchKernelEx(&cfg, actq_nvfp4_two_amax_kernel<RWKVQ_BF16>, a, cpr);
        if (e == cudaSuccess)
            e = x_dtype == RWKVQ_F16 ? cudaLaunchKernelEx(&cfg, actq_nvfp4_two_codes_kernel<RWKVQ_F16>, a, cpr)
                                     : cudaLaunchKernelEx(&cfg, actq_nvfp4_two_codes_kernel<RWKVQ_BF16>, a, cpr);
        if (e != cudaSuccess) {
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
        }
        g_launches.fetch_add(1, std::memory_order_relaxed);         // two launches: check_launch counts the other one
        return check_launch(who);
    }
    const int grid = (int)std::min<int64_t>(M, std::min<int64_t>(512, 2 * (int64_t)sm_count()));
    void* args[] = {(void*)&a};
    const void* fn = x_dtype == RWKVQ_F16 ? (const void*)actq_nvfp4_fused_kernel<RWKVQ_F16> : (const void*)actq_nvfp4_fused_kernel<RWKVQ_BF16>;
    const cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kNfQThreads), args, 0, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
    }
    return check_launch(who);
}

}  // extern "C"
