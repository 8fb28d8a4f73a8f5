// W8A8 projections for small M (decode): FP8 e4m3 x e4m3 and INT8 x INT8, single matrix or r/k/v in one launch.
//
// The kernel is HBM-bound and written for instruction count: at the HBM rate an SM has about 88 issue slots per
// 512 bytes of weights, and everything that is not a copy, a shared-memory load or an MMA eats into them.
//
// Data path.  The weight matrix [N,K] (one byte per element) is read exactly once.  A warp owns 16 weight rows
// (one "row tile") over a contiguous K range; lane (g = lane/4, t = lane%4) copies the 16 bytes
// W[n0+g][k0+16t .. +15] and W[n0+g+8][same] of each 64-byte unit with cp.async straight into its own slots of a
// per-warp ring in shared memory and reads them back with two 128-bit loads.  The WEIGHTS are the 16-row A operand
// of mma.sync (rows g and g+8 of the lane) and up to 8 tokens the B operand: INT8 two m16n8k32 per unit; FP8 the
// bytes are widened to f16 in registers (mma.sync has no fast e4m3 path on sm_100) for four m16n8k16 -- the
// converted values land directly in the A registers, so no register moves surround the MMAs.  An MMA sums over its
// k-slots, so the slots may be filled in any order as long as A and B agree; the B fragment (quantized
// activations of token g) is a consecutive register pair of a 128-bit load from the activation tile.
// All addresses inside a chunk of D units are a base register plus a compile-time offset.
//
// Work split.  A CTA (8 warps, two CTAs per SM) takes a contiguous range of the row tiles of ONE matrix and works
// through it in rounds of R tiles (R = 1, 2, 4 or 8, chosen on the host so that a CTA usually needs one round);
// 8/R warps share a tile, each with its own contiguous part of K, and add their partial sums in a fixed order
// through shared memory (run-to-run identical results).  R = 8: no reduction, the lanes store their results.
// B-fragment tokens beyond M are read from row M-1: they only feed accumulator columns that are never stored.
//
// Latency hiding.  Every warp keeps S-1 chunks (D x 512 bytes each) in flight; the ring runs ahead across rounds
// and its first S-1 chunks are issued BEFORE the prologue.  With programmatic dependent launch that prefetch also
// overlaps the tail of the previous kernel in the stream: only the weights (never written by any kernel) are
// touched before griddepcontrol.wait.
//
// Fused prologue (what prep_x / prep3_x / prep_x_int8 + the in-kernel quantization of the reference do):
//   FP8 : amax over the whole [M,K] call, inv = 448/max(amax,1e-12), code = e4m3(clamp(bf16(x)*inv)),
//         result scale (amax/448)*w_scale; the codes are kept as f16 values (2 bytes) in shared memory.
//   INT8: per row amax, s = 127/amax, code = trunc(clamp(x*s,-128,127)), row scale amax/127.
#include <cstdlib>

#include "w8a8.cuh"

namespace rwkvq {

constexpr int kGemvD = 4;                 // units per chunk (one cp.async group); a unit is 16 rows x 64 bytes = 1 KB per warp:
                                          // a lane streams 256 contiguous bytes of each of its two rows per chunk
constexpr int kGemvHeadPad = 96;          // red | xs[32] | sh[8] | pad: 160 + 96 = 256 bytes before the ring

static unsigned long long* g_gemv_trace = nullptr;

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The 2 D asynchronous 16-byte copies (global -> shared, bypassing L1) of one chunk: unit J lies J*64 bytes further
// along the two weight rows of this lane (g and g+8) and J*1024 bytes further in the warp's ring stage (row g+8 at
// +512), all as immediates of the instruction.  FULL: every unit lies inside the row; otherwise a unit whose first
// byte is at or beyond kend copies nothing and zero-fills its 16 bytes.
template <int J, int D, bool FULL>
__device__ __forceinline__ void issue_slots(uint32_t dst, const uint8_t* src0, const uint8_t* src1, int kbyte, int kend, const uint8_t* safe) {
    if constexpr (J < D) {
        if constexpr (FULL) {
            asm volatile("cp.async.cg.shared.global [%0+%2], [%1+%3], 16;" ::"r"(dst), "l"(src0), "n"(J * 1024), "n"(J * 64) : "memory");
            asm volatile("cp.async.cg.shared.global [%0+%2], [%1+%3], 16;" ::"r"(dst), "l"(src1), "n"(J * 1024 + 512), "n"(J * 64) : "memory");
        } else {
            const bool valid = kbyte + J * 64 < kend;
            const int n = valid ? 16 : 0;
            asm volatile("cp.async.cg.shared.global [%0+%3], [%1], 16, %2;" ::"r"(dst), "l"(valid ? src0 + J * 64 : safe), "r"(n), "n"(J * 1024) : "memory");
            asm volatile("cp.async.cg.shared.global [%0+%3], [%1], 16, %2;" ::"r"(dst), "l"(valid ? src1 + J * 64 : safe), "r"(n), "n"(J * 1024 + 512) : "memory");
        }
        issue_slots<J + 1, D, FULL>(dst, src0, src1, kbyte, kend, safe);
    }
}

// One chunk of the K loop.  The WEIGHTS are the 16-row A operand of the MMA (rows g and g+8 of this lane), up to 8
// tokens the B operand: xb[i] points at this lane's 16 k-values of token min(8i+g, M-1) for unit 0.  FP8: a lane's
// 16 bytes per row are widened to eight f16 pairs and feed four m16n8k16 together with the other row's; the B
// registers are consecutive pairs of two 128-bit loads.  INT8: two m16n8k32 per unit, B from one 128-bit load.
// FP8 on pre-quantized codes (WIDE = false): the tile holds the e4m3 codes as they come (1 byte each), a lane's 16 codes of
// a unit arrive with one 128-bit load and are widened here (8 conversions per token tile and unit).
template <int QT, bool WIDE, int NT, int D, typename T>
__device__ __forceinline__ void chunk_body(const uint8_t* st, const uint8_t* const (&xb)[NT], T (&c)[NT][4], T (&c2)[NT][4]) {
#pragma unroll
    for (int j = 0; j < D; ++j) {
        const uint4 wg = *reinterpret_cast<const uint4*>(st + j * 1024);
        const uint4 wh = *reinterpret_cast<const uint4*>(st + j * 1024 + 512);
        if constexpr (QT == QT_FP8) {
            const uint4 g01 = e4m3x8_to_f16x8(make_uint2(wg.x, wg.y)), g23 = e4m3x8_to_f16x8(make_uint2(wg.z, wg.w));
            const uint4 h01 = e4m3x8_to_f16x8(make_uint2(wh.x, wh.y)), h23 = e4m3x8_to_f16x8(make_uint2(wh.z, wh.w));
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                uint4 b0, b1;
                if constexpr (WIDE) {
                    b0 = *reinterpret_cast<const uint4*>(xb[i] + j * 128);
                    b1 = *reinterpret_cast<const uint4*>(xb[i] + j * 128 + 16);
                } else {
                    const uint4 bc = *reinterpret_cast<const uint4*>(xb[i] + j * 64);
                    b0 = e4m3x8_to_f16x8(make_uint2(bc.x, bc.y));
                    b1 = e4m3x8_to_f16x8(make_uint2(bc.z, bc.w));
                }
                mma_f16(c[i], g01.x, h01.x, g01.y, h01.y, b0.x, b0.y);
                mma_f16(c2[i], g01.z, h01.z, g01.w, h01.w, b0.z, b0.w);
                mma_f16(c[i], g23.x, h23.x, g23.y, h23.y, b1.x, b1.y);
                mma_f16(c2[i], g23.z, h23.z, g23.w, h23.w, b1.z, b1.w);
            }
        } else {
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                const uint4 b = *reinterpret_cast<const uint4*>(xb[i] + j * 64);
                mma_s8(c[i], wg.x, wh.x, wg.y, wh.y, b.x, b.y);
                mma_s8(c2[i], wg.z, wh.z, wg.w, wh.w, b.z, b.w);
            }
        }
    }
}

// Results of one 16-row tile, straight from the accumulator fragments: lane (g, t) holds weight rows n0+g (values 0, 1)
// and n0+g+8 (values 2, 3) for the tokens 8i+2t and 8i+2t+1.
template <int QT, int NT, bool RELU2, typename T>
__device__ __forceinline__ void store_tile(const W8Args& a, int mat, int n0, int g, int t, const T (&c)[NT][4], float act_scale,
                                           const float* xs, float wscale, float (&hmax)[2]) {
    // weight scale of this lane's two rows: one per matrix, or one per output row with RWKVQ_FLAG_WSCALE_PER_ROW
    float wlo = wscale, whi = wscale;
    if (a.flags & RWKVQ_FLAG_WSCALE_PER_ROW) {
        wlo = a.ws[mat][min(n0 + g, a.N - 1)];
        whi = a.ws[mat][min(n0 + g + 8, a.N - 1)];
    }
    const float out_lo = act_scale * wlo, out_hi = act_scale * whi;     // FP8: (amax/448) * w_scale, formed before the product
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = i * 8 + 2 * t + (j & 1), n = n0 + g + ((j & 2) ? 8 : 0);
            if (m >= a.M || n >= a.N) continue;
            float f;
            if constexpr (QT == QT_FP8) {
                f = c[i][j] * ((j & 2) ? out_hi : out_lo);
            } else {
                if (a.acc[mat]) a.acc[mat][(int64_t)m * a.ldacc + n] = c[i][j];
                f = (float)c[i][j] * (xs[m] * ((j & 2) ? whi : wlo));
            }
            if (a.flags & RWKVQ_FLAG_OUT_VIA_BF16) f = bf16_round(f);
            __half y = __float2half_rn(f);
            if constexpr (RELU2) {
                // the engine's relu_square on the fp16 result: fp16(max(y, 0)^2) in fp32 arithmetic; its maximum (over the
                // bf16-rounded values where the consumer takes its amax there) is published for the projection that follows
                const float v = fmaxf(__half2float(y), 0.f);
                y = __float2half_rn(v * v);
                const float hv = __half2float(y);
                if constexpr (QT == QT_FP8) hmax[0] = fmaxf(hmax[0], (a.flags & RWKVQ_FLAG_AMAX_AFTER_BF16) ? bf16_round(hv) : hv);
                else hmax[j & 1] = fmaxf(hmax[j & 1], hv);          // INT8 scales its activations per row: tokens 2t and 2t + 1 (NT = 1)
            }
            a.out[mat][(int64_t)m * a.ldo + n] = y;
        }
}

// S: stages of each warp's shared-memory weight ring.  NT: token tiles of 8 (M <= 8 NT).
// Everything between the kernel's entry and its first copies, and between the dependency release and the first
// MMA, is a single pass of dependent scalar code and shows up in full in a 5-15 us launch: the tile split and all
// divisions are done on the host (W8Args::tq, trem, lgR), and whatever does not need the activations is computed
// before griddepcontrol.wait.
// PRE: the activations arrive as codes (a.codes / a.ascale, quantized once by an earlier launch) and the prologue is
// one bulk copy per row into the tile -- no arithmetic, M*K bytes per CTA; otherwise the prologue quantizes x itself.
// FFN: 0 = plain projection; 1 = relu^2 in the epilogue and its maximum published (rwkvq_gemv_fp8_relu2); 2 = quantize with
// the published amax (rwkvq_gemv_fp8_preamax).  Separate instantiations: the plain kernel carries none of that code.
template <int QT, int DT, int NT, int S, bool PRE, int FFN = 0>
__global__ void __launch_bounds__(kThr, 2) gemv_w8a8_kernel(const W8Args a) {
    using T = typename Acc<QT>::T;
    constexpr int D = kGemvD;
    constexpr bool WIDE = !PRE;
    constexpr int AB = (QT == QT_FP8 && WIDE) ? 2 : 1;          // bytes per activation in the shared-memory tile
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: red[kWarps][NT*4][32] | xs[32] | sh[8] | xbar + pad (96 B) | ring[kWarps][S][D][2][32 lanes] x 16 B | xq[M][pitch] + 512 B
    T* red = reinterpret_cast<T*>(smem);
    float* xs = reinterpret_cast<float*>(smem + kWarps * NT * 4 * 32 * 4);
    float* sh = xs + 32;
    uint64_t* xbar = reinterpret_cast<uint64_t*>(sh + 8);          // FP8: the raw activations have landed in the tile
    uint8_t* ring = reinterpret_cast<uint8_t*>(sh + 8) + kGemvHeadPad;   // ring and tile start on a 128-byte boundary
    uint8_t* xq = ring + (size_t)kWarps * S * D * 1024;

    griddep_launch_dependents();
    w8_mark(a, 0);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int mat = ((int)blockIdx.x >= a.cpm) + ((int)blockIdx.x >= 2 * a.cpm);
    const int cb = (int)blockIdx.x - mat * a.cpm;
    const int tb = cb * a.tq + min(cb, a.trem), te = tb + a.tq + (cb < a.trem ? 1 : 0);   // this CTA's 16-row tiles
    const int lgR = a.lgR, R = 1 << lgR, lgKS = 3 - lgR, KS = 1 << lgKS;
    const int slot = warp >> lgKS, ks = warp & (KS - 1);     // which tile of a round, which part of K
    const int rounds = (te - tb + R - 1) >> lgR;
    const int units = (a.K + 63) >> 6, upw = (units + KS - 1) >> lgKS;
    const int ub = ks * upw, ue = min(ub + upw, units);
    const int nch = (max(ue - ub, 0) + D - 1) / D;           // chunks per tile for this warp (D is a power of two)
    const int kbeg = ub * 64 + 16 * t;                       // this lane's first byte of a weight row
    const int kend = min(ue * 64, a.K);
    const bool full = ((ue - ub) % D == 0) && (a.K % 64 == 0);
    const int my_rounds = (nch > 0 && te - tb > slot) ? ((te - tb - slot + R - 1) >> lgR) : 0;   // rounds in which this warp has a tile
    uint8_t* my_ring = ring + (size_t)warp * S * D * 1024 + lane * 16;
    const uint32_t my_ring_s = (uint32_t)__cvta_generic_to_shared(my_ring);
    const uint8_t* wbase = a.w[mat];

    // producer side of the ring: chunk p_ch of the tile of round p_round goes to stage p_stage; one group per chunk
    int p_round = 0, p_ch = 0, p_stage = 0;
    const uint8_t *p_src0 = wbase, *p_src1 = wbase;
    auto set_rows = [&](int round) {
        const int n0 = (tb + round * R + slot) << 4;
        p_src0 = wbase + (int64_t)min(n0 + g, a.N - 1) * a.ldw + kbeg;
        p_src1 = wbase + (int64_t)min(n0 + g + 8, a.N - 1) * a.ldw + kbeg;
    };
    if (my_rounds > 0) set_rows(0);
    auto issue = [&]() {
        if (p_round < my_rounds) {
            const uint32_t dst = my_ring_s + p_stage * (D * 1024);
            if (full) issue_slots<0, D, true>(dst, p_src0, p_src1, 0, 0, wbase);
            else issue_slots<0, D, false>(dst, p_src0, p_src1, kbeg + p_ch * (D * 64), kend, wbase);
            p_src0 += D * 64;
            p_src1 += D * 64;
            if (++p_ch == nch) {
                p_ch = 0;
                if (++p_round < my_rounds) set_rows(p_round);
            }
        }
        cp_async_commit();
        if (++p_stage == S) p_stage = 0;
    };
#pragma unroll
    for (int i = 0; i < S - 1; ++i) issue();
    w8_mark(a, 1);

    // bytes of the activation tile that chunk overruns and rows shorter than their pitch can touch must be finite
    {
        const int padv = (a.pitch - a.K * AB) >> 4;          // 16-byte vectors of padding per row
        for (int r = 0; r < a.M; ++r)
            if ((int)threadIdx.x < padv) *reinterpret_cast<uint4*>(xq + (size_t)r * a.pitch + a.K * AB + threadIdx.x * 16) = make_uint4(0, 0, 0, 0);
        if (threadIdx.x >= 32 && threadIdx.x < 64)
            *reinterpret_cast<uint4*>(xq + (size_t)a.M * a.pitch + (threadIdx.x - 32) * 16) = make_uint4(0, 0, 0, 0);
    }
    // this lane's token rows of the activation tile; tokens beyond M read row M-1 (columns that are never stored)
    const uint8_t* xb0[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) xb0[i] = xq + min(i * 8 + g, a.M - 1) * a.pitch + kbeg * AB;
    const float wscale = a.ws[mat][0];       // weights and their scale are never written by a kernel

    if ((QT == QT_FP8 || PRE) && threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(xbar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();  // the barrier and the zeroed pads are visible before anybody uses them

    griddep_wait();   // activations may come from the previous kernel; results may overwrite what it read
    w8_mark(a, 2);

    float out_scale = 0.f;   // FP8: amax/448 (the weight scale joins it in store_tile)
    if constexpr (PRE) {
        if (threadIdx.x == 0) {
            const uint32_t b = (uint32_t)__cvta_generic_to_shared(xbar);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"((uint32_t)(a.M * a.K)) : "memory");
#pragma unroll 1
            for (int r = 0; r < a.M; ++r)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"((uint32_t)__cvta_generic_to_shared(xq + (size_t)r * a.pitch)), "l"(a.codes[mat] + (int64_t)r * a.lda),
                               "r"((uint32_t)a.K), "r"(b) : "memory");
        }
        if constexpr (QT == QT_FP8) {
            const float am = a.ascale[mat][0];
            out_scale = a.amax_is_amax ? div_mode_f32(fmaxf(am, 1e-12f), 448.f, a.div_mode) : am;
        } else {
            if ((int)threadIdx.x < a.M) xs[threadIdx.x] = a.ascale[mat][threadIdx.x];
        }
        if (!w8_staged_or_report(xbar, a.status, a.wait_ns)) {     // reported: drain the weight ring and stop
            cp_async_wait<0>();
            return;
        }
    } else if constexpr (QT == QT_FP8) {
        const float amax = quantize_fp8_to_smem<DT, WIDE, FFN == 2>(a, mat, xq, sh, xbar);
        if (amax < 0.f) {          // the staging copy timed out (reported): drain the weight ring and stop
            cp_async_wait<0>();
            return;
        }
        out_scale = div_mode_f32(amax, 448.f, a.div_mode);
    } else {
        quantize_int8_to_smem<DT, FFN == 2>(a, mat, xq, xs, sh);
    }
    __syncthreads();
    w8_mark(a, 3);
    if (FFN == 2 && threadIdx.x == 0) {
        // every thread of this CTA has used the published amax; the last CTA to say so clears it for the next producer
        __threadfence();
        if (atomicAdd(a.ffn_count, 1) == (int)gridDim.x - 1) {
            if constexpr (QT == QT_FP8) {
                *a.ffn_amax = 0.f;
            } else {
                for (int r = 0; r < 8; ++r) a.ffn_amax[2 + r] = 0.f;
            }
            __threadfence();
            *a.ffn_count = 0;
        }
    }

    float hmax[2] = {0.f, 0.f};
    int stage = 0;
    for (int r = 0; r < rounds; ++r) {
        T c[NT][4], c2[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) c[i][j] = c2[i][j] = 0;
        if (r < my_rounds) {
            const uint8_t* xb[NT];
#pragma unroll
            for (int i = 0; i < NT; ++i) xb[i] = xb0[i];
            for (int ch = 0; ch < nch; ++ch) {
                issue();                       // keep S-1 chunks in flight
                cp_async_wait<S - 1>();        // this lane's copies of the current chunk have landed
                chunk_body<QT, WIDE, NT, D>(my_ring + stage * (D * 1024), xb, c, c2);
#pragma unroll
                for (int i = 0; i < NT; ++i) xb[i] += D * 64 * AB;
                if (++stage == S) stage = 0;
            }
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) c[i][j] += c2[i][j];      // the two accumulators halve the dependent MMA chains
        }
        const int tile = tb + r * R + slot;
        if (KS > 1) {
            // the warps of a tile add their parts of K in warp order
            T* rb = red;
            if (r > 0) __syncthreads();        // the previous round's partial sums have been read
            if (ks > 0) {
#pragma unroll
                for (int i = 0; i < NT; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) rb[((warp * NT + i) * 4 + j) * 32 + lane] = c[i][j];
            }
            __syncthreads();
            if (ks == 0 && tile < te) {
                for (int kk = 1; kk < KS; ++kk)
#pragma unroll
                    for (int i = 0; i < NT; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) c[i][j] += rb[(((warp + kk) * NT + i) * 4 + j) * 32 + lane];
                store_tile<QT, NT, FFN == 1>(a, mat, tile << 4, g, t, c, out_scale, xs, wscale, hmax);
            }
        } else if (tile < te) {
            store_tile<QT, NT, FFN == 1>(a, mat, tile << 4, g, t, c, out_scale, xs, wscale, hmax);
        }
    }
    cp_async_wait<0>();
    if constexpr (FFN == 1 && QT == QT_FP8) {          // one atomic per CTA
        const float hm = warp_max(hmax[0]);
        __syncthreads();
        if (lane == 0) sh[warp] = hm;
        __syncthreads();
        if (threadIdx.x == 0) {
            float b = sh[0];
#pragma unroll
            for (int i = 1; i < kWarps; ++i) b = fmaxf(b, sh[i]);
            atomic_max_nonneg(a.ffn_amax, b);
        }
    }
    if constexpr (FFN == 1 && QT == QT_INT8) {         // one atomic per CTA and token row
        float v0 = hmax[0], v1 = hmax[1];               // tokens 2t and 2t + 1: fold the lanes that share t (all g)
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            v0 = fmaxf(v0, __shfl_xor_sync(0xffffffffu, v0, o));
            v1 = fmaxf(v1, __shfl_xor_sync(0xffffffffu, v1, o));
        }
        __syncthreads();                                // the reduction buffer is free
        float* rowmax = reinterpret_cast<float*>(red);  // [kWarps][8]
        if (lane < 4) {
            rowmax[warp * 8 + 2 * lane] = v0;
            rowmax[warp * 8 + 2 * lane + 1] = v1;
        }
        __syncthreads();
        if ((int)threadIdx.x < a.M && threadIdx.x < 8) {
            float b = rowmax[threadIdx.x];
#pragma unroll
            for (int i = 1; i < kWarps; ++i) b = fmaxf(b, rowmax[i * 8 + threadIdx.x]);
            if (b > 0.f) atomic_max_nonneg(a.ffn_amax + 2 + threadIdx.x, b);
        }
    }
    w8_mark(a, 4);
}

static size_t smem_bytes(int NT, int M, int pitch, int S) {
    return (size_t)kWarps * NT * 4 * 32 * 4 + 32 * 4 + 8 * 4 + kGemvHeadPad + (size_t)kWarps * S * kGemvD * 1024 + (size_t)M * pitch + 512;
}

constexpr size_t kFusedSmemMax = 224 * 1024;    // of the 227 KB a CTA may opt in to

template <int QT, int DT, int NT, int S, bool PRE, int FFN = 0>
static int32_t launch_one(W8Args a, size_t smem, cudaStream_t st) {
    auto kern = gemv_w8a8_kernel<QT, DT, NT, S, PRE, FFN>;
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
    // every CTA works on one matrix: the grid is a multiple of the matrix count, at most one wave
    const int ntile = (a.N + 15) / 16;
    a.cpm = std::max(1, std::min(ntile, sm_count() * per_sm / a.nmat));
    a.tq = ntile / a.cpm;                 // CTA cb of a matrix takes tq row tiles, the first trem CTAs one more
    a.trem = ntile % a.cpm;
    // Tiles per round from the density of ONE matrix over the whole GPU, whatever the matrix count: the split of K
    // (and with it the order of the fp32 additions) is then the same for a fused r/k/v launch and for three single
    // launches, which keeps their results bit-identical.
    const int tpc = (ntile + sm_count() * per_sm - 1) / (sm_count() * per_sm);
    a.lgR = 0;
    while ((1 << a.lgR) < kWarps && (1 << a.lgR) < tpc) ++a.lgR;
    a.trace = g_gemv_trace;
    a.status = device_status_ptr();
    a.wait_ns = wait_limit_ns();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(a.cpm * a.nmat));
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

// Ring depth: the deepest ring (5, 4, 3 stages) that leaves room for two CTAs per SM; failing that, one CTA per SM with
// the deepest ring that fits beside the activation tile (long rows, many tokens) -- one CTA with a deep ring measured
// faster than two CTAs with two stages.
template <int QT, int DT, int NT, bool PRE, int FFN = 0>
static int32_t dispatch_s(const W8Args& a, cudaStream_t st) {
    const size_t s5 = smem_bytes(NT, a.M, a.pitch, 5), s4 = smem_bytes(NT, a.M, a.pitch, 4), s3 = smem_bytes(NT, a.M, a.pitch, 3),
                 s2 = smem_bytes(NT, a.M, a.pitch, 2);
    if (s5 <= kTwoPerSm) return launch_one<QT, DT, NT, 5, PRE, FFN>(a, s5, st);
    if (s4 <= kTwoPerSm) return launch_one<QT, DT, NT, 4, PRE, FFN>(a, s4, st);
    if (s3 <= kTwoPerSm) return launch_one<QT, DT, NT, 3, PRE, FFN>(a, s3, st);
    RWKVQ_REQUIRE(s2 <= kFusedSmemMax, RWKVQ_E_SHAPE, "gemv_w8a8: M*K = %d*%d does not fit the kernel's shared memory", a.M, a.K);
    if (s5 <= kFusedSmemMax) return launch_one<QT, DT, NT, 5, PRE, FFN>(a, s5, st);
    if (s4 <= kFusedSmemMax) return launch_one<QT, DT, NT, 4, PRE, FFN>(a, s4, st);
    if (s3 <= kFusedSmemMax) return launch_one<QT, DT, NT, 3, PRE, FFN>(a, s3, st);
    return launch_one<QT, DT, NT, 2, PRE, FFN>(a, s2, st);
}

template <int QT, int DT, bool PRE>
static int32_t dispatch_mt(const W8Args& a, cudaStream_t st) {
    if constexpr (!PRE) {                       // the FFN pair: up to 8 rows
        if (a.flags & (RWKVQ_FLAG_RELU2 | RWKVQ_FLAG_AMAX_GIVEN)) {
            RWKVQ_REQUIRE(a.M <= 8 && a.nmat == 1, RWKVQ_E_SHAPE, "gemv_fp8 relu2 / preamax: at most 8 rows, got %d", a.M);
            return (a.flags & RWKVQ_FLAG_RELU2) ? dispatch_s<QT, DT, 1, PRE, 1>(a, st) : dispatch_s<QT, DT, 1, PRE, 2>(a, st);
        }
    }
    if (a.M <= 8) return dispatch_s<QT, DT, 1, PRE>(a, st);
    if (a.M <= 16) return dispatch_s<QT, DT, 2, PRE>(a, st);
    return dispatch_s<QT, DT, 4, PRE>(a, st);
}

static int pitch_codes(int K) { return ((K + 127) / 128) * 128 + 64; }     // 1 byte per code
static int pitch_wide(int K) { return ((2 * K + 127) / 128) * 128 + 16; }  // f16 values of the e4m3 codes

bool gemv_codes_fits(int M, int K) {
    const int NT = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
    return M > 0 && M <= 32 && K % 16 == 0 && smem_bytes(NT, M, pitch_codes(K), 2) <= kFusedSmemMax;
}

int32_t gemv_codes_run(W8Args a, int qt, cudaStream_t st, const char* who) {
    RWKVQ_REQUIRE(a.M >= 0 && a.N >= 0 && a.K >= 0, RWKVQ_E_SHAPE, "%s: negative size", who);
    RWKVQ_REQUIRE(a.K % 16 == 0, RWKVQ_E_SHAPE, "%s: K=%d must be a multiple of 16", who, a.K);
    RWKVQ_REQUIRE(a.ldw >= a.K && a.ldw % 16 == 0, RWKVQ_E_ALIGN, "%s: ldw=%lld must be >= K and a multiple of 16", who, (long long)a.ldw);
    RWKVQ_REQUIRE(a.lda >= a.K && a.lda % 16 == 0, RWKVQ_E_ALIGN, "%s: lda=%lld must be >= K and a multiple of 16", who, (long long)a.lda);
    RWKVQ_REQUIRE(a.ldo >= a.N, RWKVQ_E_SHAPE, "%s: ldo=%lld < N", who, (long long)a.ldo);
    RWKVQ_REQUIRE(a.div_mode == RWKVQ_DIV_IEEE || a.div_mode == RWKVQ_DIV_FULL, RWKVQ_E_BADARG, "%s: div_mode %d", who, a.div_mode);
    for (int i = 0; i < a.nmat; ++i) {
        RWKVQ_REQUIRE(a.w[i] && a.ws[i] && a.out[i] && a.codes[i] && a.ascale[i], RWKVQ_E_BADARG, "%s: null pointer (matrix %d)", who, i);
        RWKVQ_REQUIRE(aligned16(a.w[i]) && aligned16(a.codes[i]), RWKVQ_E_ALIGN, "%s: weight / code pointer not 16-byte aligned", who);
    }
    if (a.M == 0 || a.N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(gemv_codes_fits(a.M, a.K), RWKVQ_E_SHAPE, "%s: M=%d K=%d does not fit the decode kernel (M <= 32, code tile in shared memory)", who, a.M, a.K);
    RWKVQ_REQUIRE((int64_t)a.nmat * ((a.N + 15) / 16) < (int64_t(1) << 27), RWKVQ_E_SHAPE, "%s: N too large", who);
    a.pitch = pitch_codes(a.K);
    a.flags &= ~(RWKVQ_FLAG_RELU2 | RWKVQ_FLAG_AMAX_GIVEN);
    return qt == QT_FP8 ? dispatch_mt<QT_FP8, RWKVQ_BF16, true>(a, st) : dispatch_mt<QT_INT8, RWKVQ_BF16, true>(a, st);
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
    // shared-memory row pitch of the activation tile: one byte per code (INT8, or FP8 with the narrow tile: dispatch_w)
    // or the f16 values of the e4m3 codes (2 B); the odd 64 / 16 bytes keep the fragment loads of different rows on
    // different banks
    a.pitch = QT == QT_FP8 ? pitch_wide(a.K) : pitch_codes(a.K);
    RWKVQ_REQUIRE((int64_t)a.nmat * ((a.N + 15) / 16) < (int64_t(1) << 27), RWKVQ_E_SHAPE, "%s: N too large", who);
    return x_dtype == RWKVQ_F16 ? dispatch_mt<QT, RWKVQ_F16, false>(a, st) : dispatch_mt<QT, RWKVQ_BF16, false>(a, st);
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

/* profiling aid: device buffer of [grid][8] uint64 that every decode GEMV launch stamps with CTA milestones */
void rwkvq_gemv_set_trace(void* device_buffer) { g_gemv_trace = reinterpret_cast<unsigned long long*>(device_buffer); }

int32_t rwkvq_gemv_fp8(const void* x, int32_t x_dtype, const float* awq, const uint8_t* w, int64_t ldw, const float* w_scale,
                       void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode,
                       uint32_t flags, void* stream) {
    W8Args a{};
    a.x[0] = x; a.awq[0] = awq; a.w[0] = w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldw = ldw; a.ldo = ldo;
    a.div_mode = div_mode; a.flags = flags & ~(RWKVQ_FLAG_RELU2 | RWKVQ_FLAG_AMAX_GIVEN);
    return run_fused<QT_FP8>(a, x_dtype, (cudaStream_t)stream, "gemv_fp8");
}

/* FFN key projection with the engine's relu_square folded into its epilogue, and the FFN value projection that takes
 * the amax the first one published.  ffn_scratch: 8 bytes owned by the caller, zeroed once; the pair leaves it zero. */
int32_t rwkvq_gemv_fp8_relu2(const void* x, int32_t x_dtype, const uint8_t* w, int64_t ldw, const float* w_scale, void* out_f16,
                             int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode, uint32_t flags,
                             void* ffn_scratch, void* stream) {
    RWKVQ_REQUIRE(ffn_scratch != nullptr && ((uintptr_t)ffn_scratch & 7) == 0, RWKVQ_E_BADARG, "gemv_fp8_relu2: ffn_scratch must be 8 aligned bytes");
    W8Args a{};
    a.x[0] = x; a.w[0] = w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldw = ldw; a.ldo = ldo;
    a.div_mode = div_mode; a.flags = (flags & ~RWKVQ_FLAG_AMAX_GIVEN) | RWKVQ_FLAG_RELU2;
    a.ffn_amax = reinterpret_cast<float*>(ffn_scratch);
    a.ffn_count = reinterpret_cast<int*>(ffn_scratch) + 1;
    return run_fused<QT_FP8>(a, x_dtype, (cudaStream_t)stream, "gemv_fp8_relu2");
}

int32_t rwkvq_gemv_fp8_preamax(const void* x, int32_t x_dtype, const uint8_t* w, int64_t ldw, const float* w_scale, void* out_f16,
                               int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode, uint32_t flags,
                               void* ffn_scratch, void* stream) {
    RWKVQ_REQUIRE(ffn_scratch != nullptr && ((uintptr_t)ffn_scratch & 7) == 0, RWKVQ_E_BADARG, "gemv_fp8_preamax: ffn_scratch must be 8 aligned bytes");
    W8Args a{};
    a.x[0] = x; a.w[0] = w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldw = ldw; a.ldo = ldo;
    a.div_mode = div_mode; a.flags = (flags & ~RWKVQ_FLAG_RELU2) | RWKVQ_FLAG_AMAX_GIVEN;
    a.ffn_amax = reinterpret_cast<float*>(ffn_scratch);
    a.ffn_count = reinterpret_cast<int*>(ffn_scratch) + 1;
    return run_fused<QT_FP8>(a, x_dtype, (cudaStream_t)stream, "gemv_fp8_preamax");
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
    a.div_mode = div_mode; a.flags = flags & ~(RWKVQ_FLAG_RELU2 | RWKVQ_FLAG_AMAX_GIVEN);
    return run_fused<QT_FP8>(a, x_dtype, (cudaStream_t)stream, "gemv_fp8_rkv");
}

int32_t rwkvq_gemv_int8(const void* x, int32_t x_dtype, const int8_t* w, int64_t ldw, const float* w_scale, void* out_f16,
                        int64_t ldo, int32_t* acc_out, int64_t ldacc, int64_t M, int64_t N, int64_t K, int64_t ldx,
                        int32_t div_mode, uint32_t flags, void* stream) {
    W8Args a{};
    a.x[0] = x; a.w[0] = (const uint8_t*)w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16; a.acc[0] = acc_out;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldw = ldw; a.ldo = ldo; a.ldacc = ldacc;
    a.div_mode = div_mode; a.flags = flags & ~(RWKVQ_FLAG_RELU2 | RWKVQ_FLAG_AMAX_GIVEN);
    RWKVQ_REQUIRE(acc_out == nullptr || ldacc >= N, RWKVQ_E_SHAPE, "gemv_int8: ldacc < N");
    return run_fused<QT_INT8>(a, x_dtype, (cudaStream_t)stream, "gemv_int8");
}

/* The FFN pair on INT8 weights (up to 8 rows).  INT8 activations carry one scale per ROW, so the key projection
 * publishes the maximum of fp16(max(y, 0)^2) per token row and the value projection quantizes every row with its own
 * published maximum.  ffn_scratch: 64 bytes owned by the caller (the FP8 pair uses the first 8 of the same block),
 * zeroed once; the pair leaves it zero.  Results equal projection -> relu_square -> projection bit for bit. */
int32_t rwkvq_gemv_int8_relu2(const void* x, int32_t x_dtype, const int8_t* w, int64_t ldw, const float* w_scale, void* out_f16,
                              int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode, uint32_t flags,
                              void* ffn_scratch, void* stream) {
    RWKVQ_REQUIRE(ffn_scratch != nullptr && ((uintptr_t)ffn_scratch & 7) == 0, RWKVQ_E_BADARG, "gemv_int8_relu2: ffn_scratch must be 64 bytes, 8-byte aligned");
    W8Args a{};
    a.x[0] = x; a.w[0] = (const uint8_t*)w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldw = ldw; a.ldo = ldo;
    a.div_mode = div_mode; a.flags = (flags & ~RWKVQ_FLAG_AMAX_GIVEN) | RWKVQ_FLAG_RELU2;
    a.ffn_amax = reinterpret_cast<float*>(ffn_scratch);
    a.ffn_count = reinterpret_cast<int*>(ffn_scratch) + 1;
    return run_fused<QT_INT8>(a, x_dtype, (cudaStream_t)stream, "gemv_int8_relu2");
}

int32_t rwkvq_gemv_int8_preamax(const void* x, int32_t x_dtype, const int8_t* w, int64_t ldw, const float* w_scale, void* out_f16,
                                int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode, uint32_t flags,
                                void* ffn_scratch, void* stream) {
    RWKVQ_REQUIRE(ffn_scratch != nullptr && ((uintptr_t)ffn_scratch & 7) == 0, RWKVQ_E_BADARG, "gemv_int8_preamax: ffn_scratch must be 64 bytes, 8-byte aligned");
    W8Args a{};
    a.x[0] = x; a.w[0] = (const uint8_t*)w; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldw = ldw; a.ldo = ldo;
    a.div_mode = div_mode; a.flags = (flags & ~RWKVQ_FLAG_RELU2) | RWKVQ_FLAG_AMAX_GIVEN;
    a.ffn_amax = reinterpret_cast<float*>(ffn_scratch);
    a.ffn_count = reinterpret_cast<int*>(ffn_scratch) + 1;
    return run_fused<QT_INT8>(a, x_dtype, (cudaStream_t)stream, "gemv_int8_preamax");
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
    a.div_mode = div_mode; a.flags = flags & ~(RWKVQ_FLAG_RELU2 | RWKVQ_FLAG_AMAX_GIVEN);
    return run_fused<QT_INT8>(a, x_dtype, (cudaStream_t)stream, "gemv_int8_rkv");
}

/* Several decode projections with ONE call across the boundary: the descriptors are walked in order and each is
 * launched exactly as the entry point of its kind would launch it (same kernels, same results). */
int32_t rwkvq_gemv_batch(const rwkvq_proj_desc* descs, int32_t count, void* stream) {
    RWKVQ_REQUIRE(descs != nullptr || count == 0, RWKVQ_E_BADARG, "gemv_batch: null descriptors");
    for (int32_t i = 0; i < count; ++i) {
        const rwkvq_proj_desc& d = descs[i];
        int32_t rc;
        switch (d.kind) {
            case RWKVQ_PROJ_FP8:
                rc = rwkvq_gemv_fp8(d.x[0], d.x_dtype, d.awq[0], (const uint8_t*)d.w[0], d.ldw, d.w_scale[0], d.out[0], d.ldo, d.M, d.N, d.K,
                                    d.ldx, d.div_mode, d.flags, stream);
                break;
            case RWKVQ_PROJ_FP8_RKV:
                rc = rwkvq_gemv_fp8_rkv(d.x[0], d.x[1], d.x[2], d.x_dtype, d.awq[0], d.awq[1], (const uint8_t*)d.w[0], (const uint8_t*)d.w[1],
                                        (const uint8_t*)d.w[2], d.ldw, d.w_scale[0], d.w_scale[1], d.w_scale[2], d.out[0], d.out[1], d.out[2],
                                        d.ldo, d.M, d.N, d.K, d.ldx, d.div_mode, d.flags, stream);
                break;
            case RWKVQ_PROJ_INT8:
                rc = rwkvq_gemv_int8(d.x[0], d.x_dtype, (const int8_t*)d.w[0], d.ldw, d.w_scale[0], d.out[0], d.ldo, nullptr, 0, d.M, d.N, d.K,
                                     d.ldx, d.div_mode, d.flags, stream);
                break;
            case RWKVQ_PROJ_INT8_RKV:
                rc = rwkvq_gemv_int8_rkv(d.x[0], d.x[1], d.x[2], d.x_dtype, (const int8_t*)d.w[0], (const int8_t*)d.w[1], (const int8_t*)d.w[2],
                                         d.ldw, d.w_scale[0], d.w_scale[1], d.w_scale[2], d.out[0], d.out[1], d.out[2], d.ldo, d.M, d.N, d.K,
                                         d.ldx, d.div_mode, d.flags, stream);
                break;
            default:
                return fail(RWKVQ_E_BADARG, "gemv_batch: descriptor %d has unknown kind %d", i, d.kind);
        }
        if (rc != RWKVQ_OK) return rc;
    }
    return RWKVQ_OK;
}

}  // extern "C"
