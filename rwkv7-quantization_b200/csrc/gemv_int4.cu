// Group-wise INT4 weight-only GEMV (W4A16, fp16 activations, M <= 16) for the decode shapes: HBM-bound streaming of
// the packed nibbles [N, K/2] straight into mma.sync.m16n8k16.f16 fragments.
//
// Lane (g = lane/4, t = lane%4) of a warp loads the 16 bytes = 32 nibbles W[n0+g][k0+32t .. +31]; a warp therefore
// covers 8 weight rows x 128 k per load, which is one quantization group (or half of a 256-group) per row.
//
// Nibbles become fp16 operands with one AND each and no arithmetic: a nibble u left in the low mantissa bits of an
// fp16 is the SUBNORMAL value u * 2^-24, which mma.sync multiplies exactly.  For a 32-bit word with nibbles n0..n7:
// w & 0x000F000F is the fp16 pair (n0, n4) * 2^-24, w & 0x00F000F0 is (n1, n5) * 2^-20, and the same two masks on
// w >> 8 give (n2, n6) and (n3, n7).  The MMA sums over its k slots in any order as long as A and B agree, so the
// activations are stored in shared memory with each run of 8 permuted to [0,4,1,5,2,6,3,7] -- one 128-bit shared
// load per word then yields exactly the A pairs that match the four nibble pairs -- and the pairs that meet the
// *16 nibbles are pre-divided by 16 (exact).  The common factor 2^24 is multiplied back with the group scale.
//
// Per 128-k unit the 8 MMAs accumulate sum_k x[k] * u4[k] exactly (fp32); the group's scale and zero are applied
// after the unit:  y += scale[n,g] * acc + zero[n,g] * sum_{k in unit} x[k],  with the activation sums precomputed once
// per CTA.  Scales and zeros travel in the same register ring as the weights, so their latency is hidden too.
// Work split, persistence and the fixed-order cross-warp reduction are those of the W8A8 GEMV.
#include <cstdlib>
#include <type_traits>

#include "w8a8.cuh"

namespace rwkvq {

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct I4Args {
    const __half* x;        // [M, ldx] fp16
    const uint8_t* w;       // [N, ldw] bytes
    const void* scales;     // [N, K/group] fp32 or fp16
    const float* zeros;     // [N, K/group] fp32 or null (zero = -8 * scale)
    __half* out;            // [M, ldo]
    int64_t ldx, ldw, ldo;
    int M, N, K, group, scale_f16, pitch, ngroups;
    int* status;                 // the library's per-device status word
    unsigned long long wait_ns;  // wall-time limit of the bounded waits
};

struct I4Slot {
    uint4 w;
    float s0, s1, z0, z1;   // scale / zero of weight rows n0+2t and n0+2t+1 for this unit's group
};

template <int D>
__global__ void __launch_bounds__(kThr, 2) gemv_int4_group_kernel(const I4Args a) {
    extern __shared__ __align__(16) uint8_t smem[];
    // layout: red[kWarps][4][32] floats | xsum[M][units] floats | xs[M][pitch] bytes (permuted fp16)
    const int units = a.K >> 7;
    float* red = reinterpret_cast<float*>(smem);
    float* xsum = red + kWarps * 4 * 32;
    uint8_t* xs = reinterpret_cast<uint8_t*>(xsum + ((a.M * units + 3) & ~3));

    griddep_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ntile = (a.N + 7) >> 3;
    const int tb = (int)((int64_t)ntile * blockIdx.x / gridDim.x), te = (int)((int64_t)ntile * (blockIdx.x + 1) / gridDim.x);
    const int upw = (units + kWarps - 1) / kWarps;
    const int nchunks = (upw + D - 1) / D;
    const int gshift = a.group == 128 ? 0 : 1;        // units per group: 1 (group 128) or 2 (group 256)

    auto fetch = [&](int tile, int c, int j) -> I4Slot {
        I4Slot s;
        s.w = make_uint4(0, 0, 0, 0);
        s.s0 = s.s1 = s.z0 = s.z1 = 0.f;
        const int u = warp + (c * D + j) * kWarps;
        if (tile >= te || u >= units) return s;
        const int n0 = tile << 3;
        s.w = ldg_stream(a.w + (int64_t)min(n0 + g, a.N - 1) * a.ldw + (u << 6) + 16 * t);
        const int grp = u >> gshift;
        const int64_t i0 = (int64_t)min(n0 + 2 * t, a.N - 1) * a.ngroups + grp, i1 = (int64_t)min(n0 + 2 * t + 1, a.N - 1) * a.ngroups + grp;
        if (a.scale_f16) {
            s.s0 = __half2float(__ldg(reinterpret_cast<const __half*>(a.scales) + i0));
            s.s1 = __half2float(__ldg(reinterpret_cast<const __half*>(a.scales) + i1));
        } else {
            s.s0 = __ldg(reinterpret_cast<const float*>(a.scales) + i0);
            s.s1 = __ldg(reinterpret_cast<const float*>(a.scales) + i1);
        }
        if (a.zeros) { s.z0 = __ldg(a.zeros + i0); s.z1 = __ldg(a.zeros + i1); }
        else { s.z0 = -8.f * s.s0; s.z1 = -8.f * s.s1; }
        return s;
    };

    I4Slot ring[D];
#pragma unroll
    for (int j = 0; j < D; ++j) ring[j] = fetch(tb, 0, j);

    griddep_wait();
    // ---- prologue: permuted fp16 activations and per-unit activation sums
    {
        const int kv = a.K >> 3;
        for (int r = 0; r < a.M; ++r) {
            const char* xr = reinterpret_cast<const char*>(a.x + (int64_t)r * a.ldx);
            for (int i = threadIdx.x; i < kv; i += kThr) {
                const uint4 v = *reinterpret_cast<const uint4*>(xr + (size_t)i * 16);
                // halves h0..h7 -> (h0,h4), (h1,h5)/16, (h2,h6), (h3,h7)/16
                const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
                uint4 p;
                p.x = __byte_perm(v.x, v.z, 0x5410);
                p.y = __byte_perm(v.x, v.z, 0x7632);
                p.z = __byte_perm(v.y, v.w, 0x5410);
                p.w = __byte_perm(v.y, v.w, 0x7632);
                *reinterpret_cast<__half2*>(&p.y) = __hmul2(*reinterpret_cast<__half2*>(&p.y), sixteenth);
                *reinterpret_cast<__half2*>(&p.w) = __hmul2(*reinterpret_cast<__half2*>(&p.w), sixteenth);
                *reinterpret_cast<uint4*>(xs + (size_t)r * a.pitch + (size_t)i * 16) = p;
            }
        }
        __syncthreads();
        for (int i = warp; i < a.M * units; i += kWarps) {
            const int r = i / units, u = i - r * units;
            const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(a.x + (int64_t)r * a.ldx) + ((size_t)u << 8) + lane * 8);   // 4 halves per lane
            const float2 f0 = cvt2<RWKVQ_F16>(v.x), f1 = cvt2<RWKVQ_F16>(v.y);
            const float sum = warp_sum((f0.x + f0.y) + (f1.x + f1.y));
            if (lane == 0) xsum[i] = sum;
        }
        __syncthreads();
    }

    for (int tile = tb; tile < te; ++tile) {
        const int n0 = tile << 3;
        float tot[4] = {0.f, 0.f, 0.f, 0.f};
        for (int ch = 0; ch < nchunks; ++ch) {
            const bool last = ch + 1 == nchunks;
#pragma unroll
            for (int j = 0; j < D; ++j) {
                const I4Slot sl = ring[j];
                ring[j] = fetch(last ? tile + 1 : tile, last ? 0 : ch + 1, j);
                const int u = warp + (ch * D + j) * kWarps;
                if (u < units) {                      // uniform within the warp
                    // four independent accumulators (one per 32-bit word): the MMAs of a unit do not wait on each other
                    float c4[4][4];
                    const uint32_t wd[4] = {sl.w.x, sl.w.y, sl.w.z, sl.w.w};
                    const size_t koff = ((size_t)u << 8) + (size_t)t * 64;          // bytes into the fp16 row
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        c4[i][0] = c4[i][1] = c4[i][2] = c4[i][3] = 0.f;
                        uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0;
                        if (g < a.M) a0 = *reinterpret_cast<const uint4*>(xs + (size_t)g * a.pitch + koff + i * 16);
                        if (g + 8 < a.M) a1 = *reinterpret_cast<const uint4*>(xs + (size_t)(g + 8) * a.pitch + koff + i * 16);
                        const uint32_t hi = wd[i] >> 8;
                        mma_f16(c4[i], a0.x, a1.x, a0.y, a1.y, wd[i] & 0x000F000Fu, wd[i] & 0x00F000F0u);
                        mma_f16(c4[i], a0.z, a1.z, a0.w, a1.w, hi & 0x000F000Fu, hi & 0x00F000F0u);
                    }
                    float c[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) c[q] = (c4[0][q] + c4[1][q]) + (c4[2][q] + c4[3][q]);
                    const float xs0 = g < a.M ? xsum[g * units + u] : 0.f, xs1 = g + 8 < a.M ? xsum[(g + 8) * units + u] : 0.f;
                    const float e0 = sl.s0 * 16777216.f, e1 = sl.s1 * 16777216.f;     // undo the 2^-24 of the subnormals
                    tot[0] += e0 * c[0] + sl.z0 * xs0;
                    tot[1] += e1 * c[1] + sl.z1 * xs0;
                    tot[2] += e0 * c[2] + sl.z0 * xs1;
                    tot[3] += e1 * c[3] + sl.z1 * xs1;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) red[(warp * 4 + j) * 32 + lane] = tot[j];
        __syncthreads();
        if (threadIdx.x < 128) {
            const int j = threadIdx.x >> 5, l = threadIdx.x & 31;
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += red[(w * 4 + j) * 32 + l];
            const int m = (l >> 2) + ((j & 2) ? 8 : 0), n = n0 + 2 * (l & 3) + (j & 1);
            if (m < a.M && n < a.N) a.out[(int64_t)m * a.ldo + n] = __float2half_rn(s);
        }
        __syncthreads();
    }
}

// ---- fast path: group 128, fp32 scales, K a multiple of 512.
//
// Written like the W8A8 decode kernel (instruction count, per-warp cp.async rings, host-side tile split), with the
// operand roles of the MMA swapped: the WEIGHTS are the 16-row A operand and up to 8 tokens the B operand, so one
// m16n8k16 covers 16 weight rows x 16 k -- half the MMAs per byte -- and a lane's accumulators belong to the two
// weight rows (g and g+8) it loads, so it applies the scales and zeros of exactly those rows.
//
// A warp owns 16 weight rows over a contiguous K range.  Unit = 128 k (one group): lane (g, t) copies
// W[n0+g][..] and W[n0+g+8][..], 16 bytes (32 nibbles, k = 32t .. 32t+31 of the unit) each.  A chunk is 4 units
// plus the 4 scales and 4 zeros of the 16 rows (lane t = 0..3 of row pair g copies scales g, scales g+8, zeros g,
// zeros g+8 as one 16-byte vector each).  A 32-bit word of each row gives the A registers of two MMAs (masks
// 0x000F000F / 0x00F000F0 on the word and on the word >> 8, see the file header); the activations of token
// min(g, M-1) are read with the matching permutation, tokens beyond M feed accumulator columns that are never stored.
// In shared memory the 16 vectors of a unit are ordered [word q][lane t] (fast-path kernel only).
// NT: token tiles of 8 (M <= 8 NT).  S: ring stages per warp.
constexpr int kI4D = 4;                                   // units per chunk
constexpr int kI4Stage = kI4D * 1024 + 512;               // bytes per warp and stage: weights + scales/zeros

struct I4FastArgs {
    I4Args b;
    int lgR, tq, trem;            // log2 of the 16-row tiles per round; tiles per CTA (quotient, remainder)
    float* part;                  // SPLIT: fp32 partial sums [slices][M][N]
    int kslice;                   // SPLIT: k per slice (b.K holds the same value; b.ngroups stays the row pitch of the scales)
};

// SPLIT: K is cut into gridDim.y slices (the activation tile of one slice fits beside a ring with two CTAs per SM);
// CTA (x, y) works on columns [y * kslice, (y + 1) * kslice) of its row tiles and stores fp32 partial sums, which
// i4_reduce_kernel adds in slice order.  A separate instantiation: the single-launch decode path carries none of it.
template <int NT, int S, bool SPLIT = false>
__global__ void __launch_bounds__(kThr, 2) gemv_int4_g128_kernel(const I4FastArgs fa) {
    const I4Args& a = fa.b;
    const int64_t koff = SPLIT ? (int64_t)blockIdx.y * fa.kslice : 0;
    const uint8_t* const wbase = a.w + (koff >> 1);
    const __half* const xbase = a.x + koff;
    const float* const zbase = a.zeros ? a.zeros + (koff >> 7) : nullptr;
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: red[2][kWarps][NT*4][32] floats | ring[kWarps][S][kI4Stage] | xbar (128 B) | xsum[M][units] floats | xs[M][pitch]
    const int units = a.K >> 7;
    float* red = reinterpret_cast<float*>(smem);
    uint8_t* ring = smem + 2 * kWarps * NT * 4 * 32 * 4;
    uint64_t* xbar = reinterpret_cast<uint64_t*>(ring + (size_t)kWarps * S * kI4Stage);          // 128 bytes reserved
    float* xsum = reinterpret_cast<float*>(ring + (size_t)kWarps * S * kI4Stage + 128);
    uint8_t* xs = reinterpret_cast<uint8_t*>(xsum + ((a.M * units + 31) & ~31));       // 128-byte boundary

    griddep_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int cb = blockIdx.x;
    const int tb = cb * fa.tq + min(cb, fa.trem), te = tb + fa.tq + (cb < fa.trem ? 1 : 0);   // this CTA's 16-row tiles
    const int lgR = fa.lgR, R = 1 << lgR, lgKS = 3 - lgR, KS = 1 << lgKS;
    const int slot = warp >> lgKS, ks = warp & (KS - 1);
    const int rounds = (te - tb + R - 1) >> lgR;
    const int upw = (((units + KS - 1) >> lgKS) + 3) & ~3;           // units per warp and tile, whole chunks
    const int ub = ks * upw, ue = min(ub + upw, units);
    const int nch = max(ue - ub, 0) >> 2;
    const int my_rounds = (nch > 0 && te - tb > slot) ? ((te - tb - slot + R - 1) >> lgR) : 0;
    uint8_t* my_ring = ring + (size_t)warp * S * kI4Stage;
    const uint32_t my_ring_s = (uint32_t)__cvta_generic_to_shared(my_ring);
    const float* scales = reinterpret_cast<const float*>(a.scales) + (koff >> 7);
    const bool has_z = a.zeros != nullptr;

    // producer: per chunk 8 weight copies per lane and one scale / zero vector
    int p_round = 0, p_ch = 0, p_stage = 0;
    const uint8_t *p_w0 = wbase, *p_w1 = wbase;
    const float* p_sz = scales;
    const bool sz_on = t < 2 || has_z;
    auto set_rows = [&](int round) {
        const int n0 = (tb + round * R + slot) << 4;
        const int r0 = min(n0 + g, a.N - 1), r1 = min(n0 + g + 8, a.N - 1);
        p_w0 = wbase + (int64_t)r0 * a.ldw + ub * 64 + 16 * t;
        p_w1 = wbase + (int64_t)r1 * a.ldw + ub * 64 + 16 * t;
        p_sz = ((t & 2) ? zbase : scales) + (int64_t)((t & 1) ? r1 : r0) * a.ngroups + ub;
    };
    if (my_rounds > 0) set_rows(0);
    auto issue = [&]() {
        if (p_round < my_rounds) {
            const uint32_t dst = my_ring_s + p_stage * kI4Stage;
#pragma unroll
            for (int j = 0; j < kI4D; ++j) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + j * 1024 + lane * 16), "l"(p_w0 + j * 64) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + j * 1024 + 512 + lane * 16), "l"(p_w1 + j * 64) : "memory");
            }
            if (sz_on) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + kI4D * 1024 + (t * 8 + g) * 16), "l"(p_sz) : "memory");
            p_w0 += kI4D * 64;
            p_w1 += kI4D * 64;
            p_sz += kI4D;
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

    // this lane's token rows of the activation tile and of the per-unit activation sums (tokens beyond M read M-1)
    const uint8_t* xb0[NT];
    const float *xq0[NT], *xq1[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        xb0[i] = xs + min(i * 8 + g, a.M - 1) * a.pitch + ub * 256 + t * 16;
        xq0[i] = xsum + min(i * 8 + 2 * t, a.M - 1) * units + ub;
        xq1[i] = xsum + min(i * 8 + 2 * t + 1, a.M - 1) * units + ub;
    }

    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(xbar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    griddep_wait();
    {   // prologue, one read of the activations.  Thread 0 fetches the raw fp16 rows with bulk copies INTO the tile
        // (a raw row and its permuted copy have the same size; completion on an mbarrier, independent of the ring's
        // cp.async groups); a short loop then permutes in place (odd pairs / 16) and sums each unit's 16 vectors
        // over the 16 lanes that hold them.  A wait that runs out (seconds) falls back to reading global memory.
        const int kv = a.K >> 3;
        const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
        if (threadIdx.x == 0) {
            const uint32_t b = (uint32_t)__cvta_generic_to_shared(xbar);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"((uint32_t)(a.M * a.K * 2)) : "memory");
#pragma unroll 1
            for (int r = 0; r < a.M; ++r)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"((uint32_t)__cvta_generic_to_shared(xs + (size_t)r * a.pitch)), "l"(xbase + (int64_t)r * a.ldx),
                               "r"((uint32_t)(a.K * 2)), "r"(b) : "memory");
        }
        if (!w8_staged_or_report(xbar, a.status, a.wait_ns)) {     // reported: drain the weight ring and stop
            cp_async_wait<0>();
            return;
        }
#pragma unroll 1
        for (int r = 0; r < a.M; ++r) {
            uint8_t* row = xs + (size_t)r * a.pitch;
            const char* src = reinterpret_cast<const char*>(row);
#pragma unroll 1
            for (int i = threadIdx.x; i - lane < kv; i += kThr) {          // kv is a multiple of 16: half-warps are whole
                const bool on = i < kv;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (on) v = *reinterpret_cast<const uint4*>(src + (size_t)i * 16);
                uint4 p;
                p.x = __byte_perm(v.x, v.z, 0x5410);
                p.y = __byte_perm(v.x, v.z, 0x7632);
                p.z = __byte_perm(v.y, v.w, 0x5410);
                p.w = __byte_perm(v.y, v.w, 0x7632);
                *reinterpret_cast<__half2*>(&p.y) = __hmul2(*reinterpret_cast<__half2*>(&p.y), sixteenth);
                *reinterpret_cast<__half2*>(&p.w) = __hmul2(*reinterpret_cast<__half2*>(&p.w), sixteenth);
                // Inside a unit (16 vectors, held by 16 neighbouring lanes) vector 4t+q goes to place 4q+t, so that the
                // four t-lanes of a quarter-warp later read 64 contiguous bytes (no bank conflict).  In place: every
                // lane has read its vector before any lane of the warp writes.
                __syncwarp();
                if (on) *reinterpret_cast<uint4*>(row + (size_t)((i & ~15) | ((i & 3) << 2) | ((i >> 2) & 3)) * 16) = p;
                const float2 f0 = cvt2<RWKVQ_F16>(v.x), f1 = cvt2<RWKVQ_F16>(v.y), f2 = cvt2<RWKVQ_F16>(v.z), f3 = cvt2<RWKVQ_F16>(v.w);
                float s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (on && (lane & 15) == 0) xsum[r * units + (i >> 4)] = s;
            }
        }
        __syncthreads();
    }

    int stage = 0;
    for (int r = 0; r < rounds; ++r) {
        float tot[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i) tot[i][0] = tot[i][1] = tot[i][2] = tot[i][3] = 0.f;
        if (r < my_rounds) {
            const uint8_t* xb[NT];
            const float *q0[NT], *q1[NT];
#pragma unroll
            for (int i = 0; i < NT; ++i) { xb[i] = xb0[i]; q0[i] = xq0[i]; q1[i] = xq1[i]; }
            for (int ch = 0; ch < nch; ++ch) {
                issue();
                cp_async_wait<S - 1>();
                __syncwarp();                              // the scale / zero vectors are read across lanes
                const uint8_t* st = my_ring + stage * kI4Stage;
                const float4 sg = *reinterpret_cast<const float4*>(st + kI4D * 1024 + (0 * 8 + g) * 16);
                const float4 sh = *reinterpret_cast<const float4*>(st + kI4D * 1024 + (1 * 8 + g) * 16);
                float4 zg, zh;
                if (has_z) {
                    zg = *reinterpret_cast<const float4*>(st + kI4D * 1024 + (2 * 8 + g) * 16);
                    zh = *reinterpret_cast<const float4*>(st + kI4D * 1024 + (3 * 8 + g) * 16);
                } else {
                    zg = make_float4(-8.f * sg.x, -8.f * sg.y, -8.f * sg.z, -8.f * sg.w);
                    zh = make_float4(-8.f * sh.x, -8.f * sh.y, -8.f * sh.z, -8.f * sh.w);
                }
                const float sgv[4] = {sg.x, sg.y, sg.z, sg.w}, shv[4] = {sh.x, sh.y, sh.z, sh.w};
                const float zgv[4] = {zg.x, zg.y, zg.z, zg.w}, zhv[4] = {zh.x, zh.y, zh.z, zh.w};
#pragma unroll
                for (int j = 0; j < kI4D; ++j) {
                    const uint4 wg = *reinterpret_cast<const uint4*>(st + j * 1024 + lane * 16);
                    const uint4 wh = *reinterpret_cast<const uint4*>(st + j * 1024 + 512 + lane * 16);
                    const uint32_t wgw[4] = {wg.x, wg.y, wg.z, wg.w}, whw[4] = {wh.x, wh.y, wh.z, wh.w};
                    const float eg = sgv[j] * 16777216.f, eh = shv[j] * 16777216.f;     // undo the 2^-24 of the subnormals
#pragma unroll
                    for (int i = 0; i < NT; ++i) {
                        float ca[4] = {0.f, 0.f, 0.f, 0.f}, cb2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 bx = *reinterpret_cast<const uint4*>(xb[i] + j * 256 + q * 64);
                            const uint32_t hg = wgw[q] >> 8, hh = whw[q] >> 8;
                            mma_f16((q & 1) ? cb2 : ca, wgw[q] & 0x000F000Fu, whw[q] & 0x000F000Fu, wgw[q] & 0x00F000F0u, whw[q] & 0x00F000F0u, bx.x, bx.y);
                            mma_f16((q & 1) ? cb2 : ca, hg & 0x000F000Fu, hh & 0x000F000Fu, hg & 0x00F000F0u, hh & 0x00F000F0u, bx.z, bx.w);
                        }
                        const float x0 = q0[i][j], x1 = q1[i][j];
                        tot[i][0] += eg * (ca[0] + cb2[0]) + zgv[j] * x0;
                        tot[i][1] += eg * (ca[1] + cb2[1]) + zgv[j] * x1;
                        tot[i][2] += eh * (ca[2] + cb2[2]) + zhv[j] * x0;
                        tot[i][3] += eh * (ca[3] + cb2[3]) + zhv[j] * x1;
                    }
                }
                __syncwarp();                              // all lanes have read this stage before it is refilled
#pragma unroll
                for (int i = 0; i < NT; ++i) { xb[i] += kI4D * 256; q0[i] += kI4D; q1[i] += kI4D; }
                if (++stage == S) stage = 0;
            }
        }
        const int tile = tb + r * R + slot;
        bool store = tile < te;
        if (KS > 1) {
            float* rb = red + (size_t)(r & 1) * kWarps * NT * 4 * 32;
            if (ks > 0) {
#pragma unroll
                for (int i = 0; i < NT; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) rb[((warp * NT + i) * 4 + j) * 32 + lane] = tot[i][j];
            }
            __syncthreads();
            store = store && ks == 0;
            if (store) {
                for (int kk = 1; kk < KS; ++kk)
#pragma unroll
                    for (int i = 0; i < NT; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) tot[i][j] += rb[(((warp + kk) * NT + i) * 4 + j) * 32 + lane];
            }
        }
        if (store) {
            // lane (g, t): weight rows n0+g (values 0, 1) and n0+g+8 (values 2, 3), tokens 8i+2t and 8i+2t+1
            const int n0 = tile << 4;
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int m = i * 8 + 2 * t + (j & 1), n = n0 + g + ((j & 2) ? 8 : 0);
                    if (m < a.M && n < a.N) {
                        if constexpr (SPLIT) fa.part[((int64_t)blockIdx.y * a.M + m) * a.N + n] = tot[i][j];
                        else a.out[(int64_t)m * a.ldo + n] = __float2half_rn(tot[i][j]);
                    }
                }
        }
    }
    cp_async_wait<0>();
}

// out[m][n] = fp16(sum over slices, in slice order, of part[s][m][n])
__global__ void __launch_bounds__(256) i4_reduce_kernel(const float* __restrict__ part, int slices, int M, int N, __half* out, int64_t ldo) {
    griddep_launch_dependents();
    griddep_wait();
    const int64_t total = (int64_t)M * N;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
        float v = 0.f;
        for (int sl = 0; sl < slices; ++sl) v += __ldcg(part + (int64_t)sl * total + i);
        const int64_t m = i / N;
        out[m * ldo + (i - m * N)] = __float2half_rn(v);
    }
}

static size_t i4_fast_smem(int NT, int S, int M, int K) {
    const int units = K / 128;
    return (size_t)2 * kWarps * NT * 4 * 32 * 4 + (size_t)kWarps * S * kI4Stage + 128 + (size_t)((M * units + 31) & ~31) * 4 + (size_t)M * (2 * K + 16);
}

template <typename Kern, typename Args>
static int32_t launch_i4(Kern kern, Args& a, size_t smem, cudaStream_t st, int64_t tiles, bool fast, int slices = 1) {
    int per_sm = 0;
    const int32_t rc = kernel_plan(reinterpret_cast<const void*>(kern), kThr, smem, 224 * 1024, &per_sm, "gemv_int4_group");
    if (rc != RWKVQ_OK) return rc;
    cudaError_t e;
    const int grid = (int)std::min<int64_t>(tiles, std::max<int64_t>(1, (int64_t)sm_count() * std::min(per_sm, 2) / slices));
    if constexpr (std::is_same<Args, I4FastArgs>::value) {
        a.b.status = device_status_ptr();
        a.b.wait_ns = wait_limit_ns();
        a.tq = (int)(tiles / grid);
        a.trem = (int)(tiles % grid);
        const int tpc = (int)((tiles + grid - 1) / grid);
        a.lgR = 0;
        while ((1 << a.lgR) < kWarps && (1 << a.lgR) < tpc) ++a.lgR;
    }
    (void)fast;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid, (unsigned)slices);
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
        return fail(RWKVQ_E_LAUNCH, "gemv_int4_group: %s", cudaGetErrorString(e));
    }
    return check_launch("gemv_int4_group");
}

// K slices of the split form: the fewest (a power of two, whole 512-k chunks per slice) whose activation tile is at
// most about 64 KB, which leaves room for a three- or four-stage weight ring; 1 = the single launch already has that;
// 0 = not even 512-k slices fit.
static int i4_slices(int M, int64_t N, int K) {
    // measured on the 7.2B shapes: a block that still fits one launch is better left whole when the matrix has many
    // row tiles (N = 16384: 21 us whole, 23 us split at 16 rows); with few (N = 4096) the split wins (11.8 -> 10.8 us)
    if (N > 8192 && i4_fast_smem(M <= 8 ? 1 : 2, 2, M, K) <= 224 * 1024) return 1;
    static const size_t tile_max = std::getenv("RWKVQ_INT4_SPLIT_TILE") ? (size_t)std::atoll(std::getenv("RWKVQ_INT4_SPLIT_TILE")) : 66 * 1024;
    int sl = 1;
    while (sl < 32 && (size_t)M * (2 * (size_t)(K / sl) + 16) > tile_max && (K / (sl * 2)) % 512 == 0 && K / (sl * 2) >= 512) sl <<= 1;
    return i4_fast_smem(M <= 8 ? 1 : 2, 2, M, K / sl) <= 224 * 1024 ? sl : 0;
}

template <int NT>
static int32_t launch_i4_split(I4FastArgs& fa, cudaStream_t st, int slices) {
    constexpr size_t kTwo = 110 * 1024, kMax = 224 * 1024;
    const I4Args& a = fa.b;
    const int64_t tiles = (a.N + 15) / 16;
    const size_t s4 = i4_fast_smem(NT, 4, a.M, a.K), s3 = i4_fast_smem(NT, 3, a.M, a.K), s2 = i4_fast_smem(NT, 2, a.M, a.K);
    if (s2 <= kTwo) return launch_i4(gemv_int4_g128_kernel<NT, 2, true>, fa, s2, st, tiles, true, slices);
    if (s4 <= kMax) return launch_i4(gemv_int4_g128_kernel<NT, 4, true>, fa, s4, st, tiles, true, slices);
    if (s3 <= kMax) return launch_i4(gemv_int4_g128_kernel<NT, 3, true>, fa, s3, st, tiles, true, slices);
    return launch_i4(gemv_int4_g128_kernel<NT, 2, true>, fa, s2, st, tiles, true, slices);
}

template <int NT>
static int32_t launch_i4_fast(const I4Args& a, cudaStream_t st, bool* done) {
    constexpr size_t kTwo = 110 * 1024, kMax = 224 * 1024;
    I4FastArgs fa{};
    fa.b = a;
    const int64_t tiles = (a.N + 15) / 16;
    const size_t s4 = i4_fast_smem(NT, 4, a.M, a.K), s3 = i4_fast_smem(NT, 3, a.M, a.K), s2 = i4_fast_smem(NT, 2, a.M, a.K);
    *done = true;
    if (s2 <= kTwo) return launch_i4(gemv_int4_g128_kernel<NT, 2>, fa, s2, st, tiles, true);
    if (s4 <= kMax) return launch_i4(gemv_int4_g128_kernel<NT, 4>, fa, s4, st, tiles, true);
    if (s3 <= kMax) return launch_i4(gemv_int4_g128_kernel<NT, 3>, fa, s3, st, tiles, true);
    if (s2 <= kMax) return launch_i4(gemv_int4_g128_kernel<NT, 2>, fa, s2, st, tiles, true);
    *done = false;      // the activation tile leaves no room for a ring: the register-ring kernel takes the call
    return RWKVQ_OK;
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

/* K-split form of rwkvq_gemv_int4_group for blocks of activations that do not fit beside a weight ring with two CTAs
 * per SM (many rows, long rows): group 128, fp32 scales, K a multiple of 512, M <= 16.  Two launches: the streaming
 * kernel over (row tiles) x (K slices) storing fp32 partial sums into `workspace`, then their sum in slice order.
 * rwkvq_gemv_int4_ksplit_slices(M, N, K): slices this form would use (1: the plain entry does the same in one launch; 0: unsupported);
 * workspace of slices * M * N * 4 bytes, 16-byte aligned, contents irrelevant. */
int32_t rwkvq_gemv_int4_ksplit_slices(int64_t M, int64_t N, int64_t K) {
    if (M < 1 || M > 16 || N < 1 || K < 512 || K % 512) return 0;
    return i4_slices((int)M, N, (int)K);
}

int32_t rwkvq_gemv_int4_group_ksplit(const void* x_f16, int64_t ldx, const uint8_t* packed, int64_t ldw, const float* scales,
                                     const float* zeros, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                                     void* workspace, int64_t workspace_bytes, void* stream) {
    const char* who = "gemv_int4_group_ksplit";
    RWKVQ_REQUIRE(x_f16 && packed && scales && out_f16, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(M >= 0 && M <= 16 && N >= 0 && K >= 0, RWKVQ_E_SHAPE, "%s: M=%lld (0..16), N=%lld, K=%lld", who, (long long)M, (long long)N, (long long)K);
    if (M == 0 || N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(K >= 512 && K % 512 == 0, RWKVQ_E_SHAPE, "%s: K=%lld must be a multiple of 512", who, (long long)K);
    RWKVQ_REQUIRE(aligned16(packed) && ldw % 16 == 0 && ldw >= K / 2, RWKVQ_E_ALIGN, "%s: packed rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(aligned16(x_f16) && ldx % 8 == 0 && ldx >= K, RWKVQ_E_ALIGN, "%s: activation rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(aligned16(scales) && (zeros == nullptr || aligned16(zeros)), RWKVQ_E_ALIGN, "%s: scales / zeros must be 16-byte aligned", who);
    RWKVQ_REQUIRE(ldo >= N, RWKVQ_E_SHAPE, "%s: ldo < N", who);
    const int slices = i4_slices((int)M, N, (int)K);
    RWKVQ_REQUIRE(slices >= 1, RWKVQ_E_SHAPE, "%s: %lld rows of %lld do not fit shared memory even in 512-k slices", who, (long long)M, (long long)K);
    RWKVQ_REQUIRE(workspace && aligned16(workspace) && workspace_bytes >= (int64_t)slices * M * N * 4, RWKVQ_E_WORKSPACE,
                  "%s: workspace of %lld bytes needed", who, (long long)slices * M * N * 4);
    cudaStream_t st = (cudaStream_t)stream;
    I4FastArgs fa{};
    I4Args& a = fa.b;
    a.x = (const __half*)x_f16; a.w = packed; a.scales = scales; a.zeros = zeros; a.out = (__half*)out_f16;
    a.ldx = ldx; a.ldw = ldw; a.ldo = ldo; a.M = (int)M; a.N = (int)N; a.K = (int)(K / slices); a.group = 128; a.scale_f16 = 0;
    a.pitch = (int)(2 * (K / slices) + 16); a.ngroups = (int)(K / 128);
    fa.part = reinterpret_cast<float*>(workspace);
    fa.kslice = (int)(K / slices);
    int32_t rc = M <= 8 ? launch_i4_split<1>(fa, st, slices) : launch_i4_split<2>(fa, st, slices);
    if (rc != RWKVQ_OK) return rc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)std::min<int64_t>((M * N + 255) / 256, 2 * (int64_t)sm_count()));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl() ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, i4_reduce_kernel, (const float*)fa.part, slices, (int)M, (int)N, (__half*)out_f16, ldo);
    if (e != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
    }
    return check_launch(who);
}

int64_t rwkvq_gemv_int4_group_smem_bytes(int64_t M, int64_t K) {
    const int64_t units = K / 128, pitch = 2 * K + 16;
    return kWarps * 4 * 32 * 4 + ((M * units + 3) & ~int64_t(3)) * 4 + M * pitch;
}

int32_t rwkvq_gemv_int4_group(const void* x_f16, int64_t ldx, const uint8_t* packed, int64_t ldw, const void* scales,
                              const float* zeros, int32_t scale_is_f16, int32_t group, void* out_f16, int64_t ldo, int64_t M,
                              int64_t N, int64_t K, void* stream) {
    const char* who = "gemv_int4_group";
    RWKVQ_REQUIRE(x_f16 && packed && scales && out_f16, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(M >= 0 && N >= 0 && K >= 0, RWKVQ_E_SHAPE, "%s: negative size", who);
    RWKVQ_REQUIRE(M <= 16, RWKVQ_E_SHAPE, "%s: M=%lld > 16", who, (long long)M);
    RWKVQ_REQUIRE(K % 128 == 0 && (group == 128 || group == 256) && K % group == 0, RWKVQ_E_SHAPE,
                  "%s: needs K %% 128 == 0 and group 128 or 256 (K=%lld, group=%d); other layouts: gemv_int4_group_generic", who, (long long)K, group);
    RWKVQ_REQUIRE(aligned16(packed) && ldw % 16 == 0 && ldw >= K / 2, RWKVQ_E_ALIGN, "%s: packed rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(aligned16(x_f16) && ldx % 8 == 0 && ldx >= K, RWKVQ_E_ALIGN, "%s: activation rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(ldo >= N, RWKVQ_E_SHAPE, "%s: ldo < N", who);
    if (M == 0 || N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(K > 0, RWKVQ_E_SHAPE, "%s: K=0", who);
    const size_t smem = (size_t)rwkvq_gemv_int4_group_smem_bytes(M, K);
    RWKVQ_REQUIRE(smem <= 200 * 1024, RWKVQ_E_SHAPE, "%s: M*K = %lld*%lld does not fit shared memory; use gemv_int4_group_generic", who,
                  (long long)M, (long long)K);
    I4Args a{};
    a.x = (const __half*)x_f16; a.w = packed; a.scales = scales; a.zeros = zeros; a.out = (__half*)out_f16;
    a.ldx = ldx; a.ldw = ldw; a.ldo = ldo; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.group = group; a.scale_f16 = scale_is_f16;
    a.pitch = (int)(2 * K + 16); a.ngroups = (int)(K / group);
    const char* env = std::getenv("RWKVQ_INT4_FAST");
    const bool fast = K % 512 == 0 && group == 128 && !scale_is_f16 && !(env && env[0] == '0')
                      && ((uintptr_t)scales & 15) == 0 && (zeros == nullptr || ((uintptr_t)zeros & 15) == 0);
    cudaStream_t st = (cudaStream_t)stream;
    if (fast) {
        bool done = false;
        const int32_t rc = M <= 8 ? launch_i4_fast<1>(a, st, &done) : launch_i4_fast<2>(a, st, &done);
        if (done) return rc;
        // the activation tile of all M rows leaves no room for a weight ring: run blocks of as many rows as fit
        int rows = 8;
        while (rows > 0 && i4_fast_smem(1, 2, rows, a.K) > 224 * 1024) --rows;
        if (rows > 0) {
            for (int r0 = 0; r0 < (int)M; r0 += rows) {
                I4Args b = a;
                b.M = std::min(rows, (int)M - r0);
                b.x = a.x + (int64_t)r0 * a.ldx;
                b.out = a.out + (int64_t)r0 * a.ldo;
                const int32_t rcb = launch_i4_fast<1>(b, st, &done);
                if (rcb != RWKVQ_OK || !done) return rcb != RWKVQ_OK ? rcb : fail(RWKVQ_E_SHAPE, "%s: internal: row block does not fit", who);
            }
            return RWKVQ_OK;
        }
    }
    const int64_t tiles = (N + 7) / 8;
    return (K / 128 > 4 * kWarps) ? launch_i4(gemv_int4_group_kernel<8>, a, smem, st, tiles, false)
                                  : launch_i4(gemv_int4_group_kernel<4>, a, smem, st, tiles, false);
}

}  // extern "C"
