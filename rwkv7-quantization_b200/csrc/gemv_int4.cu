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

#include "w8a8.cuh"

namespace rwkvq {

struct I4Args {
    const __half* x;        // [M, ldx] fp16
    const uint8_t* w;       // [N, ldw] bytes
    const void* scales;     // [N, K/group] fp32 or fp16
    const float* zeros;     // [N, K/group] fp32 or null (zero = -8 * scale)
    __half* out;            // [M, ldo]
    int64_t ldx, ldw, ldo;
    int M, N, K, group, scale_f16, pitch, ngroups;
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

// ---- fast path: K a multiple of 4096, group 128, fp32 scales (zeros optional).  Each warp owns a CONTIGUOUS run of
// units of its 8 rows, so the scales / zeros of four units are one 128-bit load per row, every address in the unrolled
// body is a base pointer plus a compile-time offset, and a row streams 256 contiguous bytes per chunk.
struct I4Quad {
    uint4 w[4];
    float4 s0, s1, z0, z1;      // scales / zeros of rows n0+2t and n0+2t+1 for the chunk's four groups
};

__global__ void __launch_bounds__(kThr, 2) gemv_int4_g128_kernel(const I4Args a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int units = a.K >> 7;
    float* red = reinterpret_cast<float*>(smem);
    float* xsum = red + kWarps * 4 * 32;
    uint8_t* xs = reinterpret_cast<uint8_t*>(xsum + ((a.M * units + 3) & ~3));

    griddep_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ntile = (a.N + 7) >> 3;
    const int tb = (int)((int64_t)ntile * blockIdx.x / gridDim.x), te = (int)((int64_t)ntile * (blockIdx.x + 1) / gridDim.x);
    const int upw = units >> 3, nchunks = upw >> 2;           // units per warp (multiple of 4), chunks of 4 units
    const float* scales = reinterpret_cast<const float*>(a.scales);

    auto fetch = [&](int tile, int c) -> I4Quad {
        I4Quad q;
        const int n0 = tile << 3;
        const uint8_t* wp = a.w + (int64_t)min(n0 + g, a.N - 1) * a.ldw + ((warp * upw + c * 4) << 6) + 16 * t;
#pragma unroll
        for (int j = 0; j < 4; ++j) q.w[j] = ldg_stream(wp + j * 64);
        const int64_t i0 = (int64_t)min(n0 + 2 * t, a.N - 1) * a.ngroups + warp * upw + c * 4;
        const int64_t i1 = (int64_t)min(n0 + 2 * t + 1, a.N - 1) * a.ngroups + warp * upw + c * 4;
        q.s0 = __ldg(reinterpret_cast<const float4*>(scales + i0));
        q.s1 = __ldg(reinterpret_cast<const float4*>(scales + i1));
        if (a.zeros) {
            q.z0 = __ldg(reinterpret_cast<const float4*>(a.zeros + i0));
            q.z1 = __ldg(reinterpret_cast<const float4*>(a.zeros + i1));
        } else {
            q.z0 = make_float4(-8.f * q.s0.x, -8.f * q.s0.y, -8.f * q.s0.z, -8.f * q.s0.w);
            q.z1 = make_float4(-8.f * q.s1.x, -8.f * q.s1.y, -8.f * q.s1.z, -8.f * q.s1.w);
        }
        return q;
    };
    I4Quad cur = fetch(min(tb, max(te - 1, 0)), 0);

    griddep_wait();
    {   // prologue: permuted fp16 activations (odd pairs / 16) and per-unit activation sums
        const int kv = a.K >> 3;
        const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
        for (int r = 0; r < a.M; ++r) {
            const char* xr = reinterpret_cast<const char*>(a.x + (int64_t)r * a.ldx);
            for (int i = threadIdx.x; i < kv; i += kThr) {
                const uint4 v = *reinterpret_cast<const uint4*>(xr + (size_t)i * 16);
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
        for (int i = warp; i < a.M * units; i += kWarps) {
            const int r = i / units, u = i - r * units;
            const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(a.x + (int64_t)r * a.ldx) + ((size_t)u << 8) + lane * 8);
            const float2 f0 = cvt2<RWKVQ_F16>(v.x), f1 = cvt2<RWKVQ_F16>(v.y);
            const float sum = warp_sum((f0.x + f0.y) + (f1.x + f1.y));
            if (lane == 0) xsum[i] = sum;
        }
        __syncthreads();
    }
    // this lane's activation rows (g and g + 8) at its warp's first unit
    const uint8_t* xr0 = g < a.M ? xs + (size_t)g * a.pitch + ((size_t)(warp * upw) << 8) + t * 64 : nullptr;
    const uint8_t* xr1 = g + 8 < a.M ? xs + (size_t)(g + 8) * a.pitch + ((size_t)(warp * upw) << 8) + t * 64 : nullptr;
    const float* xs0p = xsum + (g < a.M ? g : 0) * units + warp * upw;
    const float* xs1p = xsum + (g + 8 < a.M ? g + 8 : 0) * units + warp * upw;
    const float m0 = g < a.M ? 1.f : 0.f, m1 = g + 8 < a.M ? 1.f : 0.f;

    for (int tile = tb; tile < te; ++tile) {
        float tot[4] = {0.f, 0.f, 0.f, 0.f};
        for (int ch = 0; ch < nchunks; ++ch) {
            const I4Quad q = cur;
            const bool last = ch + 1 == nchunks;
            if (!last || tile + 1 < te) cur = fetch(last ? tile + 1 : tile, last ? 0 : ch + 1);
            const float sc0[4] = {q.s0.x, q.s0.y, q.s0.z, q.s0.w}, sc1[4] = {q.s1.x, q.s1.y, q.s1.z, q.s1.w};
            const float zr0[4] = {q.z0.x, q.z0.y, q.z0.z, q.z0.w}, zr1[4] = {q.z1.x, q.z1.y, q.z1.z, q.z1.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float ca[4] = {0.f, 0.f, 0.f, 0.f}, cb[4] = {0.f, 0.f, 0.f, 0.f};
                const uint32_t wd[4] = {q.w[j].x, q.w[j].y, q.w[j].z, q.w[j].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0;
                    if (xr0) a0 = *reinterpret_cast<const uint4*>(xr0 + ch * 1024 + j * 256 + i * 16);
                    if (xr1) a1 = *reinterpret_cast<const uint4*>(xr1 + ch * 1024 + j * 256 + i * 16);
                    const uint32_t hi = wd[i] >> 8;
                    mma_f16((i & 1) ? cb : ca, a0.x, a1.x, a0.y, a1.y, wd[i] & 0x000F000Fu, wd[i] & 0x00F000F0u);
                    mma_f16((i & 1) ? cb : ca, a0.z, a1.z, a0.w, a1.w, hi & 0x000F000Fu, hi & 0x00F000F0u);
                }
                const float xs0 = m0 * xs0p[ch * 4 + j], xs1 = m1 * xs1p[ch * 4 + j];
                const float e0 = sc0[j] * 16777216.f, e1 = sc1[j] * 16777216.f;
                tot[0] += e0 * (ca[0] + cb[0]) + zr0[j] * xs0;
                tot[1] += e1 * (ca[1] + cb[1]) + zr1[j] * xs0;
                tot[2] += e0 * (ca[2] + cb[2]) + zr0[j] * xs1;
                tot[3] += e1 * (ca[3] + cb[3]) + zr1[j] * xs1;
            }
        }
        const int n0 = tile << 3;
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

template <typename Kern>
static int32_t launch_i4(Kern kern, const I4Args& a, size_t smem, cudaStream_t st) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "gemv_int4_group: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThr, smem);
    if (e != cudaSuccess || per_sm < 1) return fail(RWKVQ_E_LAUNCH, "gemv_int4_group: occupancy query failed");
    const int64_t tiles = (a.N + 7) / 8;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)std::min<int64_t>(tiles, (int64_t)sm_count() * per_sm));
    cfg.blockDim = dim3(kThr);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    const char* env = std::getenv("RWKVQ_PDL");
    cfg.numAttrs = (env && env[0] == '0') ? 0 : 1;
    e = cudaLaunchKernelEx(&cfg, kern, a);
    if (e != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "gemv_int4_group: %s", cudaGetErrorString(e));
    }
    return check_launch("gemv_int4_group");
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

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
    const bool fast = K % 4096 == 0 && group == 128 && !scale_is_f16 && !(env && env[0] == '0')
                      && ((uintptr_t)scales & 15) == 0 && (zeros == nullptr || ((uintptr_t)zeros & 15) == 0);
    if (fast) return launch_i4(gemv_int4_g128_kernel, a, smem, (cudaStream_t)stream);
    return (K / 128 > 4 * kWarps) ? launch_i4(gemv_int4_group_kernel<8>, a, smem, (cudaStream_t)stream)
                                  : launch_i4(gemv_int4_group_kernel<4>, a, smem, (cudaStream_t)stream);
}

}  // extern "C"
