// W8A8 projections on the 5th-generation tensor cores: TMA -> shared memory -> tcgen05.mma -> tensor memory.
//
// One persistent, warp-specialised kernel (one CTA per SM) serves both regimes:
//
//   SWAP (decode, M <= 128 tokens, HBM-bound): the WEIGHTS are the 128-row "A" operand of the MMA, the
//     quantized activations the narrow "B" operand (N = 16..128 tokens), so D^T[weight row, token] accumulates in
//     128 TMEM lanes x N columns.  Weight tiles [128 rows x 128 B] stream through a deep TMA ring straight into
//     the tensor core: no register staging, no LDS.  The (matrix, row tile, 128-byte K chunk) space is cut into
//     one contiguous range per CTA (stream-K), so every SM streams the same number of bytes; a row tile that is
//     shared by several CTAs is finished by the last one to arrive, which adds the partial sums in CTA order
//     (fixed order: results are run-to-run identical).
//     FUSED variant: four extra warps derive the amax / row scales and write the e4m3 / int8 codes of every
//     K chunk directly into the swizzled B tile of its ring stage (activation quantization in the prologue of
//     the GEMV, one launch per projection).
//
//   GEMM (prefill, compute-bound): tokens are the 128-row A operand, a block of NB = 256 weight rows the B
//     operand; both come by TMA; 128 x 256 fp32 (or int32) accumulators, double-buffered in tensor memory so the
//     epilogue of one tile overlaps the MMAs of the next.
//
// Roles: warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane) and owner of the TMEM allocation,
// warps 2-5 = epilogue (one TMEM lane quarter each), warps 6-9 = activation quantizer (SWAP+FUSED only).
// Every mbarrier wait is bounded; a timeout is reported through the status word and the CTA drains and exits.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "tc_common.cuh"
#include "tc_host.cuh"
#include "w8a8.cuh"

namespace rwkvq {
using namespace tc;

constexpr int kTcThreads = 320;
constexpr int kMaxStages = 12;
constexpr int kChunk = 128;          // bytes of K per ring stage (one swizzle row)
constexpr int kTileP = 128;          // rows of the A operand (UMMA M)
constexpr uint32_t kABytes = kTileP * kChunk;

struct TcMaps {
    CUtensorMap w[3];   // weights  [N, K] uint8
    CUtensorMap a[3];   // activation codes [M, K] uint8 (unused in the FUSED variant)
};

struct TcArgs {
    const void* x[3];          // FUSED: activations (x_dtype), rows ldx apart
    const float* awq[3];       // FUSED FP8: optional per-channel divisor
    const float* a_scale[3];   // codes route: FP8 amax-or-scale [1]; INT8 row scales [M]
    const float* ws[3];        // weight scale (one fp32 per matrix)
    __half* out[3];
    int32_t* acc[3];           // INT8: optional raw accumulators
    float* scratch;            // SWAP: partial sums [row tile][slot][M][128] (fp32 or int32 bits)
    int* counters;             // SWAP: arrivals per row tile, zero before the first use, left zero by every launch
    int* status;               // set to RWKVQ_E_TIMEOUT if a bounded wait gave up
    unsigned long long* trace; // optional [grid][16] timestamps of role milestones (profiling aid), else null
    unsigned long long wait_ns; // wall-time limit of every mbarrier wait
    float* ffn_amax;            // RWKVQ_FLAG_RELU2 (GEMM mode): maximum of the relu^2 results, atomic max -- FP8: one word; INT8: one per token row
    const uint8_t* sfa;         // NVFP4 (cluster split-K kernel only): blocked scales of the activation codes ...
    const uint8_t* sfw;         // ... and of the weight codes (rwkvq_nvfp4_pack_scales order)
    TcPush push;                // GEMM mode: also store the result into the peers' buffers and signal them (n = 0: off)
    int64_t ldx, ldo, ldacc;
    int M, N, K, nmat;
    int NB;                    // rows of the B operand (UMMA N)
    int kchunks, ptiles, qtiles, max_slots, stages, acc_stride;
    int x_dtype, div_mode, amax_is_amax;
    uint32_t flags;
};

struct Part {
    int mat, prow, qrow, kc0, kc1, tile, slot, nslots;
};

// Enumerates the parts of this CTA: SWAP = contiguous range of (tile, chunk) units; GEMM = whole tiles, strided.
template <bool SWAP>
struct PartIter {
    // all counts fit 32 bits: the host checks total * grid < 2^31
    const TcArgs& a;
    uint32_t pos, end, total;
    __device__ explicit PartIter(const TcArgs& args) : a(args) {
        if constexpr (SWAP) {
            total = (uint32_t)(a.nmat * a.ptiles * a.kchunks);
            pos = begin_of(blockIdx.x);
            end = begin_of(blockIdx.x + 1);
        } else {
            total = (uint32_t)(a.nmat * a.ptiles * a.qtiles);
            pos = blockIdx.x;
            end = total;
        }
    }
    __device__ uint32_t begin_of(uint32_t c) const { return total * c / gridDim.x; }
    __device__ int owner(uint32_t u) const {     // CTA whose range holds unit u
        uint32_t c = u * gridDim.x / total;
        while (begin_of(c + 1) <= u) ++c;
        while (c > 0 && begin_of(c) > u) --c;
        return (int)c;
    }
    __device__ bool next(Part& p) {
        if (pos >= end) return false;
        if constexpr (SWAP) {
            const uint32_t tile = pos / (uint32_t)a.kchunks;
            p.tile = (int)tile;
            p.kc0 = (int)(pos - tile * a.kchunks);
            p.kc1 = (int)min((uint32_t)a.kchunks, p.kc0 + (end - pos));
            p.mat = (int)(tile / (uint32_t)a.ptiles);
            p.prow = (int)(tile - (uint32_t)p.mat * a.ptiles) * kTileP;
            p.qrow = 0;
            if (p.kc0 == 0 && p.kc1 == a.kchunks) {
                p.slot = 0;
                p.nslots = 1;
            } else {
                const int first = owner(tile * a.kchunks), last = owner((tile + 1) * a.kchunks - 1);
                p.slot = (int)blockIdx.x - first;
                p.nslots = last - first + 1;
            }
            pos += p.kc1 - p.kc0;
        } else {
            const int per_mat = a.ptiles * a.qtiles;
            p.tile = (int)pos;
            p.mat = (int)(pos / (uint32_t)per_mat);
            const int r = (int)(pos - (uint32_t)p.mat * per_mat);
            // token tiles fastest: the CTAs running at one time share a few weight tiles (each read from HBM once and
            // served to the others from L2), while the much smaller activation codes stay in L2 for the whole GEMM
            p.prow = (r % a.ptiles) * kTileP;
            p.qrow = (r / a.ptiles) * a.NB;
            p.kc0 = 0;
            p.kc1 = a.kchunks;
            p.slot = 0;
            p.nslots = 1;
            pos += gridDim.x;
        }
        return true;
    }
};

struct TcShared {
    uint64_t full[kMaxStages], empty[kMaxStages], tfull[2], tempty[2];
    uint32_t tmem_base;
    int abort_flag;
    int last_flag;
    float amax[3];             // FUSED FP8: max(amax, 1e-12) per matrix
    float xs[3][16];           // FUSED INT8: row scales per matrix
    float red[16];             // [0..7] group_max scratch, [8..15] per-warp running maxima
    uint64_t done;             // epilogue warps have read their last accumulator
    uint64_t xbar;             // FUSED: the activation block has landed in shared memory
};

__device__ __forceinline__ void tc_mark(const TcArgs& a, int slot) {      // profiling aid, only with -DRWKVQ_TRACE
#ifdef RWKVQ_TRACE
    if (a.trace) a.trace[(size_t)blockIdx.x * 16 + slot] = global_ns();
#else
    (void)a; (void)slot;
#endif
}

__device__ __forceinline__ void tc_abort(TcShared& s, const TcArgs& a) {
    s.abort_flag = 1;
    if (a.status) atomicExch(a.status, RWKVQ_E_TIMEOUT);
}

// ---- FUSED quantizer helpers (128 threads = warps 6..9); qt = thread index within the group
constexpr int kQThreads = 256;   // warps 2..9 share the FUSED prologue

__device__ __forceinline__ float group_max(float v, float* red, int qt) {   // max over the 256 prologue threads
    v = warp_max(v);
    named_bar_sync(2, kQThreads);
    if ((qt & 31) == 0) red[qt >> 5] = v;
    named_bar_sync(2, kQThreads);
    return fmaxf(fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3])), fmaxf(fmaxf(red[4], red[5]), fmaxf(red[6], red[7])));
}

// FUSED prologue of the quantizer warps: scales (per-call amax for FP8, per-row amax for INT8) and the codes of
// the whole activation block into the compact cache [mat][row][kpad].  Two short loops (amax, then codes) with
// kQB loads in flight per thread; the second read of x hits L1/L2.  The code is kept small on purpose: it runs
// once per CTA, and straight-line code that is executed once is paced by instruction fetch, not by the ALUs.

template <int KIND, int DT>
__device__ __noinline__ void quantizer_prologue(const TcArgs& a, TcShared& s, uint8_t* cache, const uint8_t* xstage, int kpad, int qt) {
    const int kv = a.K >> 3;                          // 8-element vectors per row
    const bool after = (a.flags & RWKVQ_FLAG_AMAX_AFTER_BF16) != 0;
    for (int mat = 0; mat < a.nmat; ++mat) {
        const float* awq = KIND == KIND_F8 ? a.awq[mat] : nullptr;
        const char* xb = reinterpret_cast<const char*>(xstage) + (size_t)mat * a.M * a.K * 2;     // staged rows are K apart
        uint8_t* cb = cache + (size_t)mat * a.M * kpad;
        float sc = 0.f;
        // FP8: one scale for all rows (amax pass over the block, then the code pass); INT8: both passes row by row
        for (int pass = 0; pass < 2; ++pass) {
            for (int r = 0; r < a.M; ++r) {
                const char* xr = xb + (size_t)r * a.K * 2;
                if (KIND == KIND_F8 ? pass == 0 : true) {
                    float m = 0.f;
                    if (KIND == KIND_I8 && pass == 1) continue;
                    for (int b = qt; b < kv; b += kQThreads) {
                        const uint4 v = *reinterpret_cast<const uint4*>(xr + (size_t)b * 16);
                        if constexpr (KIND == KIND_F8) fp8_vec_amax<DT>(v, awq, b << 3, a.div_mode, after, m);
                        else m = int8_vec_amax<DT>(v, m);
                    }
                    if constexpr (KIND == KIND_F8) {
                        s.red[8 + (qt >> 5)] = fmaxf(r == 0 ? 0.f : s.red[8 + (qt >> 5)], warp_max(m));   // per-warp running max
                        if (r + 1 < a.M) continue;
                        named_bar_sync(2, kQThreads);
                        m = 0.f;
#pragma unroll
                        for (int w = 0; w < 8; ++w) m = fmaxf(m, s.red[8 + w]);
                        m = fmaxf(m, 1e-12f);
                        if (qt == 0) s.amax[mat] = m;
                        sc = div_mode_f32(448.f, m, a.div_mode);
                        named_bar_sync(2, kQThreads);
                        continue;
                    } else {
                        m = fmaxf(group_max(m, s.red, qt), 1e-12f);
                        if (qt == 0) s.xs[mat][r] = m;
                        sc = div_mode_f32(127.f, m, a.div_mode);
                    }
                }
                uint8_t* cr = cb + (size_t)r * kpad;
                for (int b = qt; b < kv; b += kQThreads) {
                    const uint4 v = *reinterpret_cast<const uint4*>(xr + (size_t)b * 16);
                    uint2 c;
                    if constexpr (KIND == KIND_F8) c = fp8_vec_codes<DT>(v, awq, b << 3, a.div_mode, sc);
                    else c = int8_vec_codes<DT>(v, sc);
                    *reinterpret_cast<uint2*>(cr + (size_t)b * 8) = c;
                }
            }
            if (KIND == KIND_I8) break;
        }
    }
    named_bar_sync(2, kQThreads);
}

// Copies the codes of K chunk kc from the cache into a swizzled B tile; one warp: lane -> (row = lane/8 + 4*pass,
// 16-byte chunk = lane%8).  Rows >= M of the tile stay zero.
__device__ __forceinline__ void copy_chunk(const TcArgs& a, const uint8_t* cache, int kpad, int mat, int kc, uint8_t* btile, int lane) {
    const int c = lane & 7;
    for (int r = lane >> 3; r < a.M; r += 4) {
        const uint4 v = *reinterpret_cast<const uint4*>(cache + ((size_t)mat * a.M + r) * kpad + kc * kChunk + c * 16);
        *reinterpret_cast<uint4*>(btile + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)) = v;
    }
}

// FUSED: bring the activation block into shared memory with bulk copies (one memory latency for all of it), zero the
// B tiles (rows >= M stay zero for the whole kernel) and the cache tail meanwhile, then quantize from shared memory.
template <int KIND, int DT>
__device__ __noinline__ bool fused_prologue(const TcArgs& a, TcShared& s, uint8_t* ring, uint32_t stage_bytes, int qt,
                                            const volatile int* abort_flag) {
    const int kpad = a.kchunks * kChunk;
    uint8_t* cache = ring + (size_t)a.stages * stage_bytes;          // [nmat][M][kpad] codes, zero beyond K
    uint8_t* xstage = cache + (size_t)a.nmat * a.M * kpad;           // [nmat][M][K] activations as given
    if (qt == 0) {
        const uint32_t row_bytes = (uint32_t)a.K * 2;
        mbar_expect_tx(&s.xbar, row_bytes * a.M * a.nmat);
        for (int mat = 0; mat < a.nmat; ++mat)
            for (int r = 0; r < a.M; ++r)
                bulk_load_1d(xstage + ((size_t)mat * a.M + r) * row_bytes,
                             reinterpret_cast<const char*>(a.x[mat]) + (int64_t)r * a.ldx * 2, row_bytes, &s.xbar);
    }
    for (int st = 0; st < a.stages; ++st) {
        uint4* b = reinterpret_cast<uint4*>(ring + (size_t)st * stage_bytes + kABytes);
        for (int i = qt; i < a.NB * kChunk / 16; i += kQThreads) b[i] = make_uint4(0, 0, 0, 0);
    }
    if (kpad != a.K)
        for (int i = qt; i < a.nmat * a.M * kpad / 16; i += kQThreads) reinterpret_cast<uint4*>(cache)[i] = make_uint4(0, 0, 0, 0);
    const bool ok = mbar_wait(&s.xbar, 0, abort_flag, a.wait_ns);
    named_bar_sync(2, kQThreads);
    if (ok) quantizer_prologue<KIND, DT>(a, s, cache, xstage, kpad, qt);
    return ok;
}

template <int KIND, bool SWAP, bool FUSED, int DT>
__global__ void __launch_bounds__(kTcThreads, SWAP ? 2 : 1) gemm_tc_kernel(const __grid_constant__ TcMaps maps, const TcArgs a) {
    using T = typename Acc<KIND == KIND_F8 ? QT_FP8 : QT_INT8>::T;
    extern __shared__ uint8_t smem_raw[];
    __shared__ TcShared s;
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t stage_bytes = kABytes + (uint32_t)a.NB * kChunk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tmem_cols = a.acc_stride * 2 <= 32 ? 32u : (a.acc_stride * 2 <= 64 ? 64u : (a.acc_stride * 2 <= 128 ? 128u : (a.acc_stride * 2 <= 256 ? 256u : 512u)));

    griddep_launch_dependents();
    if (threadIdx.x == 0) tc_mark(a, 0);

    if (threadIdx.x == 0) {
        for (int i = 0; i < a.stages; ++i) {
            mbar_init(&s.full[i], FUSED ? 2 : 1);
            mbar_init(&s.empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.tfull[i], 1);
            mbar_init(&s.tempty[i], 4);
        }
        mbar_init(&s.done, 4);
        mbar_init(&s.xbar, 1);
        s.abort_flag = 0;
        s.last_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        for (int i = 0; i < a.nmat; ++i) {
            prefetch_tmap(&maps.w[i]);
            if (!FUSED) prefetch_tmap(&maps.a[i]);
        }
    }
    if (warp == 1) tmem_alloc(&s.tmem_base, tmem_cols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = s.tmem_base;
    if (threadIdx.x == 0) tc_mark(a, 1);
    const volatile int* abort_flag = &s.abort_flag;

    if (warp == 0) {
        // ============================== TMA producer ==============================
        if (lane == 0) {
            uint32_t npre = 0;
            if constexpr (!FUSED) {
                // The weights do not depend on the previous kernel: the first pass over the ring loads them before the
                // dependency wait (each stage's barrier already expects the whole stage), so under programmatic
                // dependent launch a ring of weights is on its way while the activation quantizer still runs.
                PartIter<SWAP> pre(a);
                Part q;
                while (npre < (uint32_t)a.stages && pre.next(q))
                    for (int kc = q.kc0; kc < q.kc1 && npre < (uint32_t)a.stages; ++kc, ++npre) {
                        uint8_t* dst = ring + (size_t)npre * stage_bytes;
                        mbar_expect_tx(&s.full[npre], stage_bytes);
                        if constexpr (SWAP) tma_load_2d(dst, &maps.w[q.mat], kc * kChunk, q.prow, &s.full[npre]);
                        else tma_load_2d(dst + kABytes, &maps.w[q.mat], kc * kChunk, q.qrow, &s.full[npre]);
                    }
                tc_mark(a, 2);
                griddep_wait();                         // activation codes are written by the previous kernel
            }
            PartIter<SWAP> it(a);
            Part p;
            uint32_t n = 0;
            bool ok = true;
            while (ok && it.next(p)) {
                for (int kc = p.kc0; kc < p.kc1 && ok; ++kc, ++n) {
                    const int st = n % a.stages;
                    uint8_t* dst = ring + (size_t)st * stage_bytes;
                    if (FUSED || n >= npre) {
                        const uint32_t ph = (n / a.stages) & 1;
                        if (!mbar_wait(&s.empty[st], ph ^ 1, abort_flag, a.wait_ns)) { tc_abort(s, a); ok = false; break; }
                        mbar_expect_tx(&s.full[st], FUSED ? kABytes : stage_bytes);
                        if constexpr (SWAP) tma_load_2d(dst, &maps.w[p.mat], kc * kChunk, p.prow, &s.full[st]);
                        else tma_load_2d(dst + kABytes, &maps.w[p.mat], kc * kChunk, p.qrow, &s.full[st]);
                    }
                    if constexpr (!FUSED) {
                        if constexpr (SWAP) tma_load_2d(dst + kABytes, &maps.a[p.mat], kc * kChunk, p.qrow, &s.full[st]);
                        else tma_load_2d(dst, &maps.a[p.mat], kc * kChunk, p.prow, &s.full[st]);
                    }
                    if (FUSED && n == 0) tc_mark(a, 2);
                }
            }
            tc_mark(a, 10);
            if (!ok) {   // give copies already in flight a bounded time to land before the CTA's memory is released
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 2000000ull) {}
            }
        }
    } else if (warp == 1) {
        // ============================== MMA issuer ==============================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(KIND, kTileP, a.NB);
            PartIter<SWAP> it(a);
            Part p;
            uint32_t n = 0, pc = 0;
            bool ok = true;
            while (ok && it.next(p)) {
                const int buf = pc & 1;
                if (!mbar_wait(&s.tempty[buf], ((pc >> 1) & 1) ^ 1, abort_flag, a.wait_ns)) { tc_abort(s, a); break; }
                tc_fence_after_sync();
                const uint32_t d = tmem_base + (uint32_t)(buf * a.acc_stride);
                for (int kc = p.kc0; kc < p.kc1; ++kc, ++n) {
                    const int st = n % a.stages;
                    if (!mbar_wait(&s.full[st], (n / a.stages) & 1, abort_flag, a.wait_ns)) { tc_abort(s, a); ok = false; break; }
                    tc_fence_after_sync();
                    if (n == 0) tc_mark(a, 5);
                    const uint32_t sa = smem_u32(ring + (size_t)st * stage_bytes);
                    const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sa + kABytes);
#pragma unroll
                    for (int k = 0; k < kChunk / 32; ++k)
                        tc_mma<KIND>(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kc > p.kc0 || k > 0) ? 1u : 0u);
                    tc_commit(&s.empty[st]);            // the stage may be refilled once these MMAs have read it
                }
                if (ok) tc_commit(&s.tfull[buf]);
                ++pc;
            }
            tc_mark(a, 6);
        }
    } else if (warp < 6) {
        // ============================== epilogue ==============================
        griddep_wait();
        if constexpr (SWAP && FUSED) {
            if (!fused_prologue<KIND, DT>(a, s, ring, stage_bytes, threadIdx.x - 64, abort_flag)) tc_abort(s, a);
        }
        const int q = warp & 3;                         // TMEM lane quarter this warp may read
        const int et = (warp - 2) * 32 + lane;          // thread index inside the epilogue group
        const int prow_l = q * 32 + lane;               // row of the A operand held by this thread
        PartIter<SWAP> it(a);
        Part p;
        uint32_t pc = 0;
        while (it.next(p)) {
            const int buf = pc & 1;
            if (!mbar_wait(&s.tfull[buf], (pc >> 1) & 1, abort_flag, a.wait_ns)) { tc_abort(s, a); break; }
            tc_fence_after_sync();
            if (pc == 0 && et == 0) tc_mark(a, 7);
            const uint32_t taddr = tmem_base + (uint32_t)(buf * a.acc_stride) + ((uint32_t)(q * 32) << 16);
            const bool per_row = (a.flags & RWKVQ_FLAG_WSCALE_PER_ROW) != 0;   // one weight scale per output row
            float wsc = a.ws[p.mat][0];
            if constexpr (SWAP) {
                const int n = p.prow + prow_l;          // weight row
                if (per_row) wsc = a.ws[p.mat][min(n, a.N - 1)];
                const bool partial = p.nslots > 1;
                float act_scale = 0.f;
                if constexpr (KIND == KIND_F8) {
                    float am;
                    if constexpr (FUSED) am = s.amax[p.mat];
                    else am = a.amax_is_amax ? fmaxf(a.a_scale[p.mat][0], 1e-12f) : a.a_scale[p.mat][0];
                    act_scale = (FUSED || a.amax_is_amax) ? div_mode_f32(am, 448.f, a.div_mode) : am;
                }
                auto finish_at = [&](T v, int m, int row, float wrow) {     // element (token m, weight row) of the result
                    float f;
                    if constexpr (KIND == KIND_F8) {
                        f = v * (act_scale * wrow);
                    } else {
                        if (a.acc[p.mat]) a.acc[p.mat][(int64_t)m * a.ldacc + row] = v;
                        float rs;
                        if constexpr (FUSED) rs = div_mode_f32(s.xs[p.mat][m], 127.f, a.div_mode);
                        else rs = a.a_scale[p.mat][m];
                        f = (float)v * (rs * wrow);
                    }
                    if (a.flags & RWKVQ_FLAG_OUT_VIA_BF16) f = bf16_round(f);
                    a.out[p.mat][(int64_t)m * a.ldo + row] = __float2half_rn(f);
                };
                auto finish = [&](T v, int m) { finish_at(v, m, n, wsc); };
                T* part = reinterpret_cast<T*>(a.scratch) + ((int64_t)p.tile * a.max_slots + p.slot) * a.M * kTileP;
                for (int c0 = 0; c0 < a.M; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(taddr + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = c0 + j;
                        if (m < a.M) {
                            T v;
                            if constexpr (KIND == KIND_F8) v = __uint_as_float(r[j]); else v = (int32_t)r[j];
                            if (partial) __stcg(part + (int64_t)m * kTileP + prow_l, v);
                            else if (n < a.N) finish(v, m);
                        }
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.tempty[buf]);
                if (partial) {
                    __threadfence();
                    named_bar_sync(1, 128);
                    if (et == 0) {
                        const int old = atomicAdd(a.counters + p.tile, 1);
                        s.last_flag = old == p.nslots - 1;
                        if (s.last_flag) a.counters[p.tile] = 0;
                    }
                    named_bar_sync(1, 128);
                    if (s.last_flag) {
                        // The last arriver adds the tile's partial sums in CTA order (run-to-run identical).  This is a
                        // chain of L2 round trips on the critical path of the whole launch, so it is laid out for
                        // loads in flight: a thread takes FOUR neighbouring weight rows (one 16-byte load per slot and
                        // token) and two tokens at a time, 16 independent loads per batch.
                        __threadfence();
                        using V4 = typename std::conditional<KIND == KIND_F8, float4, int4>::type;
                        const T* base = reinterpret_cast<const T*>(a.scratch) + (int64_t)p.tile * a.max_slots * a.M * kTileP;
                        const int rg = et & 31, tl = et >> 5;           // row group (4 rows), token lane (tokens tl, tl + 4, ...)
                        const int row0 = p.prow + 4 * rg;
                        float w4[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) w4[i] = per_row ? a.ws[p.mat][min(row0 + i, a.N - 1)] : wsc;
                        for (int m0 = tl; m0 < a.M; m0 += 8) {
                            T sum[2][4] = {};
                            for (int s0 = 0; s0 < p.nslots; s0 += 8) {
                                V4 v[2][8];
#pragma unroll
                                for (int u = 0; u < 2; ++u)
#pragma unroll
                                    for (int j = 0; j < 8; ++j) {
                                        const int m = m0 + 4 * u;
                                        if (m < a.M && s0 + j < p.nslots)
                                            v[u][j] = __ldcg(reinterpret_cast<const V4*>(base + ((int64_t)(s0 + j) * a.M + m) * kTileP + 4 * rg));
                                        else
                                            v[u][j] = V4{};
                                    }
#pragma unroll
                                for (int u = 0; u < 2; ++u)
#pragma unroll
                                    for (int j = 0; j < 8; ++j) {
                                        sum[u][0] += v[u][j].x; sum[u][1] += v[u][j].y; sum[u][2] += v[u][j].z; sum[u][3] += v[u][j].w;
                                    }
                            }
#pragma unroll
                            for (int u = 0; u < 2; ++u) {
                                const int m = m0 + 4 * u;
                                if (m < a.M)
#pragma unroll
                                    for (int i = 0; i < 4; ++i)
                                        if (row0 + i < a.N) finish_at(sum[u][i], m, row0 + i, w4[i]);
                            }
                        }
                    }
                }
            } else {
                const int m = p.prow + prow_l;          // token row
                float actscale;                         // scale of this thread's token row; the weight scale joins below
                if constexpr (KIND == KIND_F8) {
                    const float am = a.a_scale[p.mat][0];
                    actscale = a.amax_is_amax ? div_mode_f32(fmaxf(am, 1e-12f), 448.f, a.div_mode) : am;
                } else {
                    actscale = m < a.M ? a.a_scale[p.mat][m] : 0.f;
                }
                const float rowscale = actscale * wsc;
                const bool vec_ok = (a.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.out[p.mat]) & 15) == 0);
                const bool relu2 = (a.flags & RWKVQ_FLAG_RELU2) != 0;
                const bool hmax_bf16 = (a.flags & RWKVQ_FLAG_AMAX_AFTER_BF16) != 0;
                float hmax = 0.f;
                // 16 accumulator columns of this thread's token row -> 8 fp16 pairs (scales, optional bf16 hop, relu^2)
                auto convert16 = [&](const uint32_t (&r)[16], int n0, uint32_t (&h)[8]) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float s0 = rowscale, s1 = rowscale;
                        if (per_row) {
                            s0 = actscale * a.ws[p.mat][min(n0 + 2 * j, a.N - 1)];
                            s1 = actscale * a.ws[p.mat][min(n0 + 2 * j + 1, a.N - 1)];
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
                        if (relu2) {
                            // the engine's relu_square on the fp16 result, fp32 arithmetic; its maximum (over the bf16-rounded
                            // values where the consumer takes its amax there) goes to the projection that follows
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
                };
                if (a.push.n > 0) {
                    // column-split projection with the all-gather riding in this epilogue (TcPush in tc_host.cuh)
                    uint8_t* stg = ring + (size_t)a.stages * stage_bytes + (size_t)(warp - 2) * kTcStgWarp;
                    const bool vec8 = vec_ok && a.N % 8 == 0;
                    for (int c0 = 0; c0 < a.NB; c0 += 64) {
#pragma unroll
                        for (int cc = 0; cc < 4; ++cc) {
                            uint32_t r[16], h[8];
                            tmem_ld16(taddr + c0 + cc * 16, r);
                            tmem_ld_wait();
                            convert16(r, p.qrow + c0 + cc * 16, h);
                            uint4* d = reinterpret_cast<uint4*>(stg + lane * kTcStgRow + cc * 32);
                            d[0] = make_uint4(h[0], h[1], h[2], h[3]);
                            d[1] = make_uint4(h[4], h[5], h[6], h[7]);
                        }
                        __syncwarp();
                        push_store_rows(a.push, stg, a.out[p.mat], a.ldo, p.prow + q * 32, p.qrow + c0, a.M, a.N, vec8, lane);
                        __syncwarp();
                    }
                } else
                for (int c0 = 0; c0 < a.NB; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(taddr + c0, r);
                    tmem_ld_wait();
                    const int n0 = p.qrow + c0;
                    if (m < a.M && n0 < a.N) {
                        uint32_t h[8];
                        convert16(r, n0, h);
                        __half* o = a.out[p.mat] + (int64_t)m * a.ldo + n0;
                        if (vec_ok && n0 + 16 <= a.N) {
                            reinterpret_cast<uint4*>(o)[0] = make_uint4(h[0], h[1], h[2], h[3]);
                            reinterpret_cast<uint4*>(o)[1] = make_uint4(h[4], h[5], h[6], h[7]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (n0 + j < a.N) o[j] = __ushort_as_half((unsigned short)((h[j >> 1] >> ((j & 1) * 16)) & 0xffff));
                        }
                        if constexpr (KIND == KIND_I8) {
                            if (a.acc[p.mat]) {
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    if (n0 + j < a.N) a.acc[p.mat][(int64_t)m * a.ldacc + n0 + j] = (int32_t)r[j];
                            }
                        }
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.tempty[buf]);
                if (relu2) {
                    if constexpr (KIND == KIND_F8) {          // one atomic per warp and tile
                        hmax = warp_max(hmax);
                        if (lane == 0 && hmax > 0.f) atomic_max_nonneg(a.ffn_amax, hmax);
                    } else {                                  // INT8 activations are scaled per token row: a thread holds one
                        if (m < a.M && hmax > 0.f) atomic_max_nonneg(a.ffn_amax + m, hmax);
                    }
                }
            }
            ++pc;
        }
        if (et == 0) tc_mark(a, 8);
        if (!SWAP && a.push.n > 0) __threadfence_system();      // this thread's peer stores are ordered before its arrival below
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.done);
    } else if (SWAP && FUSED) {
        // ============================== activation quantizer ==============================
        griddep_wait();
        const int qw = warp - 6;
        const int kpad = a.kchunks * kChunk;
        const uint8_t* cache = ring + (size_t)a.stages * stage_bytes;
        if (threadIdx.x == 6 * 32) tc_mark(a, 3);
        if (!fused_prologue<KIND, DT>(a, s, ring, stage_bytes, threadIdx.x - 64, abort_flag)) tc_abort(s, a);
        if (threadIdx.x == 6 * 32) tc_mark(a, 4);
        // each of the four warps feeds every fourth ring slot
        PartIter<SWAP> it(a);
        Part p;
        uint32_t n = 0;
        bool ok = true;
        while (ok && it.next(p)) {
            for (int kc = p.kc0; kc < p.kc1; ++kc, ++n) {
                if ((int)(n & 3) != qw) continue;
                const int st = n % a.stages;
                if (!mbar_wait(&s.empty[st], ((n / a.stages) & 1) ^ 1, abort_flag, a.wait_ns)) { tc_abort(s, a); ok = false; break; }
                copy_chunk(a, cache, kpad, p.mat, kc, ring + (size_t)st * stage_bytes + kABytes, lane);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.full[st]);
            }
        }
    }

    __syncwarp();            // single-lane roles: the other lanes wait here for their lane 0
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        // the accumulators are released only after every epilogue warp has read its last one
        if (!mbar_wait(&s.done, 0, abort_flag, a.wait_ns)) tc_abort(s, a);
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, tmem_cols);
        if (!SWAP && a.push.n > 0 && lane == 0) push_signal(a.push);
    }
}

// ------------------------------------------------------------------------------------------------ host side
constexpr size_t kTcSmemBudget = 225 * 1024;
constexpr size_t kTcSmemBudgetHalf = 110 * 1024;   // SWAP: two CTAs per SM, so the next launch can set up early
constexpr size_t kTcCacheMax = 100 * 1024;      // FUSED: the activations of a call and their codes live in shared memory

static int tc_grid() {
    static const int forced = [] {
        const char* e = std::getenv("RWKVQ_TC_GRID");
        return e ? std::atoi(e) : 0;
    }();
    return forced > 0 ? forced : sm_count();
}

// upper bound of the CTAs that share one row tile under the stream-K split
static int max_slots_for(int64_t total_units, int kchunks, int grid) {
    const int64_t per = std::max<int64_t>(1, total_units / grid);
    return (int)((kchunks + per - 1) / per) + 1;
}

template <int KIND, bool SWAP, bool FUSED, int DT>
static int32_t launch_tc(const TcMaps& maps, const TcArgs& a, int grid, cudaStream_t st, const char* who) {
    auto kern = gemm_tc_kernel<KIND, SWAP, FUSED, DT>;
    const int32_t rc = ensure_smem_optin(reinterpret_cast<const void*>(kern), (int)kTcSmemBudget, who);   // per device
    if (rc != RWKVQ_OK) return rc;
    const size_t cache = FUSED ? (size_t)a.nmat * a.M * ((size_t)a.kchunks * kChunk + (size_t)a.K * 2) : 0;
    const size_t smem = (size_t)a.stages * (kABytes + (size_t)a.NB * kChunk) + cache + 1024 + (a.push.n > 0 ? kTcStgBytes : 0);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kTcThreads);
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

// Weights as the 128-row operand with stream-K (SWAP, the only form that uses the workspace's partial sums) pays for
// few tokens only: measured on the 7.2B shapes, the GEMM mode (tokens as the 128-row operand, narrow weight tiles) is
// 2-4 x faster from 33 tokens on, except for a long K against few weight tiles (FFN value: K = 16384, N = 4096), where
// stream-K wins up to 48 tokens.
static bool takes_swap_route(int64_t M, int64_t N, int64_t K, int nmat, bool fused) {
    const int64_t narrow_tiles = (int64_t)nmat * ((M + kTileP - 1) / kTileP) * ((N + 63) / 64);
    static const int64_t long_k_max_m = std::getenv("RWKVQ_TC_SWAP_MAX_M") ? std::atoll(std::getenv("RWKVQ_TC_SWAP_MAX_M")) : 48;
    return fused || M <= 16 || (M <= long_k_max_m && K >= 8192 && 2 * narrow_tiles <= tc_grid());
}

struct TcCall {
    int kind;                 // KIND_F8 / KIND_I8
    bool fused;               // SWAP only: quantize activations in the kernel
    int x_dtype;
    const void* w[3];
    int64_t ldw;
    const void* codes[3];     // codes route
    int64_t lda;
    void* workspace;
    int64_t workspace_bytes;
};

static unsigned long long* g_trace = nullptr;

}  // namespace rwkvq

#include "gemm_tcs.cuh"        // few tokens: K split across a thread-block cluster, partial sums through distributed shared memory
#include "gemm_tcsn.cuh"       // NVFP4, one to four tokens: the same with the activation quantization inside (one launch)

namespace rwkvq {

static int32_t run_tc(TcArgs a, const TcCall& c, cudaStream_t st, const char* who) {
    a.trace = g_trace;
    a.wait_ns = wait_limit_ns();
    RWKVQ_REQUIRE(a.M >= 0 && a.N >= 0 && a.K >= 0, RWKVQ_E_SHAPE, "%s: negative size", who);
    RWKVQ_REQUIRE(a.K % 16 == 0, RWKVQ_E_SHAPE, "%s: K=%d must be a multiple of 16", who, a.K);
    RWKVQ_REQUIRE(a.ldo >= a.N, RWKVQ_E_SHAPE, "%s: ldo=%lld < N", who, (long long)a.ldo);
    RWKVQ_REQUIRE(a.div_mode == RWKVQ_DIV_IEEE || a.div_mode == RWKVQ_DIV_FULL, RWKVQ_E_BADARG, "%s: div_mode %d", who, a.div_mode);
    for (int i = 0; i < a.nmat; ++i) {
        RWKVQ_REQUIRE(c.w[i] && a.ws[i] && a.out[i], RWKVQ_E_BADARG, "%s: null weight / scale / out pointer (matrix %d)", who, i);
        if (c.fused) {
            RWKVQ_REQUIRE(a.x[i] != nullptr, RWKVQ_E_BADARG, "%s: null activation pointer", who);
            RWKVQ_REQUIRE(aligned16(a.x[i]) && a.ldx % 8 == 0 && a.ldx >= a.K, RWKVQ_E_ALIGN, "%s: activation rows must be 16-byte aligned", who);
        } else {
            RWKVQ_REQUIRE(c.codes[i] && a.a_scale[i], RWKVQ_E_BADARG, "%s: null activation codes / scale", who);
        }
    }
    if (c.fused) RWKVQ_REQUIRE(c.x_dtype == RWKVQ_F16 || c.x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, c.x_dtype);
    if (a.M == 0 || a.N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(a.K > 0, RWKVQ_E_SHAPE, "%s: K=0", who);

    const bool swap = takes_swap_route(a.M, a.N, a.K, a.nmat, c.fused);
    if (c.fused) RWKVQ_REQUIRE(a.M <= 16, RWKVQ_E_SHAPE, "%s: the fused kernel takes M <= 16, got %d", who, a.M);
    a.kchunks = (a.K + kChunk - 1) / kChunk;
    const bool pushing = a.push.n > 0 || a.push.counter != nullptr;
    if (pushing)
        RWKVQ_REQUIRE(!c.fused && a.nmat == 1 && !swap && !tcs_eligible(a.M, a.N, a.K, a.flags, 1) && !(a.flags & RWKVQ_FLAG_RELU2) && a.acc[0] == nullptr,
                      RWKVQ_E_SHAPE, "%s: %d rows run a kernel that cannot carry the all-gather (see rwkvq_tc_gemm_can_push)", who, a.M);
    if (!pushing && !c.fused && tcs_eligible(a.M, a.N, a.K, a.flags, a.nmat)) {
        a.status = nullptr;
        return run_tcs(a, c, st, who);
    }
    TcMaps maps;
    int grid;
    if (swap) {
        a.NB = a.M <= 16 ? 16 : (a.M <= 32 ? 32 : (a.M <= 64 ? 64 : 128));
        a.ptiles = (a.N + kTileP - 1) / kTileP;
        a.qtiles = 1;
        const int64_t total = (int64_t)a.nmat * a.ptiles * a.kchunks;
        grid = (int)std::min<int64_t>(tc_grid(), total);
        RWKVQ_REQUIRE(total * grid < (int64_t(1) << 31), RWKVQ_E_SHAPE, "%s: problem too large for the 32-bit tile schedule", who);
        a.max_slots = max_slots_for(total, a.kchunks, grid);
        const int64_t tiles = (int64_t)a.nmat * a.ptiles;
        RWKVQ_REQUIRE(tiles <= kWsCounterInts, RWKVQ_E_SHAPE, "%s: N=%d has too many row tiles for the workspace counters", who, a.N);
        const int64_t need = kWsHeaderBytes + tiles * a.max_slots * (int64_t)a.M * kTileP * 4;
        RWKVQ_REQUIRE(c.workspace != nullptr && c.workspace_bytes >= need, RWKVQ_E_WORKSPACE,
                      "%s: workspace of %lld bytes needed, %lld given", who, (long long)need, (long long)c.workspace_bytes);
        RWKVQ_REQUIRE(aligned16(c.workspace), RWKVQ_E_ALIGN, "%s: workspace must be 16-byte aligned", who);
        a.counters = reinterpret_cast<int*>(c.workspace);
        a.status = a.counters + kWsCounterInts;
        a.scratch = reinterpret_cast<float*>(reinterpret_cast<char*>(c.workspace) + kWsHeaderBytes);
    } else {
        if (!pushing && tc2_eligible(c.kind, a.M, a.N, a.K, a.nmat) && !(c.kind == KIND_I8 && (a.flags & RWKVQ_FLAG_RELU2)))      // many tokens: CTA pairs on 256 x 256 tiles (gemm_tc2.cu)
            return run_tc2(c.kind, c.codes[0], c.lda, a.a_scale[0], a.amax_is_amax, c.w[0], c.ldw, a.ws[0], a.out[0], a.ldo, a.acc[0], a.ldacc,
                           a.M, a.N, a.K, a.div_mode, a.flags, a.ffn_amax,
                           c.workspace ? reinterpret_cast<int*>(c.workspace) + kWsCounterInts : device_status_ptr(), st, who);
        // 256 weight rows per tile; narrower tiles while halving them still leaves no more tiles than SMs
        a.NB = 256;
        while (a.NB > 64 && 2 * (int64_t)a.nmat * ((a.M + kTileP - 1) / kTileP) * ((a.N + a.NB - 1) / a.NB) <= tc_grid()) a.NB >>= 1;
        a.ptiles = (a.M + kTileP - 1) / kTileP;
        a.qtiles = (a.N + a.NB - 1) / a.NB;
        grid = (int)std::min<int64_t>(tc_grid(), (int64_t)a.nmat * a.ptiles * a.qtiles);
        a.max_slots = 1;
        a.status = c.workspace ? reinterpret_cast<int*>(c.workspace) + kWsCounterInts : nullptr;
    }
    a.acc_stride = std::max(a.NB, 32);
    const size_t stage_bytes = kABytes + (size_t)a.NB * kChunk;
    const size_t cache_bytes = c.fused ? (size_t)a.nmat * a.M * ((size_t)a.kchunks * kChunk + (size_t)a.K * 2) : 0;
    RWKVQ_REQUIRE(cache_bytes <= kTcCacheMax, RWKVQ_E_SHAPE, "%s: %d x %d x %d activation codes do not fit the fused kernel's shared memory",
                  who, a.nmat, a.M, a.K);
    const size_t budget = (swap && cache_bytes + 5 * stage_bytes + 1024 <= kTcSmemBudgetHalf && !std::getenv("RWKVQ_TC_ONE_PER_SM"))
                              ? kTcSmemBudgetHalf : kTcSmemBudget;
    a.stages = (int)std::min<size_t>(kMaxStages, (budget - 1024 - cache_bytes - (a.push.n > 0 ? kTcStgBytes : 0)) / stage_bytes);
    RWKVQ_REQUIRE(a.stages >= 2, RWKVQ_E_SHAPE, "%s: shared memory leaves fewer than two ring stages", who);
    for (int i = 0; i < a.nmat; ++i) {
        int32_t rc = make_map(&maps.w[i], c.w[i], a.N, a.K, c.ldw, swap ? kTileP : a.NB, who);
        if (rc) return rc;
        if (!c.fused) {
            rc = make_map(&maps.a[i], c.codes[i], a.M, a.K, c.lda, swap ? a.NB : kTileP, who);
            if (rc) return rc;
        }
    }
#define RWKVQ_TC(KIND, SWAP, FUSED, DT) launch_tc<KIND, SWAP, FUSED, DT>(maps, a, grid, st, who)
    if (c.kind == KIND_F8) {
        if (c.fused) return c.x_dtype == RWKVQ_F16 ? RWKVQ_TC(KIND_F8, true, true, RWKVQ_F16) : RWKVQ_TC(KIND_F8, true, true, RWKVQ_BF16);
        return swap ? RWKVQ_TC(KIND_F8, true, false, RWKVQ_BF16) : RWKVQ_TC(KIND_F8, false, false, RWKVQ_BF16);
    }
    if (c.fused) return c.x_dtype == RWKVQ_F16 ? RWKVQ_TC(KIND_I8, true, true, RWKVQ_F16) : RWKVQ_TC(KIND_I8, true, true, RWKVQ_BF16);
    return swap ? RWKVQ_TC(KIND_I8, true, false, RWKVQ_BF16) : RWKVQ_TC(KIND_I8, false, false, RWKVQ_BF16);
#undef RWKVQ_TC
}

// NVFP4 on the cluster split-K kernel.  The tiled NVFP4 GEMM (gemm_tc_nvfp4.cu) has no K split: with few tokens a
// matrix gives it at most N / 128 tiles (32 for N = 4096), each streaming all of K through one SM.
bool tcs_nvfp4_eligible(int64_t M, int64_t N, int64_t K) {
    const char* env = std::getenv("RWKVQ_TCS_NF4_MIN_C");        // read per call: a test switches routes in one process
    const int min_c = env ? std::atoi(env) : 0;
    static const int on = std::getenv("RWKVQ_TCS") ? std::atoi(std::getenv("RWKVQ_TCS")) : 1;
    if (!on || M < 1 || M > kTcsMaxM || K % 256 || K < 2048) return false;
    // measured on the 7.2B shapes: with 128 row tiles (N = 16384) a cluster of two wins up to 32 tokens (16 tokens:
    // 14.7 against 18.5 us) and loses at 64 (23.9 against 22.1 us); from 65 tokens on a cluster of two wins again (FFN
    // value, 256 tokens: 57 -> 40 us)
    return tcs_cluster_size(M, N, K / 2) >= (min_c > 0 ? min_c : (M > 32 && M <= 64 ? 4 : 2));
}

int32_t run_tcs_nvfp4(const uint8_t* a_codes, int64_t lda, const uint8_t* a_scales_blocked, const float* a_pts, const uint8_t* w_codes,
                      int64_t ldw, const uint8_t* w_scales_blocked, const float* w_tscale, __half* out, int64_t ldo, int64_t M, int64_t N,
                      int64_t K, int* status, cudaStream_t st, const char* who) {
    TcArgs a{};
    a.a_scale[0] = a_pts; a.amax_is_amax = 0; a.ws[0] = w_tscale; a.out[0] = out;
    a.sfa = a_scales_blocked; a.sfw = w_scales_blocked;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldo = ldo; a.div_mode = RWKVQ_DIV_IEEE; a.flags = 0;
    a.kchunks = (int)(K / 256);               // ring stages of 128 bytes of codes = 256 values of k
    a.trace = g_trace;
    a.wait_ns = wait_limit_ns();
    a.status = status;
    TcCall c{};
    c.kind = KIND_NF4; c.w[0] = w_codes; c.ldw = ldw; c.codes[0] = a_codes; c.lda = lda;
    return run_tcs(a, c, st, who);
}

}  // namespace rwkvq

// ---------------------------------------------------------------------------------------------------------------
// Built-in scratch for callers that cannot provide a workspace (see rwkvq_tc_gemm_fp8_static below).  The array lives
// in every GPU's memory from the moment the library is loaded on it until the process exits.
namespace rwkvq {
constexpr size_t kStaticScratchBytes = size_t(8) << 20;      // 8 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the symbol; the device address has to be asked for, once per
// device and with that device current.
static int32_t static_scratch_ptr(void** out) {
    static std::mutex mu;
    static void* ptrs[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    RWKVQ_REQUIRE(e == cudaSuccess && dev >= 0 && dev < 64, RWKVQ_E_LAUNCH, "static scratch: cudaGetDevice: %s", cudaGetErrorString(e));
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        RWKVQ_REQUIRE(e == cudaSuccess && p != nullptr, RWKVQ_E_LAUNCH, "static scratch: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return RWKVQ_OK;
}
}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

/* profiling aid: device buffer of [grid][16] uint64 that every tensor-memory launch stamps with role milestones */
void rwkvq_tc_set_trace(void* device_buffer) { g_trace = reinterpret_cast<unsigned long long*>(device_buffer); }

int64_t rwkvq_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t nmat) {
    if (M <= 0 || N <= 0 || K <= 0 || nmat <= 0) return kWsHeaderBytes;
    const int kchunks = (int)((K + kChunk - 1) / kChunk);
    const int64_t tiles = nmat * ((N + kTileP - 1) / kTileP);
    const int64_t total = tiles * kchunks;
    const int grid = (int)std::min<int64_t>(tc_grid(), total);
    return kWsHeaderBytes + tiles * max_slots_for(total, kchunks, grid) * M * kTileP * 4;
}

int32_t rwkvq_workspace_status(const void* workspace, int32_t* host_status) {
    RWKVQ_REQUIRE(workspace && host_status, RWKVQ_E_BADARG, "workspace_status: null pointer");
    const cudaError_t e = cudaMemcpy(host_status, reinterpret_cast<const int*>(workspace) + kWsCounterInts, sizeof(int32_t), cudaMemcpyDeviceToHost);
    RWKVQ_REQUIRE(e == cudaSuccess, RWKVQ_E_LAUNCH, "workspace_status: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

static void fill_common(TcArgs& a, int nmat, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldo, int32_t div_mode, uint32_t flags) {
    if (a.ffn_amax == nullptr) flags &= ~RWKVQ_FLAG_RELU2;      // only rwkvq_tc_gemm_fp8_relu2 sets the target first
    a.nmat = nmat; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldo = ldo; a.div_mode = div_mode; a.flags = flags;
}

int32_t rwkvq_tc_gemv_fp8(const void* x, int32_t x_dtype, const float* awq, const uint8_t* w, int64_t ldw, const float* w_scale,
                          void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode,
                          uint32_t flags, void* workspace, int64_t workspace_bytes, void* stream) {
    TcArgs a{};
    a.x[0] = x; a.awq[0] = awq; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    fill_common(a, 1, M, N, K, ldx, ldo, div_mode, flags);
    TcCall c{};
    c.kind = KIND_F8; c.fused = true; c.x_dtype = x_dtype; c.w[0] = w; c.ldw = ldw; c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, "tc_gemv_fp8");
}

int32_t rwkvq_tc_gemv_fp8_rkv(const void* xr, const void* xk, const void* xv, int32_t x_dtype, const float* awq_r,
                              const float* awq_k, const uint8_t* wr, const uint8_t* wk, const uint8_t* wv, int64_t ldw,
                              const float* sr, const float* sk, const float* sv, void* out_r, void* out_k, void* out_v,
                              int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t ldx, int32_t div_mode, uint32_t flags,
                              void* workspace, int64_t workspace_bytes, void* stream) {
    TcArgs a{};
    a.x[0] = xr; a.x[1] = xk; a.x[2] = xv; a.awq[0] = awq_r; a.awq[1] = awq_k;
    a.ws[0] = sr; a.ws[1] = sk; a.ws[2] = sv;
    a.out[0] = (__half*)out_r; a.out[1] = (__half*)out_k; a.out[2] = (__half*)out_v;
    fill_common(a, 3, M, N, K, ldx, ldo, div_mode, flags);
    TcCall c{};
    c.kind = KIND_F8; c.fused = true; c.x_dtype = x_dtype; c.w[0] = wr; c.w[1] = wk; c.w[2] = wv; c.ldw = ldw;
    c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, "tc_gemv_fp8_rkv");
}

int32_t rwkvq_tc_gemv_int8(const void* x, int32_t x_dtype, const int8_t* w, int64_t ldw, const float* w_scale, void* out_f16,
                           int64_t ldo, int32_t* acc_out, int64_t ldacc, int64_t M, int64_t N, int64_t K, int64_t ldx,
                           int32_t div_mode, uint32_t flags, void* workspace, int64_t workspace_bytes, void* stream) {
    TcArgs a{};
    a.x[0] = x; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16; a.acc[0] = acc_out; a.ldacc = ldacc;
    fill_common(a, 1, M, N, K, ldx, ldo, div_mode, flags);
    RWKVQ_REQUIRE(acc_out == nullptr || ldacc >= N, RWKVQ_E_SHAPE, "tc_gemv_int8: ldacc < N");
    TcCall c{};
    c.kind = KIND_I8; c.fused = true; c.x_dtype = x_dtype; c.w[0] = w; c.ldw = ldw; c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, "tc_gemv_int8");
}

int32_t rwkvq_tc_gemv_int8_rkv(const void* xr, const void* xk, const void* xv, int32_t x_dtype, const int8_t* wr,
                               const int8_t* wk, const int8_t* wv, int64_t ldw, const float* sr, const float* sk,
                               const float* sv, void* out_r, void* out_k, void* out_v, int64_t ldo, int64_t M, int64_t N,
                               int64_t K, int64_t ldx, int32_t div_mode, uint32_t flags, void* workspace,
                               int64_t workspace_bytes, void* stream) {
    TcArgs a{};
    a.x[0] = xr; a.x[1] = xk; a.x[2] = xv;
    const bool shared = (flags & RWKVQ_FLAG_INT8_SHARED_WSCALE) != 0;
    a.ws[0] = sr; a.ws[1] = shared ? sr : sk; a.ws[2] = shared ? sr : sv;
    a.out[0] = (__half*)out_r; a.out[1] = (__half*)out_k; a.out[2] = (__half*)out_v;
    fill_common(a, 3, M, N, K, ldx, ldo, div_mode, flags);
    TcCall c{};
    c.kind = KIND_I8; c.fused = true; c.x_dtype = x_dtype; c.w[0] = wr; c.w[1] = wk; c.w[2] = wv; c.ldw = ldw;
    c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, "tc_gemv_int8_rkv");
}

int32_t rwkvq_tc_gemm_fp8(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax, const uint8_t* w,
                          int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                          int32_t div_mode, uint32_t flags, void* workspace, int64_t workspace_bytes, void* stream) {
    TcArgs a{};
    a.a_scale[0] = amax; a.amax_is_amax = amax_is_amax; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    fill_common(a, 1, M, N, K, 0, ldo, div_mode, flags);
    TcCall c{};
    c.kind = KIND_F8; c.w[0] = w; c.ldw = ldw; c.codes[0] = a_codes; c.lda = lda; c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, "tc_gemm_fp8");
}

/* FP8 projection of a few rows in ONE launch on the tensor-memory path: K split across a thread-block cluster, the
 * activation quantization (per-call abs-max, e4m3 codes) done inside by the CTAs on their own K slices, partial sums
 * exchanged through distributed shared memory.  Same bits as rwkvq_actq_fp8_fused + rwkvq_tc_gemm_fp8 on the same
 * inputs.  rwkvq_tc_cluster_gemv_route(M, N, K): 1 where this form applies (up to 32 rows, matrices with few 128-row
 * tiles); flags: RWKVQ_FLAG_AMAX_AFTER_BF16, RWKVQ_FLAG_QUANT_FROM_BF16, RWKVQ_FLAG_WSCALE_PER_ROW, RWKVQ_FLAG_OUT_VIA_BF16. */
int32_t rwkvq_tc_cluster_gemv_route(int64_t M, int64_t N, int64_t K) { return tcsq_eligible(M, N, K) ? 1 : 0; }

int32_t rwkvq_tc_cluster_gemv_fp8(const void* x, int32_t x_dtype, int64_t ldx, const uint8_t* w, int64_t ldw, const float* w_scale,
                                  void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, int32_t div_mode, uint32_t flags,
                                  void* stream) {
    const char* who = "tc_cluster_gemv_fp8";
    RWKVQ_REQUIRE(x && w && w_scale && out_f16, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, x_dtype);
    RWKVQ_REQUIRE(div_mode == RWKVQ_DIV_IEEE || div_mode == RWKVQ_DIV_FULL, RWKVQ_E_BADARG, "%s: div_mode %d", who, div_mode);
    RWKVQ_REQUIRE(M >= 0 && N >= 0 && K >= 0 && ldo >= N, RWKVQ_E_SHAPE, "%s: M=%lld N=%lld K=%lld ldo=%lld", who, (long long)M, (long long)N, (long long)K, (long long)ldo);
    if (M == 0 || N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(tcsq_eligible(M, N, K), RWKVQ_E_SHAPE, "%s: %lld x %lld x %lld is not a shape of this form (see rwkvq_tc_cluster_gemv_route)", who,
                  (long long)M, (long long)N, (long long)K);
    RWKVQ_REQUIRE(aligned16(x) && ldx % 8 == 0 && ldx >= K, RWKVQ_E_ALIGN, "%s: activation rows must be 16-byte aligned", who);
    TcArgs a{};
    a.x[0] = x; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    fill_common(a, 1, M, N, K, ldx, ldo, div_mode, flags & ~RWKVQ_FLAG_RELU2);
    return run_tcsq(a, w, ldw, x_dtype, (cudaStream_t)stream, who);
}

/* 1 if rwkvq_tc_gemm_fp8_push accepts this shape: the tiled GEMM form runs it (more rows than the few-token kernels
 * take). */
int32_t rwkvq_tc_gemm_can_push(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 16) return 0;
    return !takes_swap_route(M, N, K, 1, false) && !tcs_eligible(M, N, K, 0, 1);
}

/* rwkvq_tc_gemm_fp8 fused with the all-gather of a column-split projection: see rwkvq_tc_gemm_nvfp4_push for
 * peer_out / peer_flag / epoch.  Only shapes for which rwkvq_tc_gemm_can_push() is 1; no RELU2 flag. */
int32_t rwkvq_tc_gemm_fp8_push(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax, const uint8_t* w,
                               int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                               int32_t div_mode, uint32_t flags, void* workspace, int64_t workspace_bytes, void* const* peer_out,
                               void* const* peer_flag, int32_t npeers, uint32_t epoch, void* stream) {
    const char* who = "tc_gemm_fp8_push";
    RWKVQ_REQUIRE(M > 0 && N > 0, RWKVQ_E_SHAPE, "%s: empty result (the peers would wait for a signal that never comes)", who);
    TcArgs a{};
    const int32_t rc = make_push(&a.push, workspace, workspace_bytes, out_f16, peer_out, peer_flag, npeers, epoch, who);
    if (rc != RWKVQ_OK) return rc;
    a.a_scale[0] = amax; a.amax_is_amax = amax_is_amax; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    fill_common(a, 1, M, N, K, 0, ldo, div_mode, flags & ~RWKVQ_FLAG_RELU2);
    TcCall c{};
    c.kind = KIND_F8; c.w[0] = w; c.ldw = ldw; c.codes[0] = a_codes; c.lda = lda; c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, who);
}

/* rwkvq_tc_gemm_int8 fused with the all-gather of a column-split projection (no accumulator output in this form). */
int32_t rwkvq_tc_gemm_int8_push(const int8_t* a_codes, int64_t lda, const float* a_scales, const int8_t* w, int64_t ldw,
                                const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, uint32_t flags,
                                void* workspace, int64_t workspace_bytes, void* const* peer_out, void* const* peer_flag, int32_t npeers,
                                uint32_t epoch, void* stream) {
    const char* who = "tc_gemm_int8_push";
    RWKVQ_REQUIRE(M > 0 && N > 0, RWKVQ_E_SHAPE, "%s: empty result (the peers would wait for a signal that never comes)", who);
    TcArgs a{};
    const int32_t rc = make_push(&a.push, workspace, workspace_bytes, out_f16, peer_out, peer_flag, npeers, epoch, who);
    if (rc != RWKVQ_OK) return rc;
    a.a_scale[0] = a_scales; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    fill_common(a, 1, M, N, K, 0, ldo, RWKVQ_DIV_IEEE, flags & ~RWKVQ_FLAG_RELU2);
    TcCall c{};
    c.kind = KIND_I8; c.w[0] = w; c.ldw = ldw; c.codes[0] = a_codes; c.lda = lda; c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, who);
}

int32_t rwkvq_tc_gemm_int8(const int8_t* a_codes, int64_t lda, const float* a_scales, const int8_t* w, int64_t ldw,
                           const float* w_scale, void* out_f16, int64_t ldo, int32_t* acc_out, int64_t ldacc, int64_t M,
                           int64_t N, int64_t K, uint32_t flags, void* workspace, int64_t workspace_bytes, void* stream) {
    TcArgs a{};
    a.a_scale[0] = a_scales; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16; a.acc[0] = acc_out; a.ldacc = ldacc;
    fill_common(a, 1, M, N, K, 0, ldo, RWKVQ_DIV_IEEE, flags);
    RWKVQ_REQUIRE(acc_out == nullptr || ldacc >= N, RWKVQ_E_SHAPE, "tc_gemm_int8: ldacc < N");
    TcCall c{};
    c.kind = KIND_I8; c.w[0] = w; c.ldw = ldw; c.codes[0] = a_codes; c.lda = lda; c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, "tc_gemm_int8");
}

int32_t rwkvq_tc_gemm_fp8_rkv(const uint8_t* codes_r, const uint8_t* codes_k, const uint8_t* codes_v, int64_t lda, const float* amax3,
                              int32_t amax_is_amax, const uint8_t* wr, const uint8_t* wk, const uint8_t* wv, int64_t ldw, const float* sr,
                              const float* sk, const float* sv, void* out_r, void* out_k, void* out_v, int64_t ldo, int64_t M,
                              int64_t N, int64_t K, int32_t div_mode, uint32_t flags, void* workspace, int64_t workspace_bytes,
                              void* stream) {
    RWKVQ_REQUIRE(amax3 != nullptr, RWKVQ_E_BADARG, "tc_gemm_fp8_rkv: null amax");
    TcArgs a{};
    a.a_scale[0] = amax3; a.a_scale[1] = amax3 + 1; a.a_scale[2] = amax3 + 2; a.amax_is_amax = amax_is_amax;
    a.ws[0] = sr; a.ws[1] = sk; a.ws[2] = sv;
    a.out[0] = (__half*)out_r; a.out[1] = (__half*)out_k; a.out[2] = (__half*)out_v;
    fill_common(a, 3, M, N, K, 0, ldo, div_mode, flags);
    TcCall c{};
    c.kind = KIND_F8; c.w[0] = wr; c.w[1] = wk; c.w[2] = wv; c.ldw = ldw; c.codes[0] = codes_r; c.codes[1] = codes_k; c.codes[2] = codes_v;
    c.lda = lda; c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, "tc_gemm_fp8_rkv");
}

int32_t rwkvq_tc_gemm_int8_rkv(const int8_t* codes_r, const int8_t* codes_k, const int8_t* codes_v, int64_t lda, const float* scales_r,
                               const float* scales_k, const float* scales_v, const int8_t* wr, const int8_t* wk, const int8_t* wv,
                               int64_t ldw, const float* sr, const float* sk, const float* sv, void* out_r, void* out_k, void* out_v,
                               int64_t ldo, int64_t M, int64_t N, int64_t K, uint32_t flags, void* workspace, int64_t workspace_bytes,
                               void* stream) {
    TcArgs a{};
    a.a_scale[0] = scales_r; a.a_scale[1] = scales_k; a.a_scale[2] = scales_v;
    const bool shared = (flags & RWKVQ_FLAG_INT8_SHARED_WSCALE) != 0;
    a.ws[0] = sr; a.ws[1] = shared ? sr : sk; a.ws[2] = shared ? sr : sv;
    a.out[0] = (__half*)out_r; a.out[1] = (__half*)out_k; a.out[2] = (__half*)out_v;
    fill_common(a, 3, M, N, K, 0, ldo, RWKVQ_DIV_IEEE, flags);
    TcCall c{};
    c.kind = KIND_I8; c.w[0] = wr; c.w[1] = wk; c.w[2] = wv; c.ldw = ldw; c.codes[0] = codes_r; c.codes[1] = codes_k; c.codes[2] = codes_v;
    c.lda = lda; c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, "tc_gemm_int8_rkv");
}

/* NVFP4 projection of one to four tokens in ONE launch (activation quantization inside the cluster split-K kernel);
 * same bits as rwkvq_actq_nvfp4_fused followed by rwkvq_tc_gemm_nvfp4.  Sizes: rwkvq_tc_gemv_nvfp4_fused_route() == 1. */
int32_t rwkvq_tc_gemv_nvfp4_fused_route(int64_t M, int64_t N, int64_t K) { return tcsn_eligible(M, N, K) ? 1 : 0; }

int32_t rwkvq_tc_gemv_nvfp4_fused(const void* x, int32_t x_dtype, int64_t ldx, const uint8_t* w_codes, int64_t ldw,
                                  const uint8_t* w_scales_blocked, const float* w_tscale, void* out_f16, int64_t ldo, int64_t M, int64_t N,
                                  int64_t K, void* stream) {
    const char* who = "tc_gemv_nvfp4_fused";
    RWKVQ_REQUIRE(x && w_codes && w_scales_blocked && w_tscale && out_f16, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, x_dtype);
    RWKVQ_REQUIRE(M >= 0 && N >= 0 && K >= 0 && ldo >= N, RWKVQ_E_SHAPE, "%s: negative size or ldo < N", who);
    if (M == 0 || N == 0) return RWKVQ_OK;
    RWKVQ_REQUIRE(tcsn_eligible(M, N, K), RWKVQ_E_SHAPE, "%s: M=%lld N=%lld K=%lld is not served by the one-launch kernel (see %s_route)", who,
                  (long long)M, (long long)N, (long long)K, who);
    RWKVQ_REQUIRE(aligned16(x) && ldx % 8 == 0 && ldx >= K, RWKVQ_E_ALIGN, "%s: activation rows must be 16-byte aligned", who);
    RWKVQ_REQUIRE(aligned16(w_scales_blocked), RWKVQ_E_ALIGN, "%s: blocked scales must be 16-byte aligned", who);
    TcArgs a{};
    a.x[0] = x; a.ws[0] = w_tscale; a.out[0] = (__half*)out_f16; a.sfw = w_scales_blocked;
    a.nmat = 1; a.M = (int)M; a.N = (int)N; a.K = (int)K; a.ldx = ldx; a.ldo = ldo; a.div_mode = RWKVQ_DIV_IEEE; a.flags = 0;
    return run_tcsn(a, w_codes, ldw, x_dtype, (cudaStream_t)stream, who);
}

/* rwkvq_tc_gemm_fp8 (tiled GEMM form, M >= 17) with the engine's relu_square folded into the epilogue: stores
 * h = fp16(max(y, 0)^2) and accumulates max|h| into ffn_scratch[0] (see rwkvq_gemv_fp8_relu2). */
int32_t rwkvq_tc_gemm_fp8_relu2(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax, const uint8_t* w,
                                int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                                int32_t div_mode, uint32_t flags, void* ffn_scratch, void* workspace, int64_t workspace_bytes,
                                void* stream) {
    RWKVQ_REQUIRE(ffn_scratch != nullptr && ((uintptr_t)ffn_scratch & 7) == 0, RWKVQ_E_BADARG, "tc_gemm_fp8_relu2: ffn_scratch must be 8 aligned bytes");
    RWKVQ_REQUIRE(!takes_swap_route(M, N, K, 1, false), RWKVQ_E_SHAPE, "tc_gemm_fp8_relu2: M=%lld runs the weight-streaming form; use rwkvq_gemv_fp8_relu2 for few rows",
                  (long long)M);
    TcArgs a{};
    a.a_scale[0] = amax; a.amax_is_amax = amax_is_amax; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    a.ffn_amax = reinterpret_cast<float*>(ffn_scratch);
    fill_common(a, 1, M, N, K, 0, ldo, div_mode, flags | RWKVQ_FLAG_RELU2);
    TcCall c{};
    c.kind = KIND_F8; c.w[0] = w; c.ldw = ldw; c.codes[0] = a_codes; c.lda = lda; c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, "tc_gemm_fp8_relu2");
}

/* The same for INT8 weights: stores h = fp16(max(y, 0)^2) and folds the maximum of h per TOKEN ROW into row_max[M]
 * (floats, zero before the call; rwkvq_actq_int8_given reads and clears them).  Tiled GEMM form only (M >= 17 and not
 * the weight-streaming form); runs the single-CTA kernel at every row count. */
int32_t rwkvq_tc_gemm_int8_relu2(const int8_t* a_codes, int64_t lda, const float* a_scales, const int8_t* w, int64_t ldw,
                                 const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K, uint32_t flags,
                                 float* row_max, void* workspace, int64_t workspace_bytes, void* stream) {
    RWKVQ_REQUIRE(row_max != nullptr && ((uintptr_t)row_max & 3) == 0, RWKVQ_E_BADARG, "tc_gemm_int8_relu2: row_max must be M floats");
    RWKVQ_REQUIRE(!takes_swap_route(M, N, K, 1, false), RWKVQ_E_SHAPE, "tc_gemm_int8_relu2: M=%lld runs the weight-streaming form; use rwkvq_gemv_int8_relu2 for few rows",
                  (long long)M);
    TcArgs a{};
    a.a_scale[0] = a_scales; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    a.ffn_amax = row_max;
    fill_common(a, 1, M, N, K, 0, ldo, RWKVQ_DIV_IEEE, flags | RWKVQ_FLAG_RELU2);
    TcCall c{};
    c.kind = KIND_I8; c.w[0] = w; c.ldw = ldw; c.codes[0] = a_codes; c.lda = lda; c.workspace = workspace; c.workspace_bytes = workspace_bytes;
    return run_tc(a, c, (cudaStream_t)stream, "tc_gemm_int8_relu2");
}

/* rwkvq_tc_gemm_fp8 without a caller workspace: the split-K partial sums, arrival counters and status word live in
 * an 8 MiB array that is part of the library image on every GPU.  Nothing is allocated, here or in anything this calls.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress); make that first call
 *     outside any stream capture.  Later calls only enqueue work.
 *   - Only calls that take the stream-K form (few tokens against a matrix with too many row tiles for the cluster
 *     kernel) keep partial sums in the scratch; such a call is refused with RWKVQ_E_WORKSPACE if rwkvq_workspace_bytes(M, N, K, 1) exceeds
 *     8 MiB (a matrix of more than about 60 000 rows).  Every other shape needs the header only and is accepted.
 *   - All calls on a device share the one array and it keeps what the previous call left in it; this entry point
 *     therefore clears the counters and the status word on `stream` before the kernel.  Two calls that can overlap
 *     on the GPU (different streams, or concurrent host threads on different streams) race on it: order them. */
int32_t rwkvq_tc_gemm_fp8_static(const uint8_t* a_codes, int64_t lda, const float* amax, int32_t amax_is_amax, const uint8_t* w,
                                 int64_t ldw, const float* w_scale, void* out_f16, int64_t ldo, int64_t M, int64_t N, int64_t K,
                                 int32_t div_mode, uint32_t flags, void* stream) {
    const char* who = "tc_gemm_fp8_static";
    // only the weight-streaming form (few tokens) keeps partial sums in the scratch; the tiled GEMM uses the status word alone
    const int64_t need = (M > 0 && N > 0 && K > 0 && takes_swap_route(M, N, K, 1, false) && !tcs_eligible(M, N, K, flags, 1))
                             ? rwkvq_workspace_bytes(M, N, K, 1) : kWsHeaderBytes;
    RWKVQ_REQUIRE(need <= (int64_t)kStaticScratchBytes, RWKVQ_E_WORKSPACE, "%s: this shape needs %lld bytes of scratch, the built-in array has %lld",
                  who, (long long)need, (long long)kStaticScratchBytes);
    void* ws = nullptr;
    int32_t rc = static_scratch_ptr(&ws);
    if (rc != RWKVQ_OK) return rc;
    const cudaError_t e = cudaMemsetAsync(ws, 0, (size_t)kWsHeaderBytes, (cudaStream_t)stream);
    RWKVQ_REQUIRE(e == cudaSuccess, RWKVQ_E_LAUNCH, "%s: cudaMemsetAsync: %s", who, cudaGetErrorString(e));
    TcArgs a{};
    a.a_scale[0] = amax; a.amax_is_amax = amax_is_amax; a.ws[0] = w_scale; a.out[0] = (__half*)out_f16;
    fill_common(a, 1, M, N, K, 0, ldo, div_mode, flags);
    TcCall c{};
    c.kind = KIND_F8; c.w[0] = w; c.ldw = ldw; c.codes[0] = a_codes; c.lda = lda; c.workspace = ws; c.workspace_bytes = (int64_t)kStaticScratchBytes;
    return run_tc(a, c, (cudaStream_t)stream, who);
}

/* The status word of the built-in array (RWKVQ_E_TIMEOUT if a bounded wait of a rwkvq_tc_gemm_fp8_static call gave up
 * since the last call cleared it).  Copies four bytes to the host: synchronizes, allocates nothing. */
int32_t rwkvq_tc_static_status(int32_t* host_status) {
    RWKVQ_REQUIRE(host_status != nullptr, RWKVQ_E_BADARG, "tc_static_status: null pointer");
    void* ws = nullptr;
    const int32_t rc = static_scratch_ptr(&ws);
    if (rc != RWKVQ_OK) return rc;
    return rwkvq_workspace_status(ws, host_status);
}

}  // extern "C"
