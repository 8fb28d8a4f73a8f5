// GEMM for FEW tokens (decode batches, short prefill chunks: up to 256 rows) on pre-quantized codes -- FP8 and INT8
// (W8A8) and, with block-scaled MMAs, NVFP4 (W4A4): the weights are the 128-row operand of tcgen05.mma, the tokens the
// other one (16 ... 128 per tile), and K is split across a THREAD-BLOCK CLUSTER.
//
// Why.  With few tokens the projection is a pure weight stream, and a matrix has far fewer 128-row tiles than the GPU
// has SMs (N = 4096: 32), so every tile's K range has to be shared by several CTAs.  Sharing it through global memory
// (partial sums to a scratch buffer, fence, arrival counter, last arriver adds them: the stream-K form in gemm_tc.cu)
// puts four dependent L2 round trips plus the reduction's own loads behind the end of the stream: 6-16 us measured at
// 16-32 tokens against 12 us for the stream itself.  Here the C CTAs of a cluster (C = 2, 4, 8) each stream 1/C of
// the tile's K range into their own tensor memory and exchange the partial sums through DISTRIBUTED SHARED MEMORY:
// CTA r owns 128/C of the tile's rows, every CTA stores its partial sums of those rows straight into CTA r's shared
// memory (st.shared::cluster) and arrives on CTA r's mbarrier; CTA r adds the C contributions in rank order
// (run-to-run identical) and writes fp16.  No scratch, no counters, nothing to clear, nothing between launches.
//
// Roles per CTA: warp 0 = TMA producer (one lane), warp 1 = tensor-memory owner and MMA issuer (one lane),
// warps 2-5 = epilogue / exchange.  Up to 64 tokens two CTAs fit an SM (about 105 KB of shared memory each); token
// tiles of 128 take an SM each.  The first pass over the
// ring loads weights BEFORE the dependency wait of programmatic dependent launch: they do not depend on the
// activation quantizer that runs in front.  Every wait is bounded; all CTAs of a cluster meet at a cluster barrier
// before any of them exits, so no CTA's shared memory is written after it has gone.
//
// NVFP4 (KIND_NF4): a ring stage carries 256 values of k per row (128 bytes of packed e2m1 codes) plus the 2 KB chunk
// of e4m3 block scales of the weight tile and of the token tile (the blocked order of rwkvq_nvfp4_pack_scales); the
// MMA issuer copies the chunks to tensor memory with tcgen05.cp (two alternating column sets behind the accumulator)
// and issues four tcgen05.mma.kind::mxf4nvf4.block_scale of K = 64 per stage.  Exchange and final pass are the same.
//
// Included by gemm_tc.cu (shares its argument structs and tensor maps).
#pragma once

namespace rwkvq {

constexpr int kTcsThreads = 192;
constexpr int kTcsMaxStages = 8;
constexpr int kTcsMaxM = 256;              // two token tiles of 128

struct TcsShared {
    uint64_t full[kTcsMaxStages], empty[kTcsMaxStages], tfull[3], rx, rxfree;
    uint32_t tmem_base;
    int abort_flag;
    float row_scale[3][128];     // INT8: the token rows' activation scales, fetched before the exchange
};

__device__ __forceinline__ uint32_t tcs_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void tcs_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void tcs_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t tcs_mapa(uint32_t local, uint32_t rank) {      // `local` in CTA `rank` of this cluster
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
// One warp-wide store of 32 consecutive words lands as one 128-byte packet in the peer's shared memory; 16-byte
// vector stores to 32 different rows were measured 1.8 x slower for the same bytes.
__device__ __forceinline__ void tcs_st_remote(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void tcs_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// the peers' stores that precede their arrivals become visible with an acquire at cluster scope
__device__ __forceinline__ bool tcs_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool tcs_wait_cluster(uint64_t* bar, uint32_t parity, const volatile int* abort_flag, unsigned long long limit_ns) {
#pragma unroll 1
    for (int i = 0; i < 4096; ++i)
        if (tcs_try_wait_cluster(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 1024; ++i) {
            if (tcs_try_wait_cluster(bar, parity)) return true;
            __nanosleep(64);
        }
        if (*abort_flag) return false;
        if (global_ns() - t0 > limit_ns) return false;
    }
}

__device__ __forceinline__ void tcs_abort(TcsShared& s, const TcArgs& a) {
    s.abort_flag = 1;
    if (a.status) atomicExch(a.status, RWKVQ_E_TIMEOUT);
}

// a.qtiles carries the cluster size C, a.ptiles the 128-row tiles of one matrix, a.max_slots the token tiles (of a.NB
// tokens); grid = token tiles * ptiles * C.  With three
// matrices (r, k, v) a CTA streams its K range of the same row tile of each matrix in turn into three accumulators;
// the exchange of one matrix overlaps the stream of the next.  The K split is the same as for a single matrix, so the
// three-in-one launch and three single launches give the same bits.
template <int KIND>
__global__ void __launch_bounds__(kTcsThreads, 2) gemm_tcs_kernel(const __grid_constant__ TcMaps maps, const TcArgs a) {
    using T = typename Acc<KIND == KIND_I8 ? QT_INT8 : QT_FP8>::T;
    constexpr uint32_t kSfBytes = KIND == KIND_NF4 ? 2 * kNfSfStage : 0;     // NVFP4: block scales of both tiles ride in the stage
    constexpr uint32_t kSfCol = 128;                                         // NVFP4: first tensor-memory column of the scale factors
    extern __shared__ uint8_t smem_raw[];
    __shared__ TcsShared s;
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t stage_bytes = kABytes + (uint32_t)a.NB * kChunk + kSfBytes;
    const uint32_t sf_off = kABytes + (uint32_t)a.NB * kChunk;
    T* rxbuf = reinterpret_cast<T*>(ring + (size_t)a.stages * stage_bytes);        // [C][Mt][R]: partial sums per source CTA, token, row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = a.qtiles, R = kTileP / C;
    const int rank = (int)tcs_ctarank();
    const int cid = (int)blockIdx.x / C;                     // cluster = (token tile, row tile), row tiles fastest
    const int prow = (cid % a.ptiles) * kTileP;
    const int m0 = (cid / a.ptiles) * a.NB, Mt = min(a.NB, a.M - m0);       // this cluster's tokens
    const int kc0 = a.kchunks * rank / C, kc1 = a.kchunks * (rank + 1) / C;
    const int nk = kc1 - kc0, total = a.nmat * nk;          // ring units of this CTA: matrix-major
    const uint32_t need_cols = KIND == KIND_NF4 ? 256u : (uint32_t)(a.nmat * a.acc_stride);     // NVFP4: accumulator, then two sets of scale columns
    const uint32_t tmem_cols = need_cols <= 32 ? 32u : (need_cols <= 64 ? 64u : (need_cols <= 128 ? 128u : (need_cols <= 256 ? 256u : 512u)));
    const volatile int* abort_flag = &s.abort_flag;

    griddep_launch_dependents();
    if (threadIdx.x == 0) tc_mark(a, 0);
    if (threadIdx.x == 0) {
        for (int i = 0; i < a.stages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        for (int i = 0; i < 3; ++i) mbar_init(&s.tfull[i], 1);
        mbar_init(&s.rx, (uint32_t)(C * (R >= 32 ? R / 32 : 1)));      // one arrival per sending warp (half warp) and CTA
        mbar_init(&s.rxfree, (uint32_t)C);                              // one arrival per owner that has emptied its buffer
        s.abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        for (int i = 0; i < a.nmat; ++i) {
            prefetch_tmap(&maps.w[i]);
            prefetch_tmap(&maps.a[i]);
        }
    }
    if (warp == 1) tmem_alloc(&s.tmem_base, tmem_cols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = s.tmem_base;
    tcs_cluster_arrive();            // this CTA's barriers exist; the matching wait comes just before the exchange
    if (threadIdx.x == 0) tc_mark(a, 1);

    if (warp == 0) {
        // ============================== TMA producer ==============================
        if (lane == 0) {
            const int npre = min(total, a.stages);
            const int64_t k64 = (int64_t)a.kchunks * 4;          // NVFP4: 512-byte scale chunks (128 rows x 64 k) per row tile
            for (int n = 0; n < npre; ++n) {           // weights first: they do not depend on the previous kernel
                const int mat = n / nk, kc = kc0 + (n - mat * nk);
                mbar_expect_tx(&s.full[n], stage_bytes);
                tma_load_2d(ring + (size_t)n * stage_bytes, &maps.w[mat], kc * kChunk, prow, &s.full[n]);
                if constexpr (KIND == KIND_NF4)
                    bulk_load_1d(ring + (size_t)n * stage_bytes + sf_off, a.sfw + ((int64_t)(prow / kTileP) * k64 + kc * 4) * kNfSfChunk, kNfSfStage, &s.full[n]);
            }
            tc_mark(a, 2);
            griddep_wait();                            // the activation codes are written by the previous kernel
            tc_mark(a, 3);
            for (int n = 0; n < total; ++n) {
                const int st = n % a.stages;
                const int mat = n / nk, kc = kc0 + (n - mat * nk);
                uint8_t* dst = ring + (size_t)st * stage_bytes;
                if (n >= npre) {
                    if (!mbar_wait(&s.empty[st], ((n / a.stages) & 1) ^ 1, abort_flag, a.wait_ns)) { tcs_abort(s, a); break; }
                    mbar_expect_tx(&s.full[st], stage_bytes);
                    tma_load_2d(dst, &maps.w[mat], kc * kChunk, prow, &s.full[st]);
                    if constexpr (KIND == KIND_NF4)
                        bulk_load_1d(dst + sf_off, a.sfw + ((int64_t)(prow / kTileP) * k64 + kc * 4) * kNfSfChunk, kNfSfStage, &s.full[st]);
                }
                tma_load_2d(dst + kABytes, &maps.a[mat], kc * kChunk, m0, &s.full[st]);
                if constexpr (KIND == KIND_NF4)
                    bulk_load_1d(dst + sf_off + kNfSfStage, a.sfa + ((int64_t)(m0 / kNfTileM) * k64 + kc * 4) * kNfSfChunk, kNfSfStage, &s.full[st]);
            }
            tc_mark(a, 10);
        }
    } else if (warp == 1) {
        // ============================== MMA issuer ==============================
        if (lane == 0) {
            const uint32_t idesc = KIND == KIND_NF4 ? nvfp4_idesc(a.NB) : umma_idesc(KIND, kTileP, a.NB);
            for (int n = 0; n < total; ++n) {
                const int st = n % a.stages;
                const int mat = n / nk, i = n - mat * nk;
                if (!mbar_wait(&s.full[st], (n / a.stages) & 1, abort_flag, a.wait_ns)) { tcs_abort(s, a); break; }
                tc_fence_after_sync();
                const uint32_t sa = smem_u32(ring + (size_t)st * stage_bytes);
                const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sa + kABytes);
                const uint32_t d = tmem_base + (uint32_t)(mat * a.acc_stride);
                if constexpr (KIND == KIND_NF4) {
                    // scale factors of this stage (weights = the 128-row operand, tokens the other): two alternating
                    // column sets, so a copy never lands in columns the previous stage's MMAs may still be reading
                    const uint32_t tsfa = tmem_base + kSfCol + (uint32_t)(n & 1) * 64, tsfb = tsfa + 16;
                    const uint32_t ssf = sa + sf_off;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        tc_cp_sf(tsfa + k * 4, sf_desc(ssf + k * kNfSfChunk));
                        tc_cp_sf(tsfb + k * 4, sf_desc(ssf + kNfSfStage + k * kNfSfChunk));
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc_mma_nvfp4(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, tsfa + k * 4, tsfb + k * 4, (i > 0 || k > 0) ? 1u : 0u);
                } else {
#pragma unroll
                    for (int k = 0; k < kChunk / 32; ++k)
                        tc_mma<KIND>(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit(&s.empty[st]);
                if (i == nk - 1) tc_commit(&s.tfull[mat]);
                if (n == 0) tc_mark(a, 5);
            }
            tc_mark(a, 6);
        }
    }
    __syncwarp();                    // single-lane roles: the other lanes wait here for their lane 0
    tcs_cluster_wait();              // every CTA of the cluster has initialised its barriers
    if (warp < 2) tcs_cluster_arrive();      // these warps never touch a peer's shared memory (the epilogue warps arrive after their last store)

    if (warp >= 2) {
        // ============================== exchange + epilogue ==============================
        griddep_wait();
        const int q = warp & 3;                         // TMEM lane quarter this warp may read
        const int et = (warp - 2) * 32 + lane;          // thread index inside the epilogue group
        const int l = q * 32 + lane;                    // row of the tile held by this thread
        const uint32_t owner = (uint32_t)(l / R);
        const int lr = l - (int)owner * R;
        const uint32_t remote = tcs_mapa(smem_u32(rxbuf), owner) + (uint32_t)(((size_t)rank * Mt * R + lr) * 4);
        const uint32_t remote_rx = tcs_mapa(smem_u32(&s.rx), owner);
        // what the final pass needs from global memory is fetched now, not behind the exchange: a thread of the final
        // pass keeps EIGHT consecutive weight rows (R is a multiple of 16) and walks the tokens -- two 16-byte loads per
        // contribution, one 16-byte store per token (one row per thread and 2-byte stores took 9.5 us at 256 tokens)
        const int gpr = R >> 3, my_cg = et % gpr, my_m0 = et / gpr, m_step = 128 / gpr;
        const int my_row = prow + rank * R + my_cg * 8;
        const bool per_row = (a.flags & RWKVQ_FLAG_WSCALE_PER_ROW) != 0;
        float act_scale[3];
        for (int i = 0; i < a.nmat; ++i) {
            act_scale[i] = 0.f;
            if constexpr (KIND != KIND_I8) {
                const float v = __ldg(a.a_scale[i]);
                act_scale[i] = a.amax_is_amax ? div_mode_f32(fmaxf(v, 1e-12f), 448.f, a.div_mode) : v;
            } else {
                if (et < Mt) s.row_scale[i][et] = __ldg(a.a_scale[i] + m0 + et);      // read again only behind the named barrier below
            }
        }
        if constexpr (KIND == KIND_I8) named_bar_sync(1, 128);
        for (int mat = 0; mat < a.nmat; ++mat) {
            float wrow[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) wrow[j] = __ldg(a.ws[mat] + (per_row ? min(my_row + j, a.N - 1) : 0));
            bool have = mbar_wait(&s.tfull[mat], 0, abort_flag, a.wait_ns);
            if (!have) tcs_abort(s, a);
            have = __all_sync(0xffffffffu, have);       // the tensor-memory loads below are warp-wide
            tc_fence_after_sync();
            if (et == 0 && mat == a.nmat - 1) tc_mark(a, 7);
            // the owners' buffers are reused from matrix to matrix: every owner reports when it has emptied its own
            if (mat > 0 && !tcs_wait_cluster(&s.rxfree, (uint32_t)((mat - 1) & 1), abort_flag, a.wait_ns)) tcs_abort(s, a);
            // this CTA's partial sums of row l go to slot `rank` of the owner's buffer (zeros after a timeout, so that
            // the peers' waits end)
            const uint32_t taddr = tmem_base + (uint32_t)(mat * a.acc_stride) + ((uint32_t)(q * 32) << 16);
            for (int c0 = 0; c0 < Mt; c0 += 32) {            // two tensor-memory loads in flight, then 32 warp-wide peer stores
                uint32_t r[16], r2[16];
                if (have) {
                    tmem_ld16(taddr + c0, r);
                    if (c0 + 16 < Mt) tmem_ld16(taddr + c0 + 16, r2);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = r2[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (c0 + j < Mt) tcs_st_remote(remote + (uint32_t)((c0 + j) * R * 4), r[j]);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (c0 + 16 + j < Mt) tcs_st_remote(remote + (uint32_t)((c0 + 16 + j) * R * 4), r2[j]);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane % min(R, 32) == 0) tcs_arrive_remote(remote_rx);
            if (et == 0 && mat == a.nmat - 1) tc_mark(a, 8);
            if (mat == a.nmat - 1) tcs_cluster_arrive();      // this thread's last access to a peer's shared memory is behind it
            // ---- this CTA's rows: add the C contributions in rank order, scale, store
            const bool got = tcs_wait_cluster(&s.rx, (uint32_t)(mat & 1), abort_flag, a.wait_ns);
            if (!got) tcs_abort(s, a);
            if (et == 0 && mat == a.nmat - 1) tc_mark(a, 9);
            if (got && !*abort_flag && my_row < a.N) {
                const bool vec = (a.ldo & 7) == 0 && (reinterpret_cast<uintptr_t>(a.out[mat]) & 15) == 0 && my_row + 8 <= a.N;
                for (int m = my_m0; m < Mt; m += m_step) {
                    T sum[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) sum[j] = 0;
#pragma unroll
                    for (int src = 0; src < 8; ++src)          // the contributions are added in rank order
                        if (src < C) {
                            const uint4* p = reinterpret_cast<const uint4*>(rxbuf + ((size_t)src * Mt + m) * R + my_cg * 8);
                            const uint4 lo = p[0], hi = p[1];
                            const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                if constexpr (KIND != KIND_I8) sum[j] += __uint_as_float(w[j]);
                                else sum[j] += (int32_t)w[j];
                            }
                        }
                    float tok_scale;
                    if constexpr (KIND != KIND_I8) tok_scale = act_scale[mat];
                    else tok_scale = s.row_scale[mat][m];
                    if constexpr (KIND == KIND_I8) {
                        if (a.acc[mat]) {
                            int32_t* ap = a.acc[mat] + (int64_t)(m0 + m) * a.ldacc + my_row;
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (my_row + j < a.N) ap[j] = sum[j];
                        }
                    }
                    uint32_t h[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float f0 = (float)sum[2 * j] * (tok_scale * wrow[2 * j]), f1 = (float)sum[2 * j + 1] * (tok_scale * wrow[2 * j + 1]);
                        if (a.flags & RWKVQ_FLAG_OUT_VIA_BF16) {
                            f0 = bf16_round(f0);
                            f1 = bf16_round(f1);
                        }
                        const __half2 hh = __floats2half2_rn(f0, f1);
                        h[j] = *reinterpret_cast<const uint32_t*>(&hh);
                    }
                    __half* o = a.out[mat] + (int64_t)(m0 + m) * a.ldo + my_row;
                    if (vec) {
                        *reinterpret_cast<uint4*>(o) = make_uint4(h[0], h[1], h[2], h[3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (my_row + j < a.N) o[j] = __ushort_as_half((unsigned short)((h[j >> 1] >> ((j & 1) * 16)) & 0xffff));
                    }
                }
            }
            if (mat + 1 < a.nmat) {                    // this CTA's buffer is empty: tell every sender of the cluster
                named_bar_sync(1, 128);
                if (et < C) tcs_arrive_remote(tcs_mapa(smem_u32(&s.rxfree), (uint32_t)et));
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, tmem_cols);
    }
    if (threadIdx.x == 64) tc_mark(a, 11);
    tcs_cluster_wait();              // nobody leaves while a peer may still store into its shared memory
    if (threadIdx.x == 64) tc_mark(a, 12);
}

// ---------------------------------------------------------------------------------------------------------------
// The same kernel with the FP8 activation quantization INSIDE (one launch per projection, up to 32 rows).  A cluster
// spans all of K, and a CTA needs the codes of ITS K slice only: four more warps read that slice of the activations,
// the CTAs exchange their abs-max through distributed shared memory (one float per CTA, one mbarrier), and the same
// warps then write the e4m3 codes of each 128-byte step straight into the ring stage -- in the 128-byte-swizzled layout
// a TMA load would have produced -- while the TMA warp loads only the weights.  No quantizer launch in front, no codes
// in global memory; amax, codes and K split are those of the two-launch route, so the results are the same bits.
// Measured SLOWER than the two launches on the FFN value shape (16 rows: 23.2 against 18.7 us): each of the 32 clusters
// reads and quantizes the whole block again (the same 512 KB from L2, twice), whereas the quantizer kernel does it once
// while this kernel's weight prefetch already runs.  Kept as an entry point of its own; the dispatcher does not use it.
constexpr int kTcsqThreads = 320;
constexpr int kTcsqMaxM = 32;

struct TcsqShared {
    TcsShared b;
    uint64_t amaxbar;            // one arrival per CTA of the cluster
    float amax_part[8];          // slot r: abs-max of CTA r's slice
    float amax;                  // max over the cluster = over the whole block of activations
    float red[4];
};

__device__ __forceinline__ void tcs_st_remote_f32(uint32_t cluster_addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

template <int DT>
__global__ void __launch_bounds__(kTcsqThreads, 2) gemm_tcsq_kernel(const __grid_constant__ TcMaps maps, const TcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ TcsqShared sq;
    TcsShared& s = sq.b;
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t stage_bytes = kABytes + (uint32_t)a.NB * kChunk;
    float* rxbuf = reinterpret_cast<float*>(ring + (size_t)a.stages * stage_bytes);    // [C][M][R]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = a.qtiles, R = kTileP / C;
    const int rank = (int)tcs_ctarank();
    const int prow = ((int)blockIdx.x / C) * kTileP;
    const int Mt = a.M;
    const int kc0 = a.kchunks * rank / C, kc1 = a.kchunks * (rank + 1) / C, nk = kc1 - kc0;
    const uint32_t tmem_cols = 32u;                          // one accumulator of at most 32 tokens
    const volatile int* abort_flag = &s.abort_flag;

    griddep_launch_dependents();
    if (threadIdx.x == 0) {
        for (int i = 0; i < a.stages; ++i) {
            mbar_init(&s.full[i], 2);                         // the TMA warp's expect_tx arrival and the quantizer's
            mbar_init(&s.empty[i], 1);
        }
        mbar_init(&s.tfull[0], 1);
        mbar_init(&s.rx, (uint32_t)(C * (R >= 32 ? R / 32 : 1)));
        mbar_init(&sq.amaxbar, (uint32_t)C);
        s.abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tmap(&maps.w[0]);
    }
    if (warp == 1) tmem_alloc(&s.tmem_base, tmem_cols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = s.tmem_base;
    tcs_cluster_arrive();

    if (warp == 0) {
        // ============================== TMA producer: weights only, nothing to wait for ==============================
        if (lane == 0) {
            for (int n = 0; n < nk; ++n) {
                const int st = n % a.stages;
                if (n >= a.stages && !mbar_wait(&s.empty[st], ((n / a.stages) & 1) ^ 1, abort_flag, a.wait_ns)) { tcs_abort(s, a); break; }
                mbar_expect_tx(&s.full[st], kABytes);
                tma_load_2d(ring + (size_t)st * stage_bytes, &maps.w[0], (kc0 + n) * kChunk, prow, &s.full[st]);
            }
        }
    } else if (warp == 1) {
        // ============================== MMA issuer ==============================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(KIND_F8, kTileP, a.NB);
            for (int n = 0; n < nk; ++n) {
                const int st = n % a.stages;
                if (!mbar_wait(&s.full[st], (n / a.stages) & 1, abort_flag, a.wait_ns)) { tcs_abort(s, a); break; }
                tc_fence_after_sync();
                const uint32_t sa = smem_u32(ring + (size_t)st * stage_bytes);
                const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sa + kABytes);
#pragma unroll
                for (int k = 0; k < kChunk / 32; ++k)
                    tc_mma<KIND_F8>(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (n > 0 || k > 0) ? 1u : 0u);
                tc_commit(&s.empty[st]);
                if (n == nk - 1) tc_commit(&s.tfull[0]);
            }
        }
    }
    __syncwarp();
    tcs_cluster_wait();              // every CTA of the cluster has initialised its barriers
    if (warp < 2) tcs_cluster_arrive();

    if (warp >= 6) {
        // ============================== activation quantizer (4 warps) ==============================
        const int qt = (int)threadIdx.x - 6 * 32;
        const bool after_bf16 = (a.flags & RWKVQ_FLAG_AMAX_AFTER_BF16) != 0, from_bf16 = (a.flags & RWKVQ_FLAG_QUANT_FROM_BF16) != 0;
        const char* x = reinterpret_cast<const char*>(a.x[0]);
        const int kv = a.K >> 3;                                             // 16-byte vectors per row
        const int v0 = kc0 * 16, v1 = min(kc1 * 16, kv), vs = max(v1 - v0, 0);    // this CTA's vectors of every row
        griddep_wait();                                                      // the activations may come from the previous kernel
        // ---- pass 1: abs-max of the slice.  Dependent round trips to L2 are what this phase costs (the whole kernel
        // waits for the maximum), so a thread keeps 16 loads in flight.
        float m = 0.f;
        const int total = Mt * vs;
#pragma unroll 1
        for (int i0 = qt; i0 < total; i0 += 128 * 16) {
            uint4 v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int idx = i0 + j * 128;
                v[j] = make_uint4(0, 0, 0, 0);
                if (idx < total) {
                    const int r = idx / vs, c = idx - r * vs;
                    v[j] = *reinterpret_cast<const uint4*>(x + ((int64_t)r * a.ldx + (int64_t)(v0 + c) * 8) * 2);
                }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float2 f = cvt2<DT>(w[q]);
                    if (DT == RWKVQ_F16 && after_bf16) { f.x = bf16_round(f.x); f.y = bf16_round(f.y); }
                    m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
                }
            }
        }
        m = warp_max(m);
        if (lane == 0) sq.red[warp - 6] = m;
        named_bar_sync(2, 128);
        if (qt < C) {                                                        // this CTA's maximum into slot `rank` of every CTA
            const float mine = fmaxf(fmaxf(sq.red[0], sq.red[1]), fmaxf(sq.red[2], sq.red[3]));
            tcs_st_remote_f32(tcs_mapa(smem_u32(&sq.amax_part[rank]), (uint32_t)qt), mine);
            tcs_arrive_remote(tcs_mapa(smem_u32(&sq.amaxbar), (uint32_t)qt));
        }
        if (!tcs_wait_cluster(&sq.amaxbar, 0, abort_flag, a.wait_ns)) tcs_abort(s, a);
        float amax = sq.amax_part[0];
        for (int i = 1; i < C; ++i) amax = fmaxf(amax, sq.amax_part[i]);
        if (qt == 0) sq.amax = amax;
        const float inv = scale_inv(448.f, fmaxf(amax, 1e-12f), a.div_mode);
        // ---- pass 2: codes of one 128-byte step after the other, straight into the ring stage (128-byte swizzle: the
        // 16-byte piece j of row r sits at piece j ^ (r % 8) of its 128-byte row inside the 8-row atom)
        const int items = Mt * 8;                                            // (row, 16-code piece) pairs per step
        auto load_item = [&](int n, int it, uint4 (&v)[2]) {
            const int r = it >> 3, j = it & 7;
            const int vec = (kc0 + n) * 16 + j * 2;                          // first of the two vectors behind the piece
            const char* p = x + ((int64_t)r * a.ldx + (int64_t)vec * 8) * 2;
            v[0] = vec < kv ? *reinterpret_cast<const uint4*>(p) : make_uint4(0, 0, 0, 0);
            v[1] = vec + 1 < kv ? *reinterpret_cast<const uint4*>(p + 16) : make_uint4(0, 0, 0, 0);
        };
        auto codes8 = [&](const uint4& v) -> uint2 {
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t c[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float2 f = cvt2<DT>(w[q]);
                if (DT == RWKVQ_F16 && from_bf16) { f.x = bf16_round(f.x); f.y = bf16_round(f.y); }
                c[q] = e4m3x2(f.x * inv, f.y * inv);
            }
            return make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
        };
        // Each of the four warps takes every fourth step (four steps' loads are in flight at once); within its steps a
        // warp works in batches of 128 (row, piece) items, the next batch's loads issued before the current one is
        // converted.
        const int qw = warp - 6;
        const int nbatch = (items + 127) >> 7;
        auto load_batch = [&](int n, int bt, uint4 (&v)[4][2]) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int it = bt * 128 + j * 32 + lane;
                if (it < items) load_item(n, it, v[j]);
            }
        };
        uint4 cur[4][2], nxt[4][2];
        int n = qw, bt = 0;
        if (n < nk) load_batch(n, 0, cur);
#pragma unroll 1
        while (n < nk) {
            int n2 = n, bt2 = bt + 1;
            if (bt2 == nbatch) { bt2 = 0; n2 = n + 4; }
            if (n2 < nk) load_batch(n2, bt2, nxt);
            const int st = n % a.stages;
            if (bt == 0 && n >= a.stages) {                                  // lane 0 waits for the stage, the warp follows
                int okv = 1;
                if (lane == 0) okv = mbar_wait(&s.empty[st], ((n / a.stages) & 1) ^ 1, abort_flag, a.wait_ns) ? 1 : 0;
                okv = __shfl_sync(0xffffffffu, okv, 0);
                if (!okv) {
                    tcs_abort(s, a);
                    break;
                }
            }
            uint8_t* btile = ring + (size_t)st * stage_bytes + kABytes;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int it = bt * 128 + j * 32 + lane;
                if (it < items) {
                    const int r = it >> 3, pc = it & 7;
                    const uint2 lo = codes8(cur[j][0]), hi = codes8(cur[j][1]);
                    *reinterpret_cast<uint4*>(btile + (r >> 3) * 1024 + (r & 7) * 128 + ((pc ^ (r & 7)) << 4)) = make_uint4(lo.x, lo.y, hi.x, hi.y);
                }
            }
            if (bt == nbatch - 1) {
                fence_proxy_async();                                         // these generic-proxy stores are read by the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.full[st]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) { cur[j][0] = nxt[j][0]; cur[j][1] = nxt[j][1]; }
            n = n2;
            bt = bt2;
        }
        tcs_cluster_arrive();
    } else if (warp >= 2) {
        // ============================== exchange + epilogue ==============================
        const int q = warp & 3;
        const int et = (warp - 2) * 32 + lane;
        const int l = q * 32 + lane;
        const uint32_t owner = (uint32_t)(l / R);
        const int lr = l - (int)owner * R;
        const uint32_t remote = tcs_mapa(smem_u32(rxbuf), owner) + (uint32_t)(((size_t)rank * Mt * R + lr) * 4);
        const uint32_t remote_rx = tcs_mapa(smem_u32(&s.rx), owner);
        const int my_c = et % R, my_m0 = et / R, m_step = 128 / R;
        const int my_row = prow + rank * R + my_c;
        const bool per_row = (a.flags & RWKVQ_FLAG_WSCALE_PER_ROW) != 0;
        const float wrow = __ldg(a.ws[0] + (per_row ? min(my_row, a.N - 1) : 0));
        bool have = mbar_wait(&s.tfull[0], 0, abort_flag, a.wait_ns);
        if (!have) tcs_abort(s, a);
        have = __all_sync(0xffffffffu, have);
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
        for (int c0 = 0; c0 < Mt; c0 += 16) {
            uint32_t r[16];
            if (have) {
                tmem_ld16(taddr + c0, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (c0 + j < Mt) tcs_st_remote(remote + (uint32_t)((c0 + j) * R * 4), r[j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane % min(R, 32) == 0) tcs_arrive_remote(remote_rx);
        tcs_cluster_arrive();
        const bool got = tcs_wait_cluster(&s.rx, 0, abort_flag, a.wait_ns);
        if (!got) tcs_abort(s, a);
        if (got && !*abort_flag && my_row < a.N) {
            // the block's abs-max was written by the quantizer warps before their first arrival on a `full` barrier
            const float act_scale = div_mode_f32(fmaxf(sq.amax, 1e-12f), 448.f, a.div_mode);
            for (int m = my_m0; m < Mt; m += m_step) {
                float v[8];
#pragma unroll
                for (int src = 0; src < 8; ++src) v[src] = src < C ? rxbuf[((size_t)src * Mt + m) * R + my_c] : 0.f;
                float sum = 0.f;
#pragma unroll
                for (int src = 0; src < 8; ++src)
                    if (src < C) sum += v[src];
                float f = sum * (act_scale * wrow);
                if (a.flags & RWKVQ_FLAG_OUT_VIA_BF16) f = bf16_round(f);
                a.out[0][(int64_t)m * a.ldo + my_row] = __float2half_rn(f);
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, tmem_cols);
    }
    tcs_cluster_wait();
}

// ------------------------------------------------------------------------------------------------ host side
// Cluster size: as many CTAs per (128-row tile, token tile) as keep the whole grid resident at once -- two CTAs per SM
// up to 64 tokens, one per SM with token tiles of 128 -- at most 8 and at most one per two 128-byte steps of K.  It
// depends on the shape alone (not on how many matrices a launch carries), so a fused r/k/v launch and three single
// launches split K alike and give the same bits.
static int tcs_token_tile(int64_t M) { return M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128)); }
static int tcs_cluster_size(int64_t M, int64_t N, int64_t K) {
    const int64_t ptiles = (N + kTileP - 1) / kTileP, kchunks = (K + kChunk - 1) / kChunk;
    const int nb = tcs_token_tile(M);
    const int64_t units = ptiles * ((M + nb - 1) / nb), room = (int64_t)sm_count() * (nb <= 64 ? 2 : 1);
    static const int cmax = std::getenv("RWKVQ_TCS_CMAX") ? std::atoi(std::getenv("RWKVQ_TCS_CMAX")) : 8;
    int c = 1;
    while (c < cmax && units * (c * 2) <= room && kchunks >= c * 2) c <<= 1;
    return c;
}

// Measured on the 7.2B shapes: the cluster kernel wins where a matrix has few row tiles (N = 4096: 32), i.e. where the
// tiled GEMM form cannot give every SM a tile; with 128 row tiles (N = 16384) the GEMM form is as fast or faster.
static bool tcs_eligible(int64_t M, int64_t N, int64_t K, uint32_t flags, int nmat) {
    (void)nmat;                  // the K split and the grid are those of one matrix
    static const int on = std::getenv("RWKVQ_TCS") ? std::atoi(std::getenv("RWKVQ_TCS")) : 1;
    static const int64_t max_m = std::getenv("RWKVQ_TCS_MAX_M") ? std::atoll(std::getenv("RWKVQ_TCS_MAX_M")) : kTcsMaxM;
    if (!on || M < 1 || M > std::min<int64_t>(max_m, kTcsMaxM) || (flags & RWKVQ_FLAG_RELU2)) return false;
    const int c = tcs_cluster_size(M, N, K);
    // token tiles of 128 (65 ... 256 rows): measured faster than the tiled GEMM form only against a long K (FFN value,
    // K = 16384: 57 -> 29 us at 96 rows, 61 -> 52 us at 256); at K = 4096 the GEMM form wins from about 160 rows on and
    // the three-matrix launch everywhere
    return K >= 1024 && (M <= 64 ? c >= 4 : (c >= 2 && K >= 8192));
}

static int32_t run_tcs(TcArgs a, const TcCall& c, cudaStream_t st, const char* who) {
    const int64_t kbytes = c.kind == KIND_NF4 ? a.K / 2 : a.K;          // bytes of K per row: two e2m1 values per byte
    const int C = tcs_cluster_size(a.M, a.N, kbytes);
    a.NB = tcs_token_tile(a.M);
    a.ptiles = (a.N + kTileP - 1) / kTileP;
    a.qtiles = C;
    a.max_slots = (a.M + a.NB - 1) / a.NB;                       // token tiles
    a.acc_stride = std::max(a.NB, 32);
    if (a.status == nullptr) a.status = c.workspace ? reinterpret_cast<int*>(c.workspace) + kWsCounterInts : device_status_ptr();
    const size_t stage_bytes = kABytes + (size_t)a.NB * kChunk + (c.kind == KIND_NF4 ? 2 * kNfSfStage : 0);
    const size_t rx_bytes = (size_t)std::min(a.M, a.NB) * kTileP * 4;       // [C][tokens of a tile][128 / C] partial sums
    const size_t budget = a.NB <= 64 ? kTcSmemBudgetHalf : kTcSmemBudget;
    const int per_cta = (a.kchunks + C - 1) / C;
    a.stages = (int)std::min<size_t>(std::min<int>(kTcsMaxStages, per_cta * a.nmat), (budget - 1024 - rx_bytes) / stage_bytes);
    RWKVQ_REQUIRE(a.stages >= 2 || per_cta * a.nmat == 1, RWKVQ_E_SHAPE, "%s: shared memory leaves fewer than two ring stages", who);
    a.stages = std::max(a.stages, 1);
    TcMaps maps;
    for (int i = 0; i < a.nmat; ++i) {
        int32_t rc = make_map(&maps.w[i], c.w[i], a.N, kbytes, c.ldw, kTileP, who);
        if (rc) return rc;
        rc = make_map(&maps.a[i], c.codes[i], a.M, kbytes, c.lda, a.NB, who);
        if (rc) return rc;
    }
    auto kern = c.kind == KIND_F8 ? gemm_tcs_kernel<KIND_F8> : (c.kind == KIND_I8 ? gemm_tcs_kernel<KIND_I8> : gemm_tcs_kernel<KIND_NF4>);
    const int32_t rc = ensure_smem_optin(reinterpret_cast<const void*>(kern), (int)kTcSmemBudget, who);
    if (rc) return rc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(a.max_slots * a.ptiles * C));
    cfg.blockDim = dim3(kTcsThreads);
    cfg.dynamicSmemBytes = (size_t)a.stages * stage_bytes + rx_bytes + 1024;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl() ? 2 : 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kern, maps, a);
    if (err != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(err));
    }
    return check_launch(who);
}

// one-launch form: FP8, a single matrix, up to 32 rows, the shapes the cluster kernel takes anyway
static bool tcsq_eligible(int64_t M, int64_t N, int64_t K) {
    static const int on = std::getenv("RWKVQ_TCSQ") ? std::atoi(std::getenv("RWKVQ_TCSQ")) : 1;
    return on && M >= 1 && M <= kTcsqMaxM && K % 8 == 0 && tcs_eligible(M, N, K, 0, 1);
}

static int32_t run_tcsq(TcArgs a, const void* w, int64_t ldw, int x_dtype, cudaStream_t st, const char* who) {
    const int C = tcs_cluster_size(a.M, a.N, a.K);
    a.NB = tcs_token_tile(a.M);
    a.kchunks = (a.K + kChunk - 1) / kChunk;
    a.ptiles = (a.N + kTileP - 1) / kTileP;
    a.qtiles = C;
    a.max_slots = 1;
    a.acc_stride = 32;
    a.wait_ns = wait_limit_ns();
    a.status = device_status_ptr();
    const size_t stage_bytes = kABytes + (size_t)a.NB * kChunk;
    const size_t rx_bytes = (size_t)a.M * kTileP * 4;
    const int per_cta = (a.kchunks + C - 1) / C;
    a.stages = (int)std::min<size_t>(std::min<int>(kTcsMaxStages, per_cta), (kTcSmemBudgetHalf - 1024 - rx_bytes) / stage_bytes);
    RWKVQ_REQUIRE(a.stages >= 2 || per_cta == 1, RWKVQ_E_SHAPE, "%s: shared memory leaves fewer than two ring stages", who);
    a.stages = std::max(a.stages, 1);
    TcMaps maps;
    const int32_t rcm = make_map(&maps.w[0], w, a.N, a.K, ldw, kTileP, who);
    if (rcm) return rcm;
    auto kern = x_dtype == RWKVQ_F16 ? gemm_tcsq_kernel<RWKVQ_F16> : gemm_tcsq_kernel<RWKVQ_BF16>;
    const int32_t rc = ensure_smem_optin(reinterpret_cast<const void*>(kern), (int)kTcSmemBudget, who);
    if (rc) return rc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(a.ptiles * C));
    cfg.blockDim = dim3(kTcsqThreads);
    cfg.dynamicSmemBytes = (size_t)a.stages * stage_bytes + rx_bytes + 1024;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl() ? 2 : 1;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kern, maps, a);
    if (err != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(err));
    }
    return check_launch(who);
}

}  // namespace rwkvq
