// NVFP4 (W4A4) projection of ONE to FOUR tokens in ONE launch: the cluster split-K kernel of gemm_tcs.cuh (weights =
// the 128-row operand of tcgen05.mma.kind::mxf4nvf4.block_scale, K split across a thread-block cluster, partial sums
// through distributed shared memory) with the activation quantization inside.
//
// Why.  With so few tokens the block of activations is tiny (4 x 16384 values = 128 KB) and the call is a chain of
// launches that wait for one another: quantizer -> GEMM costs 13 us for a 38 MB matrix whose stream takes 6.  Here the
// CTAs of a cluster together span K, so four extra warps per CTA read that CTA's K slice of the activations ONCE into
// registers, the CTAs exchange their abs-max through distributed shared memory (one float per CTA, one mbarrier), and
// the same warps write the e2m1 codes -- in the 128-byte-swizzled layout a TMA load would have produced -- and the e4m3
// block scales -- in the 512-byte chunk layout tcgen05.cp copies -- of ALL ring steps of the slice into a token area of
// shared memory that stays put (16 rows x 128 bytes + 2 KB of scales per step), while the TMA warp streams only the
// weights and their scale chunks.  Amax, tensor scale, block scales, codes and the K split are those of
// rwkvq_actq_nvfp4_fused followed by the cluster kernel, so the results are the same bits.
// Measured as fast or SLOWER than those two launches (FFN value [4096, 16384], one token: 14.0 against 12.8 us; FFN key
// [16384, 4096]: 12.2 against 12.0): the separate quantizer is one small cluster launch that already runs under the
// GEMM's weight prefetch, and here the MMAs wait for the same abs-max exchange inside a heavier CTA.  Kept as an entry
// point of its own (rwkvq_tc_gemv_nvfp4_fused); the Python dispatcher takes it only on request.
//
// Included by gemm_tc.cu after gemm_tcs.cuh (shares its argument structs, tensor maps and cluster helpers).
#pragma once

namespace rwkvq {

constexpr int kTcsnThreads = 320;
constexpr int kTcsnMaxM = 4;
constexpr int kTcsnBlocksPerThread = 4;                     // 16-blocks of activations a quantizer thread keeps in registers
constexpr uint32_t kTcsnWStage = kABytes + kNfSfStage;      // ring stage: weight codes + their scale chunks
constexpr uint32_t kTcsnTokStage = 16 * kChunk + kNfSfStage; // token area per ring step: 16 code rows + scale chunks

struct TcsnShared {
    TcsShared b;
    uint64_t amaxbar;            // one arrival per CTA of the cluster
    uint64_t tokbar;             // the token area is complete
    float amax_part[8];          // slot r: abs-max of CTA r's slice
    float amax;                  // max over the cluster = over the whole block of activations
    float red[4];
};

template <int DT>
__global__ void __launch_bounds__(kTcsnThreads, 2) gemm_tcsn_kernel(const __grid_constant__ TcMaps maps, const TcArgs a) {
    constexpr uint32_t kSfCol = 128;                         // first tensor-memory column of the scale factors
    extern __shared__ uint8_t smem_raw[];
    __shared__ TcsnShared sq;
    TcsShared& s = sq.b;
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = a.qtiles, R = kTileP / C;
    const int rank = (int)tcs_ctarank();
    const int prow = ((int)blockIdx.x / C) * kTileP;
    const int Mt = a.M;
    const int kc0 = a.kchunks * rank / C, kc1 = a.kchunks * (rank + 1) / C, nk = kc1 - kc0;
    uint8_t* tok = ring + (size_t)a.stages * kTcsnWStage;                         // [max_slots steps][kTcsnTokStage]
    float* rxbuf = reinterpret_cast<float*>(tok + (size_t)a.max_slots * kTcsnTokStage);   // [C][Mt][R]
    const uint32_t tmem_cols = 256u;                         // accumulator, then two sets of scale columns
    const volatile int* abort_flag = &s.abort_flag;

    griddep_launch_dependents();
    if (threadIdx.x == 0) {
        for (int i = 0; i < a.stages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        mbar_init(&s.tfull[0], 1);
        mbar_init(&s.rx, (uint32_t)(C * (R >= 32 ? R / 32 : 1)));
        mbar_init(&sq.amaxbar, (uint32_t)C);
        mbar_init(&sq.tokbar, 1);
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
    tcs_cluster_arrive();            // this CTA's barriers exist; the matching wait comes before any remote access

    if (warp == 0) {
        // ============================== TMA producer: weights and their scales, nothing to wait for ==============================
        if (lane == 0) {
            const int64_t k64 = (int64_t)a.kchunks * 4;
            for (int n = 0; n < nk; ++n) {
                const int st = n % a.stages;
                if (n >= a.stages && !mbar_wait(&s.empty[st], ((n / a.stages) & 1) ^ 1, abort_flag, a.wait_ns)) { tcs_abort(s, a); break; }
                uint8_t* dst = ring + (size_t)st * kTcsnWStage;
                mbar_expect_tx(&s.full[st], kTcsnWStage);
                tma_load_2d(dst, &maps.w[0], (kc0 + n) * kChunk, prow, &s.full[st]);
                bulk_load_1d(dst + kABytes, a.sfw + ((int64_t)(prow / kTileP) * k64 + (int64_t)(kc0 + n) * 4) * kNfSfChunk, kNfSfStage, &s.full[st]);
            }
        }
    } else if (warp == 1) {
        // ============================== MMA issuer ==============================
        if (lane == 0) {
            const uint32_t idesc = nvfp4_idesc(16);
            bool ok = mbar_wait(&sq.tokbar, 0, abort_flag, a.wait_ns);          // token codes and scales are in place
            if (!ok) tcs_abort(s, a);
            for (int n = 0; n < nk && ok; ++n) {
                const int st = n % a.stages;
                if (!mbar_wait(&s.full[st], (n / a.stages) & 1, abort_flag, a.wait_ns)) { tcs_abort(s, a); break; }
                tc_fence_after_sync();
                const uint32_t sa = smem_u32(ring + (size_t)st * kTcsnWStage);
                const uint32_t sb = smem_u32(tok + (size_t)n * kTcsnTokStage);
                const uint32_t tsfa = tmem_base + kSfCol + (uint32_t)(n & 1) * 64, tsfb = tsfa + 16;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    tc_cp_sf(tsfa + k * 4, sf_desc(sa + kABytes + k * kNfSfChunk));
                    tc_cp_sf(tsfb + k * 4, sf_desc(sb + 16 * kChunk + k * kNfSfChunk));
                }
                const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sb);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tc_mma_nvfp4(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, tsfa + k * 4, tsfb + k * 4, (n > 0 || k > 0) ? 1u : 0u);
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
        const char* x = reinterpret_cast<const char*>(a.x[0]);
        const int per_step = Mt * 16;                        // 16-blocks per ring step (256 values of k per row)
        const int nblk = nk * per_step;                      // <= 128 * kTcsnBlocksPerThread (checked on the host)
        griddep_wait();                                      // the activations may come from the previous kernel
        // ---- this thread's blocks: two 16-byte vectors each, all loads in flight, kept for the codes
        uint4 v[kTcsnBlocksPerThread][2];
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < kTcsnBlocksPerThread; ++i) {
            const int b = qt + 128 * i;
            v[i][0] = v[i][1] = make_uint4(0, 0, 0, 0);
            if (b < nblk) {
                const int n = b / per_step, it = b - n * per_step, r = it >> 4, blk = it & 15;
                const char* p = x + ((int64_t)r * a.ldx + (int64_t)(kc0 + n) * 256 + blk * 16) * 2;
                v[i][0] = *reinterpret_cast<const uint4*>(p);
                v[i][1] = *reinterpret_cast<const uint4*>(p + 16);
            }
        }
#pragma unroll
        for (int i = 0; i < kTcsnBlocksPerThread; ++i) m = fmaxf(m, fmaxf(packed_absmax8<DT>(v[i][0]), packed_absmax8<DT>(v[i][1])));
        m = warp_max(m);
        if (lane == 0) sq.red[warp - 6] = m;
        named_bar_sync(2, 128);
        if (qt < C) {                                        // this CTA's maximum into slot `rank` of every CTA
            const float mine = fmaxf(fmaxf(sq.red[0], sq.red[1]), fmaxf(sq.red[2], sq.red[3]));
            tcs_st_remote_f32(tcs_mapa(smem_u32(&sq.amax_part[rank]), (uint32_t)qt), mine);
            tcs_arrive_remote(tcs_mapa(smem_u32(&sq.amaxbar), (uint32_t)qt));
        }
        if (!tcs_wait_cluster(&sq.amaxbar, 0, abort_flag, a.wait_ns)) tcs_abort(s, a);
        float amax = sq.amax_part[0];
        for (int i = 1; i < C; ++i) amax = fmaxf(amax, sq.amax_part[i]);
        amax = fmaxf(amax, 1e-12f);
        if (qt == 0) sq.amax = amax;
        const float pts = __fdiv_rn(amax, 2688.f);
        const float inv_pts = __fdiv_rn(1.f, pts), k448 = __fdiv_rn(448.f, amax);
        // ---- codes (two e2m1 per byte, 128-byte swizzle: the 16-byte piece j of row r sits at piece j ^ (r % 8)) and
        // block scales (chunk of 64 k: byte (r % 32) * 16 + (r / 32) * 4 + block % 4) of every step
#pragma unroll
        for (int i = 0; i < kTcsnBlocksPerThread; ++i) {
            const int b = qt + 128 * i;
            if (b < nblk) {
                const int n = b / per_step, it = b - n * per_step, r = it >> 4, blk = it & 15;
                const uint32_t wv[8] = {v[i][0].x, v[i][0].y, v[i][0].z, v[i][0].w, v[i][1].x, v[i][1].y, v[i][1].z, v[i][1].w};
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
                const float bs = e4m3_to_float(sc);
                uint32_t out[2] = {0u, 0u};
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    out[q >> 2] |= e2m1x2(__fdiv_rn(f[2 * q] * inv_pts, bs), __fdiv_rn(f[2 * q + 1] * inv_pts, bs)) << (8 * (q & 3));
                uint8_t* tn = tok + (size_t)n * kTcsnTokStage;
                *reinterpret_cast<uint2*>(tn + (r >> 3) * 1024 + (r & 7) * 128 + (((blk >> 1) ^ (r & 7)) << 4) + (blk & 1) * 8) = make_uint2(out[0], out[1]);
                tn[16 * kChunk + (blk >> 2) * kNfSfChunk + (r & 31) * 16 + (r >> 5) * 4 + (blk & 3)] = (uint8_t)sc;
            }
        }
        fence_proxy_async();                                 // these generic-proxy stores are read by the tensor core
        named_bar_sync(2, 128);
        if (qt == 0) mbar_arrive(&sq.tokbar);
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
        const int gpr = R >> 3, my_cg = et % gpr, my_m0 = et / gpr, m_step = 128 / gpr;
        const int my_row = prow + rank * R + my_cg * 8;
        const float w_ts = __ldg(a.ws[0]);
        bool have = mbar_wait(&s.tfull[0], 0, abort_flag, a.wait_ns);
        if (!have) tcs_abort(s, a);
        have = __all_sync(0xffffffffu, have);
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
        {
            uint32_t r[16];
            if (have) {
                tmem_ld16(taddr, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < kTcsnMaxM; ++j)
                if (j < Mt) tcs_st_remote(remote + (uint32_t)(j * R * 4), r[j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane % min(R, 32) == 0) tcs_arrive_remote(remote_rx);
        tcs_cluster_arrive();
        const bool got = tcs_wait_cluster(&s.rx, 0, abort_flag, a.wait_ns);
        if (!got) tcs_abort(s, a);
        if (got && !*abort_flag && my_row < a.N) {
            // the block's abs-max was written by the quantizer warps before the token area was declared complete
            const float scale = __fdiv_rn(sq.amax, 2688.f) * w_ts;
            const bool vec = (a.ldo & 7) == 0 && (reinterpret_cast<uintptr_t>(a.out[0]) & 15) == 0 && my_row + 8 <= a.N;
            for (int m = my_m0; m < Mt; m += m_step) {
                float sum[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) sum[j] = 0.f;
#pragma unroll
                for (int src = 0; src < 8; ++src)          // the contributions are added in rank order
                    if (src < C) {
                        const uint4* p = reinterpret_cast<const uint4*>(rxbuf + ((size_t)src * Mt + m) * R + my_cg * 8);
                        const uint4 lo = p[0], hi = p[1];
                        const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                        for (int j = 0; j < 8; ++j) sum[j] += __uint_as_float(w[j]);
                    }
                uint32_t h[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half2 hh = __floats2half2_rn(sum[2 * j] * scale, sum[2 * j + 1] * scale);
                    h[j] = *reinterpret_cast<const uint32_t*>(&hh);
                }
                __half* o = a.out[0] + (int64_t)m * a.ldo + my_row;
                if (vec) {
                    *reinterpret_cast<uint4*>(o) = make_uint4(h[0], h[1], h[2], h[3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (my_row + j < a.N) o[j] = __ushort_as_half((unsigned short)((h[j >> 1] >> ((j & 1) * 16)) & 0xffff));
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, tmem_cols);
    }
    tcs_cluster_wait();              // nobody leaves while a peer may still store into its shared memory
}

// ------------------------------------------------------------------------------------------------ host side
static bool tcsn_eligible(int64_t M, int64_t N, int64_t K) {
    const char* env = std::getenv("RWKVQ_TCSN");                 // read per call: a test switches routes in one process
    if ((env && std::atoi(env) == 0) || M < 1 || M > kTcsnMaxM || K % 256 || K < 2048) return false;
    const int C = tcs_cluster_size(M, N, K / 2);
    const int64_t per_cta = (K / 256 + C - 1) / C;
    // a quantizer thread keeps at most kTcsnBlocksPerThread blocks; the token area (4 KB per step) must leave two ring stages
    return C >= 2 && per_cta <= 16 && M * per_cta * 16 <= 128 * kTcsnBlocksPerThread;
}

static int32_t run_tcsn(TcArgs a, const void* w, int64_t ldw, int x_dtype, cudaStream_t st, const char* who) {
    const int C = tcs_cluster_size(a.M, a.N, a.K / 2);
    a.NB = 16;
    a.kchunks = a.K / 256;
    a.ptiles = (a.N + kTileP - 1) / kTileP;
    a.qtiles = C;
    a.acc_stride = 32;
    a.wait_ns = wait_limit_ns();
    a.status = device_status_ptr();
    const int per_cta = (a.kchunks + C - 1) / C;
    a.max_slots = per_cta;                                       // steps of the token area
    const size_t rx_bytes = (size_t)a.M * kTileP * 4;
    const size_t tok_bytes = (size_t)per_cta * kTcsnTokStage;
    a.stages = (int)std::min<size_t>(std::min<int>(kTcsMaxStages, per_cta), (kTcSmemBudgetHalf - 1024 - rx_bytes - tok_bytes) / kTcsnWStage);
    RWKVQ_REQUIRE(a.stages >= 2 || per_cta == 1, RWKVQ_E_SHAPE, "%s: shared memory leaves fewer than two ring stages", who);
    a.stages = std::max(a.stages, 1);
    TcMaps maps;
    const int32_t rcm = make_map(&maps.w[0], w, a.N, a.K / 2, ldw, kTileP, who);
    if (rcm) return rcm;
    auto kern = x_dtype == RWKVQ_F16 ? gemm_tcsn_kernel<RWKVQ_F16> : gemm_tcsn_kernel<RWKVQ_BF16>;
    const int32_t rc = ensure_smem_optin(reinterpret_cast<const void*>(kern), (int)kTcSmemBudget, who);
    if (rc) return rc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(a.ptiles * C));
    cfg.blockDim = dim3(kTcsnThreads);
    cfg.dynamicSmemBytes = (size_t)a.stages * kTcsnWStage + tok_bytes + rx_bytes + 1024;
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
