// Activation preparation kernels: bf16 copy + per-call amax (FP8 path), per-call e4m3 codes
// (large-M FP8 path) and per-row int8 codes (INT8 path).  All HBM/L2-bound elementwise work:
// 128-bit loads and stores, one row segment per CTA, block reduction + one atomic per CTA.
#include <cooperative_groups.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"

namespace rwkvq {

thread_local char g_err[512] = "";
std::atomic<int64_t> g_launches{0};

int32_t fail(int32_t code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int32_t check_launch(const char* what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    return RWKVQ_OK;
}

int sm_count() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != cached_dev) {
        cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
        cached_dev = dev;
    }
    return cached > 0 ? cached : 148;
}

extern "C" void rwkvq_set_wait_limit_us(int64_t);
static std::atomic<long long>& wait_limit_override();

unsigned long long wait_limit_ns() {
    static const long long from_env = [] {
        const char* e = std::getenv("RWKVQ_WAIT_LIMIT_US");
        const long long v = e ? std::atoll(e) : 0;
        return v > 0 ? v : 1500000ll;
    }();
    const long long o = wait_limit_override().load(std::memory_order_relaxed);
    return (unsigned long long)(o > 0 ? o : from_env) * 1000ull;
}

// per kernel and device: opt in to `bytes` of dynamic shared memory once
int32_t ensure_smem_optin(const void* kern, int bytes, const char* who) {
    static std::mutex mu;
    static std::vector<std::pair<const void*, int>> done;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    for (const auto& d : done)
        if (d.first == kern && d.second == dev) return RWKVQ_OK;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    RWKVQ_REQUIRE(e == cudaSuccess, RWKVQ_E_LAUNCH, "%s: cudaFuncSetAttribute: %s", who, cudaGetErrorString(e));
    done.emplace_back(kern, dev);
    return RWKVQ_OK;
}

int32_t kernel_plan(const void* kern, int threads, size_t smem, int optin_bytes, int* per_sm, const char* who) {
    struct Entry { const void* kern; int dev; size_t smem; int per_sm; };
    static std::mutex mu;
    static std::vector<Entry> done;
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lock(mu);
        for (const auto& d : done)
            if (d.kern == kern && d.dev == dev && d.smem == smem) { *per_sm = d.per_sm; return RWKVQ_OK; }
    }
    const int32_t rc = ensure_smem_optin(kern, optin_bytes, who);
    if (rc != RWKVQ_OK) return rc;
    int n = 0;
    const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, smem);
    RWKVQ_REQUIRE(e == cudaSuccess && n >= 1, RWKVQ_E_LAUNCH, "%s: occupancy query failed (%s)", who, cudaGetErrorString(e));
    std::lock_guard<std::mutex> lock(mu);
    done.push_back({kern, dev, smem, n});
    *per_sm = n;
    return RWKVQ_OK;
}

bool use_pdl() {
    static const bool on = [] {
        const char* e = std::getenv("RWKVQ_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

static __device__ int g_device_status;

int* device_status_ptr() {
    static std::mutex mu;
    static int* ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
        ptrs[dev] = reinterpret_cast<int*>(p);
    }
    return ptrs[dev];
}

constexpr int kThreads = 256;
constexpr int kSegElems = kThreads * 8 * 4;   // elements of one row handled by one CTA (vector path)

__device__ __forceinline__ float block_max(float v, float* sh) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = sh[0];
#pragma unroll
    for (int i = 1; i < kThreads / 32; ++i) r = fmaxf(r, sh[i]);
    __syncthreads();
    return r;
}

template <int DT>
__device__ __forceinline__ float load1(const void* x, int64_t i) {
    const uint16_t v = reinterpret_cast<const uint16_t*>(x)[i];
    if (DT == RWKVQ_F16) return __half2float(__ushort_as_half(v));
    return __uint_as_float((uint32_t)v << 16);
}

// ----------------------------------------------------------------------------------------
// prep_x for up to three tensors: bf16 copy (optional), amax per tensor.
struct Prep3Args {
    const void* x[3];
    const float* awq[3];
    void* out[3];
    float* amax;      // [ntensors]
};

template <int DT, bool VEC>
__global__ void __launch_bounds__(kThreads) prep_x_kernel(Prep3Args a, int64_t K, int64_t ldx, int64_t ldo, int div_mode, int after_bf16) {
    __shared__ float sh[kThreads / 32];
    const int t = blockIdx.z;
    const int64_t row = blockIdx.x;
    const int64_t k0 = (int64_t)blockIdx.y * kSegElems;
    const char* xrow = reinterpret_cast<const char*>(a.x[t]) + row * ldx * 2;
    uint16_t* orow = a.out[t] ? reinterpret_cast<uint16_t*>(a.out[t]) + row * ldo : nullptr;
    const float* awq = a.awq[t];
    float m = 0.f;
    if (VEC) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t k = k0 + ((int64_t)j * kThreads + threadIdx.x) * 8;
            if (k < K) {
                const uint4 v = *reinterpret_cast<const uint4*>(xrow + k * 2);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                uint32_t o[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float2 f = cvt2<DT>(w[q]);
                    if (awq) {
                        f.x = div_mode_f32(f.x, awq[k + 2 * q], div_mode);
                        f.y = div_mode_f32(f.y, awq[k + 2 * q + 1], div_mode);
                    }
                    o[q] = pack_bf16x2(f.x, f.y);
                    if (after_bf16) f = cvt2<RWKVQ_BF16>(o[q]);
                    m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
                }
                if (orow) *reinterpret_cast<uint4*>(orow + k) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    } else {
        const int64_t kend = (k0 + kSegElems < K) ? k0 + kSegElems : K;
        for (int64_t k = k0 + threadIdx.x; k < kend; k += kThreads) {
            float f = load1<DT>(xrow, k);
            if (awq) f = div_mode_f32(f, awq[k], div_mode);
            m = fmaxf(m, fabsf(after_bf16 ? bf16_round(f) : f));
            if (orow) {
                __nv_bfloat16 b = __float2bfloat16_rn(f);
                orow[k] = *reinterpret_cast<uint16_t*>(&b);
            }
        }
    }
    m = block_max(m, sh);
    if (threadIdx.x == 0) atomic_max_nonneg(a.amax + t, m);
}

static int32_t launch_prep(const Prep3Args& a, int nt, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, int64_t ldo,
                           int32_t div_mode, cudaStream_t st, int after_bf16 = 0) {
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "prep_x: x_dtype %d", x_dtype);
    RWKVQ_REQUIRE(div_mode == RWKVQ_DIV_IEEE || div_mode == RWKVQ_DIV_FULL || div_mode == RWKVQ_DIV_TORCH, RWKVQ_E_BADARG, "prep_x: div_mode %d", div_mode);
    RWKVQ_REQUIRE(M >= 0 && K >= 0 && ldx >= K, RWKVQ_E_SHAPE, "prep_x: M=%lld K=%lld ldx=%lld", (long long)M, (long long)K, (long long)ldx);
    RWKVQ_REQUIRE(a.amax != nullptr, RWKVQ_E_BADARG, "prep_x: amax is null");
    if (cudaMemsetAsync(a.amax, 0, sizeof(float) * nt, st) != cudaSuccess) return check_launch("prep_x memset");
    if (M == 0 || K == 0) return RWKVQ_OK;
    bool vec = (K % 8 == 0) && (ldx % 8 == 0);
    for (int t = 0; t < nt; ++t) {
        RWKVQ_REQUIRE(a.x[t] != nullptr, RWKVQ_E_BADARG, "prep_x: x[%d] is null", t);
        vec = vec && aligned16(a.x[t]) && (a.out[t] == nullptr || (aligned16(a.out[t]) && ldo % 8 == 0));
        RWKVQ_REQUIRE(a.out[t] == nullptr || ldo >= K, RWKVQ_E_SHAPE, "prep_x: ldo=%lld < K", (long long)ldo);
    }
    const int64_t segs = (K + kSegElems - 1) / kSegElems;
    RWKVQ_REQUIRE(segs <= 65535, RWKVQ_E_SHAPE, "prep_x: K=%lld too large", (long long)K);
    dim3 grid((unsigned)M, (unsigned)segs, nt);
#define RWKVQ_PREP(DT, V) prep_x_kernel<DT, V><<<grid, kThreads, 0, st>>>(a, K, ldx, ldo, div_mode, after_bf16)
    if (x_dtype == RWKVQ_F16) { if (vec) RWKVQ_PREP(RWKVQ_F16, true); else RWKVQ_PREP(RWKVQ_F16, false); }
    else                      { if (vec) RWKVQ_PREP(RWKVQ_BF16, true); else RWKVQ_PREP(RWKVQ_BF16, false); }
#undef RWKVQ_PREP
    return check_launch("prep_x");
}

// ----------------------------------------------------------------------------------------
// prep_x_fp8, second pass: e4m3 codes from the per-call amax (IEEE divisions, as torch computes them).
template <int DT, bool VEC>
__global__ void __launch_bounds__(kThreads) quant_fp8_kernel(const void* x, uint8_t* codes, float* scale, const float* amax_p,
                                                             int64_t K, int64_t ldx, int64_t ldc, int div_mode, int from_bf16) {
    const int64_t row = blockIdx.x;
    const int64_t k0 = (int64_t)blockIdx.y * kSegElems;
    const float amax = *amax_p;
    const float inv = scale_inv(448.f, fmaxf(amax, 1e-12f), div_mode);
    if (scale && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *scale = scale_fwd(amax, 448.f, div_mode);
    const char* xrow = reinterpret_cast<const char*>(x) + row * ldx * 2;
    uint8_t* crow = codes + row * ldc;
    if (VEC) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t k = k0 + ((int64_t)j * kThreads + threadIdx.x) * 8;
            if (k < K) {
                const uint4 v = *reinterpret_cast<const uint4*>(xrow + k * 2);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                uint32_t c[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float2 f = cvt2<DT>(w[q]);
                    if (from_bf16) { f.x = bf16_round(f.x); f.y = bf16_round(f.y); }
                    c[q] = e4m3x2(clamp448(f.x * inv), clamp448(f.y * inv));
                }
                *reinterpret_cast<uint2*>(crow + k) = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
            }
        }
    } else {
        const int64_t kend = (k0 + kSegElems < K) ? k0 + kSegElems : K;
        for (int64_t k = k0 + threadIdx.x; k < kend; k += kThreads) {
            float f = load1<DT>(xrow, k);
            if (from_bf16) f = bf16_round(f);
            crow[k] = (uint8_t)(e4m3x2(clamp448(f * inv), 0.f) & 0xff);
        }
    }
}

// ----------------------------------------------------------------------------------------
// prep_x_int8 (and the three of prep3_x_int8 in one launch: blockIdx.y picks the tensor): one CTA per row; the row is
// read twice (second read hits L1/L2).
struct QInt8Args {
    const void* x[3];
    int8_t* codes[3];
    float* scales[3];
};

// KEEP: decode-sized grids (latency counts, occupancy does not): a separate instantiation, so that the many-row form
// keeps its small register footprint.
template <int DT, bool VEC, bool KEEP = false>
__global__ void __launch_bounds__(kThreads) quant_int8_kernel(const QInt8Args qa, int64_t K, int64_t ldx, int64_t ldc, int div_mode) {
    __shared__ float sh[kThreads / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a projection behind this launch may prefetch its weights
    asm volatile("griddepcontrol.wait;" ::: "memory");                // launched early itself: wait for the producer of x
    const int64_t row = blockIdx.x;
    const char* xrow = reinterpret_cast<const char*>(qa.x[blockIdx.y]) + row * ldx * 2;
    int8_t* crow = qa.codes[blockIdx.y] + row * ldc;
    float* scales = qa.scales[blockIdx.y];
    float m = 0.f;
    if (VEC && KEEP && K <= (int64_t)kThreads * 8 * 8) {
        // rows of up to 16384 elements: a thread's (at most 8) vectors stay in registers between the abs-max and the
        // codes -- one read of the row, all loads in flight at once
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t k = ((int64_t)threadIdx.x + j * kThreads) * 8;
            v[j] = make_uint4(0, 0, 0, 0);
            if (k < K) v[j] = *reinterpret_cast<const uint4*>(xrow + k * 2);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = cvt2<DT>(w[q]);
                m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
        }
        m = fmaxf(block_max(m, sh), 1e-12f);
        const float s = div_mode_f32(127.f, m, div_mode);
        if (threadIdx.x == 0) scales[row] = div_mode_f32(m, 127.f, div_mode);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t k = ((int64_t)threadIdx.x + j * kThreads) * 8;
            if (k >= K) continue;
            const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
            uint32_t c[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = cvt2<DT>(w[q]);
                const uint32_t lo = (uint32_t)(__float2int_rz(fminf(fmaxf(f.x * s, -128.f), 127.f))) & 0xffu;
                const uint32_t hi = (uint32_t)(__float2int_rz(fminf(fmaxf(f.y * s, -128.f), 127.f))) & 0xffu;
                c[q] = lo | (hi << 8);
            }
            *reinterpret_cast<uint2*>(crow + k) = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
        }
        return;
    }
    if (VEC) {
        for (int64_t k = (int64_t)threadIdx.x * 8; k < K; k += kThreads * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(xrow + k * 2);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = cvt2<DT>(w[q]);
                m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
        }
    } else {
        for (int64_t k = threadIdx.x; k < K; k += kThreads) m = fmaxf(m, fabsf(load1<DT>(xrow, k)));
    }
    m = fmaxf(block_max(m, sh), 1e-12f);
    const float s = div_mode_f32(127.f, m, div_mode);
    if (threadIdx.x == 0) scales[row] = div_mode_f32(m, 127.f, div_mode);
    auto q8 = [s](float f) -> uint32_t {
        return (uint32_t)(__float2int_rz(fminf(fmaxf(f * s, -128.f), 127.f))) & 0xffu;
    };
    if (VEC) {
        for (int64_t k = (int64_t)threadIdx.x * 8; k < K; k += kThreads * 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(xrow + k * 2);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t c[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = cvt2<DT>(w[q]);
                c[q] = q8(f.x) | (q8(f.y) << 8);
            }
            *reinterpret_cast<uint2*>(crow + k) = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
        }
    } else {
        for (int64_t k = threadIdx.x; k < K; k += kThreads) crow[k] = (int8_t)q8(load1<DT>(xrow, k));
    }
}

// ----------------------------------------------------------------------------------------
// FP8 activation quantization in ONE launch, for one tensor or for xr, xk, xv together: per-CTA partial maxima, a
// grid-wide rendezvous, then the code pass (rows kept in registers, or a second read that hits L2).  The grid is
// launched cooperatively (all CTAs resident); the rendezvous wait is bounded all the same.
//
// Rendezvous.  The scratch holds one slot and one flag per CTA and an EPOCH word.  Every CTA reads the epoch E when it
// starts, publishes its maximum and then the value E+1 in its flag; a CTA passes once all flags of its tensor read
// E+1; CTA 0 stores E+1 as the new epoch on its way out.  All epoch reads happen before any CTA can pass, and the bump
// after, so the next launch on the scratch -- a later call, or the next replay of a captured graph -- starts from
// E+1 and cannot be satisfied by the flags this launch left behind.  Nothing is drawn on the host.
constexpr int kFusedThreads = 512;
constexpr int kFusedMaxCtas = 512;
constexpr int kFusedEpochWord = 2 * kFusedMaxCtas;          // slots[512] | flags[512] | epoch

struct ActqArgs {
    const void* x[3];
    uint8_t* codes[3];
    float* amax_out;          // [nt]
    float* scale_out[3];      // optional, one float each
    float* slots;
    uint32_t* flags;          // flags[kFusedMaxCtas] is the epoch word
    int* status;
    unsigned long long wait_ns;
    int64_t ldx, ldc;
    int M, K, nt, cpt;        // tensors, CTAs per tensor (grid = nt * cpt)
    int div_mode, after_bf16, from_bf16;
};

// KEEP: a CTA has at most 8 rows of at most kFusedThreads vectors: every thread holds its vectors in registers across
// the rendezvous, so the activations are read once and all of a thread's loads are in flight together.
template <int DT, bool KEEP>
__global__ void __launch_bounds__(kFusedThreads, 2) actq_fp8_fused_kernel(const ActqArgs a) {
    __shared__ float sh[kFusedThreads / 32];
    __shared__ float s_amax;
    __shared__ int s_fail;
    __shared__ uint32_t s_token;
    // a projection launched behind this kernel with programmatic dependent launch may start now and prefetch its
    // weights; it waits (griddepcontrol.wait) for this grid to finish before it reads the codes
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int kv = a.K >> 3, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = (int)blockIdx.x / a.cpt, cb = (int)blockIdx.x - t * a.cpt, G = a.cpt;
    const char* x = reinterpret_cast<const char*>(a.x[t]);
    uint8_t* codes = a.codes[t];
    const int M = a.M;
    const int64_t ldx = a.ldx, ldc = a.ldc;
    const bool after_bf16 = a.after_bf16 != 0, from_bf16 = a.from_bf16 != 0;
    if (threadIdx.x == 0) {
        s_token = ld_acquire_u32(a.flags + kFusedMaxCtas) + 1u;
        s_fail = 0;
    }
    // ---- pass 1: partial maximum of this CTA's rows; four rows per step, so four loads per thread are in flight
    float m = 0.f;
    auto vec_max = [&](const uint4& v) {
        if (DT == RWKVQ_F16 && after_bf16) {
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = cvt2<DT>(w[q]);
                m = fmaxf(m, fmaxf(fabsf(bf16_round(f.x)), fabsf(bf16_round(f.y))));
            }
        } else if (DT == RWKVQ_F16) {
            const __half2* h = reinterpret_cast<const __half2*>(&v);
            const __half2 t2 = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
            m = fmaxf(m, fmaxf(__low2float(t2), __high2float(t2)));
        } else {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
            const __nv_bfloat162 t2 = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
            m = fmaxf(m, fmaxf(__low2float(t2), __high2float(t2)));
        }
    };
    uint4 keep[KEEP ? 8 : 1];
    if constexpr (KEEP) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int rj = cb + j * G;
            keep[j] = make_uint4(0, 0, 0, 0);
            if (rj < M && (int)threadIdx.x < kv)
                keep[j] = *reinterpret_cast<const uint4*>(x + ((int64_t)rj * ldx + (int64_t)threadIdx.x * 8) * 2);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) vec_max(keep[j]);
    } else {
        for (int r = cb; r < M; r += 4 * G) {
            for (int i = threadIdx.x; i < kv; i += kFusedThreads) {
                uint4 v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int rj = min(r + j * G, M - 1);              // a clamped row repeats a value: harmless for a maximum
                    v[j] = *reinterpret_cast<const uint4*>(x + ((int64_t)rj * ldx + (int64_t)i * 8) * 2);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) vec_max(v[j]);
            }
        }
    }
    m = warp_max(m);
    if (lane == 0) sh[warp] = m;
    __syncthreads();
    const uint32_t token = s_token;
    if (threadIdx.x == 0) {
        float b = sh[0];
        for (int i = 1; i < kFusedThreads / 32; ++i) b = fmaxf(b, sh[i]);
        a.slots[blockIdx.x] = b;
        __threadfence();
        st_release_u32(a.flags + blockIdx.x, token);    // the epoch was read before this store (release orders it)
    }
    // ---- rendezvous: thread i waits for the flag of CTA i of this tensor, then the maxima are combined.  CTA 0 waits
    // for the flags of ALL tensors' CTAs: once they all read E+1, every CTA of the launch has read the epoch.
    const int nwait = blockIdx.x == 0 ? a.nt * G : G, base = blockIdx.x == 0 ? 0 : t * G;
    float g = 0.f;
    if ((int)threadIdx.x < nwait) {
        if (!wait_flag_eq(a.flags + base + threadIdx.x, token, a.wait_ns)) s_fail = 1;
        else if ((int)threadIdx.x < G) g = __ldcg(a.slots + base + threadIdx.x);
    }
    g = warp_max(g);
    __syncthreads();
    if (lane == 0) sh[warp] = g;
    __syncthreads();
    if (threadIdx.x == 0) {
        float b = sh[0];
        for (int i = 1; i < kFusedThreads / 32; ++i) b = fmaxf(b, sh[i]);
        s_amax = b;
        if (cb == 0) {
            a.amax_out[t] = b;
            if (a.scale_out[t]) *a.scale_out[t] = scale_fwd(b, 448.f, a.div_mode);
        }
        if (s_fail && a.status) atomicExch(a.status, RWKVQ_E_TIMEOUT);
        // all flags read E+1, so nobody will read the old epoch any more: move it on for the next launch.  After a
        // timeout the epoch stays and the caller has to clear the scratch.
        if (blockIdx.x == 0 && !s_fail) st_release_u32(a.flags + kFusedMaxCtas, token);
    }
    __syncthreads();
    if (s_fail) return;
    // ---- pass 2: codes
    const float inv = scale_inv(448.f, fmaxf(s_amax, 1e-12f), a.div_mode);
    auto vec_codes = [&](const uint4& v, int rj, int i) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t c[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float2 f = cvt2<DT>(w[q]);
            if (DT == RWKVQ_F16 && from_bf16) { f.x = bf16_round(f.x); f.y = bf16_round(f.y); }
            c[q] = e4m3x2(f.x * inv, f.y * inv);
        }
        *reinterpret_cast<uint2*>(codes + (int64_t)rj * ldc + (size_t)i * 8) = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
    };
    if constexpr (KEEP) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int rj = cb + j * G;
            if (rj < M && (int)threadIdx.x < kv) vec_codes(keep[j], rj, threadIdx.x);
        }
    } else {
        for (int r = cb; r < M; r += 4 * G) {
            for (int i = threadIdx.x; i < kv; i += kFusedThreads) {
                uint4 v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int rj = min(r + j * G, M - 1);
                    v[j] = *reinterpret_cast<const uint4*>(x + ((int64_t)rj * ldx + (int64_t)i * 8) * 2);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (r + j * G < M) vec_codes(v[j], r + j * G, i);
            }
        }
    }
}

// Few rows (decode): a CLUSTER of 1 to 8 CTAs of 1024 threads per tensor does the whole job -- abs-max over the block,
// then the codes -- with up to 8 vectors per thread kept in registers between the two (one read of the activations,
// all loads in flight together).  The CTAs of a cluster exchange their maxima through distributed shared memory and
// one cluster barrier; there is no grid rendezvous and no scratch, so the kernel can be launched with programmatic
// dependent launch: it becomes resident while its predecessor drains, releases its own dependents at once (the
// projection behind it starts prefetching weights) and waits for its input.
// The CTA size is the launch's (blockDim.x): 256 threads for blocks of up to 16384 vectors -- such a CTA takes a quarter
// of an SM's registers and becomes resident beside the CTAs of the projection in front, whereas a 1024-thread CTA takes
// the whole register file and has to wait for a drained SM -- and 1024 threads for larger blocks.
constexpr int kSmallThreads = 1024;
constexpr int kSmallThreadsLight = 256;
constexpr int kSmallKeep = 8;

template <int DT>
__global__ void __launch_bounds__(kSmallThreads, 1) actq_fp8_small_kernel(const ActqArgs a) {
    __shared__ float sh[kSmallThreads / 32];
    __shared__ float s_part[8];           // maxima of the cluster's CTAs (each CTA writes its slot in every CTA)
    __shared__ float s_amax;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    cooperative_groups::cluster_group cl = cooperative_groups::this_cluster();
    const int C = (int)cl.num_blocks(), cr = (int)cl.block_rank();
    const int t = (int)blockIdx.x / C, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const char* x = reinterpret_cast<const char*>(a.x[t]);
    uint8_t* codes = a.codes[t];
    const int kv = a.K >> 3, nvec = a.M * kv;
    const uint32_t inv_kv = 0xFFFFFFFFu / (uint32_t)kv + 1u;          // row of a flat vector index without a division
    const bool after_bf16 = a.after_bf16 != 0, from_bf16 = a.from_bf16 != 0;
    const int nthr = (int)blockDim.x;
    const bool keep = nvec <= kSmallKeep * nthr * C;
    asm volatile("griddepcontrol.wait;" ::: "memory");                // the activations may come from the previous kernel
    auto vec_ptr = [&](int idx) {
        const int r = (int)__umulhi((uint32_t)idx, inv_kv), c = idx - r * kv;
        return x + ((int64_t)r * a.ldx + (int64_t)c * 8) * 2;
    };
    auto vec_max = [&](const uint4& v, float m) {
        if (DT == RWKVQ_F16 && after_bf16) {
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = cvt2<DT>(w[q]);
                m = fmaxf(m, fmaxf(fabsf(bf16_round(f.x)), fabsf(bf16_round(f.y))));
            }
            return m;
        } else if (DT == RWKVQ_F16) {
            const __half2* h = reinterpret_cast<const __half2*>(&v);
            const __half2 t2 = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
            return fmaxf(m, fmaxf(__low2float(t2), __high2float(t2)));
        } else {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
            const __nv_bfloat162 t2 = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
            return fmaxf(m, fmaxf(__low2float(t2), __high2float(t2)));
        }
    };
    // the cluster's threads take the vectors round-robin: thread (cr, tid) vectors first, first + step, ...
    const int first = cr * nthr + (int)threadIdx.x, step = C * nthr;
    uint4 v[kSmallKeep];
    float m = 0.f;
#pragma unroll 1
    for (int i0 = first; i0 < nvec; i0 += kSmallKeep * step) {
#pragma unroll
        for (int j = 0; j < kSmallKeep; ++j)
            if (i0 + j * step < nvec) v[j] = *reinterpret_cast<const uint4*>(vec_ptr(i0 + j * step));
#pragma unroll
        for (int j = 0; j < kSmallKeep; ++j)
            if (i0 + j * step < nvec) m = vec_max(v[j], m);
    }
    m = warp_max(m);
    if (lane == 0) sh[warp] = m;
    __syncthreads();
    if (warp == 0) {
        const float b = warp_max(lane < (nthr >> 5) ? sh[lane] : 0.f);
        if (lane < C) *cl.map_shared_rank(&s_part[cr], lane) = b;      // this CTA's maximum into slot cr of CTA `lane`
    }
    cl.sync();                                                          // all slots written (and visible) in every CTA
    if (threadIdx.x == 0) {
        float b = s_part[0];
        for (int i = 1; i < C; ++i) b = fmaxf(b, s_part[i]);
        s_amax = b;
        if (cr == 0) {
            a.amax_out[t] = b;
            if (a.scale_out[t]) *a.scale_out[t] = scale_fwd(b, 448.f, a.div_mode);
        }
    }
    __syncthreads();
    const float inv = scale_inv(448.f, fmaxf(s_amax, 1e-12f), a.div_mode);
    auto vec_codes = [&](const uint4& vv, int idx) {
        const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
        uint32_t c[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float2 f = cvt2<DT>(w[q]);
            if (DT == RWKVQ_F16 && from_bf16) { f.x = bf16_round(f.x); f.y = bf16_round(f.y); }
            c[q] = e4m3x2(f.x * inv, f.y * inv);
        }
        const int r = (int)__umulhi((uint32_t)idx, inv_kv), cc = idx - r * kv;
        *reinterpret_cast<uint2*>(codes + (int64_t)r * a.ldc + (size_t)cc * 8) = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
    };
    if (keep) {
#pragma unroll
        for (int j = 0; j < kSmallKeep; ++j)
            if (first + j * step < nvec) vec_codes(v[j], first + j * step);
    } else {
#pragma unroll 1
        for (int i0 = first; i0 < nvec; i0 += kSmallKeep * step) {
#pragma unroll
            for (int j = 0; j < kSmallKeep; ++j)
                if (i0 + j * step < nvec) v[j] = *reinterpret_cast<const uint4*>(vec_ptr(i0 + j * step));
#pragma unroll
            for (int j = 0; j < kSmallKeep; ++j)
                if (i0 + j * step < nvec) vec_codes(v[j], i0 + j * step);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Two plain launches for blocks between the cluster kernel above and the many-token cooperative kernel: an abs-max
// pass and a codes pass, chained by programmatic dependent launch.  A cooperative launch costs several microseconds
// more than a plain one and cannot start early behind its predecessor; here the second kernel is resident while the
// first runs and re-reads the activations from L2.  `two` = 4 words of the caller's zeroed scratch: the maxima of up
// to three tensors (float bits, non-negative, so an integer atomicMax orders them) and a count of codes-pass CTAs; the
// last one to finish clears all four, so the words are zero again before the next launch on the stream can reach
// them (it waits for this grid first) and a captured graph replays.
constexpr int kTwoThreads = 256;
constexpr int kTwoWord = kFusedEpochWord + 4;
// up to 4096 rows of 16384 elements; larger blocks: one cooperative launch.  (Measured at 2048 rows: the prefill step over
// all projections runs 1.6 % faster with the two launches than with the cooperative one, 13.98 against 14.21 ms.)
constexpr int64_t kTwoMaxVectors = 1 << 23;

template <int DT>
__device__ __forceinline__ float two_vec_max(const uint4& v, float m, bool after_bf16) {
    if (DT == RWKVQ_F16 && after_bf16) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 f = cvt2<DT>(w[q]);
            m = fmaxf(m, fmaxf(fabsf(bf16_round(f.x)), fabsf(bf16_round(f.y))));
        }
        return m;
    } else if (DT == RWKVQ_F16) {
        const __half2* h = reinterpret_cast<const __half2*>(&v);
        const __half2 t2 = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
        return fmaxf(m, fmaxf(__low2float(t2), __high2float(t2)));
    } else {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
        const __nv_bfloat162 t2 = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
        return fmaxf(m, fmaxf(__low2float(t2), __high2float(t2)));
    }
}

// grid (rows * cpr, nt): CTA (b, t) takes every cpr-th group of kTwoThreads vectors of row b / cpr (and of every
// (gridDim.x / cpr)-th row after it) of tensor t.
template <int DT>
__global__ void __launch_bounds__(kTwoThreads) actq_two_amax_kernel(const ActqArgs a, int cpr) {
    __shared__ float sh[kTwoThreads / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int t = blockIdx.y, kv = a.K >> 3, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = (int)blockIdx.x % cpr, rstep = (int)gridDim.x / cpr, cstep = cpr * kTwoThreads;
    const char* x = reinterpret_cast<const char*>(a.x[t]);
    const bool after_bf16 = a.after_bf16 != 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float m = 0.f;
    for (int r = (int)blockIdx.x / cpr; r < a.M; r += rstep) {
        const char* row = x + (int64_t)r * a.ldx * 2;
        for (int c0 = seg * kTwoThreads + (int)threadIdx.x; c0 < kv; c0 += 4 * cstep) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c0 + j * cstep < kv) v[j] = *reinterpret_cast<const uint4*>(row + (int64_t)(c0 + j * cstep) * 16);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c0 + j * cstep < kv) m = two_vec_max<DT>(v[j], m, after_bf16);
        }
    }
    m = warp_max(m);
    if (lane == 0) sh[warp] = m;
    __syncthreads();
    if (warp == 0) {
        m = warp_max(lane < kTwoThreads / 32 ? sh[lane] : 0.f);
        if (lane == 0 && m > 0.f) atomicMax(reinterpret_cast<int*>(a.flags) + kTwoWord - kFusedMaxCtas + t, __float_as_int(m));
    }
}

template <int DT>
__global__ void __launch_bounds__(kTwoThreads) actq_two_codes_kernel(const ActqArgs a, int cpr) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int t = blockIdx.y, kv = a.K >> 3;
    const int seg = (int)blockIdx.x % cpr, rstep = (int)gridDim.x / cpr, cstep = cpr * kTwoThreads;
    const char* x = reinterpret_cast<const char*>(a.x[t]);
    uint8_t* codes = a.codes[t];
    const bool from_bf16 = a.from_bf16 != 0;
    int* two = reinterpret_cast<int*>(a.flags) + kTwoWord - kFusedMaxCtas;
    asm volatile("griddepcontrol.wait;" ::: "memory");              // the abs-max pass is complete and visible
    const float amax = __int_as_float(__ldcg(two + t));
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        a.amax_out[t] = amax;
        if (a.scale_out[t]) *a.scale_out[t] = scale_fwd(amax, 448.f, a.div_mode);
    }
    const float inv = scale_inv(448.f, fmaxf(amax, 1e-12f), a.div_mode);
    for (int r = (int)blockIdx.x / cpr; r < a.M; r += rstep) {
        const char* row = x + (int64_t)r * a.ldx * 2;
        uint8_t* crow = codes + (int64_t)r * a.ldc;
        for (int c0 = seg * kTwoThreads + (int)threadIdx.x; c0 < kv; c0 += 4 * cstep) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c0 + j * cstep < kv) v[j] = *reinterpret_cast<const uint4*>(row + (int64_t)(c0 + j * cstep) * 16);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (c0 + j * cstep >= kv) continue;
                const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
                uint32_t q[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 f = cvt2<DT>(w[i]);
                    if (DT == RWKVQ_F16 && from_bf16) { f.x = bf16_round(f.x); f.y = bf16_round(f.y); }
                    q[i] = e4m3x2(f.x * inv, f.y * inv);
                }
                *reinterpret_cast<uint2*>(crow + (int64_t)(c0 + j * cstep) * 8) = make_uint2(q[0] | (q[1] << 16), q[2] | (q[3] << 16));
            }
        }
    }
    __syncthreads();                                    // every thread of this CTA has read the maximum
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(two + 3, 1) == (int)(gridDim.x * gridDim.y) - 1) {
            two[0] = 0; two[1] = 0; two[2] = 0;
            __threadfence();
            two[3] = 0;
        }
    }
}

// FP8 codes of h with an amax that the PRODUCER of h published (the FFN key projection with relu^2 in its epilogue):
// purely elementwise -- no abs-max pass, no grid rendezvous -- so it is launched with programmatic dependent launch.
// ffn[0] = the published amax (float), ffn[1] = count of CTAs that have read it; the last one clears both for the next
// producer.  amax_out / scale_out are this call's own copies for the GEMM that follows.
template <int DT>
__global__ void __launch_bounds__(kThreads) quant_fp8_given_kernel(const void* x, uint8_t* codes, float* amax_out, float* scale_out,
                                                                   float* ffn, int M, int64_t K, int64_t ldx, int64_t ldc, int div_mode,
                                                                   int from_bf16) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float amax = __ldcg(ffn);
    const float inv = scale_inv(448.f, fmaxf(amax, 1e-12f), div_mode);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        *amax_out = amax;
        if (scale_out) *scale_out = scale_fwd(amax, 448.f, div_mode);
    }
    const int64_t kv = K >> 3, nvec = (int64_t)M * kv;
    for (int64_t i0 = (int64_t)blockIdx.x * kThreads + threadIdx.x; i0 < nvec; i0 += (int64_t)gridDim.x * kThreads * 4) {
        uint4 v[4];
        int64_t r[4], c[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t idx = i0 + (int64_t)j * gridDim.x * kThreads;
            r[j] = idx / kv;
            c[j] = idx - r[j] * kv;
            if (idx < nvec) v[j] = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(x) + (r[j] * ldx + c[j] * 8) * 2);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (i0 + (int64_t)j * gridDim.x * kThreads >= nvec) continue;
            const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
            uint32_t q[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                float2 f = cvt2<DT>(w[p]);
                if (DT == RWKVQ_F16 && from_bf16) { f.x = bf16_round(f.x); f.y = bf16_round(f.y); }
                q[p] = e4m3x2(f.x * inv, f.y * inv);
            }
            *reinterpret_cast<uint2*>(codes + r[j] * ldc + c[j] * 8) = make_uint2(q[0] | (q[1] << 16), q[2] | (q[3] << 16));
        }
    }
    __syncthreads();                                    // every thread of this CTA has used the amax
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(reinterpret_cast<int*>(ffn) + 1, 1) == (int)gridDim.x - 1) {
            ffn[0] = 0.f;
            __threadfence();
            reinterpret_cast<int*>(ffn)[1] = 0;
        }
    }
}

// INT8 codes of h with row maxima that the PRODUCER of h published (the FFN key GEMM with relu^2 in its epilogue):
// no abs-max pass; one CTA per row, four vectors in flight per thread; the CTA clears its row's maximum when every
// thread has used it, so the array is zero again for the next producer (graph replay safe).
template <int DT>
__global__ void __launch_bounds__(kThreads) quant_int8_given_kernel(const void* x, int8_t* codes, float* scales, float* row_max, int64_t K,
                                                                    int64_t ldx, int64_t ldc, int div_mode) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t row = blockIdx.x;
    const char* xrow = reinterpret_cast<const char*>(x) + row * ldx * 2;
    int8_t* crow = codes + row * ldc;
    const float m = fmaxf(__ldcg(row_max + row), 1e-12f);
    const float s = div_mode_f32(127.f, m, div_mode);
    if (threadIdx.x == 0) scales[row] = div_mode_f32(m, 127.f, div_mode);
    for (int64_t k0 = (int64_t)threadIdx.x * 8; k0 < K; k0 += (int64_t)kThreads * 8 * 4) {
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t k = k0 + (int64_t)j * kThreads * 8;
            if (k < K) v[j] = *reinterpret_cast<const uint4*>(xrow + k * 2);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t k = k0 + (int64_t)j * kThreads * 8;
            if (k >= K) continue;
            const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
            uint32_t c[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = cvt2<DT>(w[q]);
                const uint32_t lo = (uint32_t)(__float2int_rz(fminf(fmaxf(f.x * s, -128.f), 127.f))) & 0xffu;
                const uint32_t hi = (uint32_t)(__float2int_rz(fminf(fmaxf(f.y * s, -128.f), 127.f))) & 0xffu;
                c[q] = lo | (hi << 8);
            }
            *reinterpret_cast<uint2*>(crow + k) = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
        }
    }
    __syncthreads();                                    // every thread of this CTA has used the maximum
    if (threadIdx.x == 0) row_max[row] = 0.f;
}

// A kernel whose only job is to let a bounded wait run out: one CTA waits for an mbarrier phase that nothing
// completes (mode 0) or for a flag value that nothing stores (mode 1), gives up after `limit_ns`, records
// RWKVQ_E_TIMEOUT in *status and returns normally -- the path every kernel of this library takes when a producer
// never shows up, exercised without any fault or hang.
__global__ void selftest_timeout_kernel(int* status, uint32_t* never_written, unsigned long long limit_ns, int mode) {
    __shared__ uint64_t bar;
    bool ok;
    if (mode == 0) {
        const uint32_t b = (uint32_t)__cvta_generic_to_shared(&bar);
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const unsigned long long t0 = global_ns();
        ok = false;
        for (;;) {
            uint32_t done = 0;
#pragma unroll 1
            for (int i = 0; i < 256 && !done; ++i) {
                asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                             : "=r"(done) : "r"(b) : "memory");
                __nanosleep(64);
            }
            if (done) { ok = true; break; }
            if (global_ns() - t0 > limit_ns) break;
        }
    } else {
        ok = wait_flag_eq(never_written, ld_acquire_u32(never_written) + 1u, limit_ns);
    }
    if (!ok) atomicExch(status, RWKVQ_E_TIMEOUT);
}

__global__ void div_kernel(const float* a, const float* b, float* o, int64_t n, int mode) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) o[i] = div_mode_f32(a[i], b[i], mode);
}

}  // namespace rwkvq

static std::atomic<long long>& rwkvq::wait_limit_override() {
    static std::atomic<long long> v{-1};
    return v;
}

using namespace rwkvq;

extern "C" {

int32_t rwkvq_version(void) { return 100; }
const char* rwkvq_last_error_string(void) { return g_err; }
int64_t rwkvq_launch_count(void) { return g_launches.load(); }

int32_t rwkvq_device_ok(void) {
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(RWKVQ_E_ARCH, "no CUDA device");
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (major != 10) return fail(RWKVQ_E_ARCH, "device compute capability major %d, need 10 (sm_100a)", major);
    return RWKVQ_OK;
}

int32_t rwkvq_div_f32(const float* a, const float* b, float* out, int64_t n, int32_t div_mode, void* stream) {
    RWKVQ_REQUIRE(a && b && out, RWKVQ_E_BADARG, "div_f32: null pointer");
    if (n <= 0) return RWKVQ_OK;
    div_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a, b, out, n, div_mode);
    return check_launch("div_f32");
}

int32_t rwkvq_prep_x(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, const float* awq, void* out_bf16,
                     int64_t ldo, float* amax, int32_t div_mode, void* stream) {
    Prep3Args a{};
    a.x[0] = x; a.awq[0] = awq; a.out[0] = out_bf16; a.amax = amax;
    return launch_prep(a, 1, x_dtype, M, K, ldx, ldo, div_mode, (cudaStream_t)stream);
}

int32_t rwkvq_prep3_x(const void* xr, const void* xk, const void* xv, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx,
                      const float* awq_r, const float* awq_k, void* out_r, void* out_k, void* out_v, int64_t ldo,
                      float* amax3, int32_t div_mode, void* stream) {
    Prep3Args a{};
    a.x[0] = xr; a.x[1] = xk; a.x[2] = xv;
    a.awq[0] = awq_r; a.awq[1] = awq_k; a.awq[2] = nullptr;
    a.out[0] = out_r; a.out[1] = out_k; a.out[2] = out_v;
    a.amax = amax3;
    return launch_prep(a, 3, x_dtype, M, K, ldx, ldo, div_mode, (cudaStream_t)stream);
}

int32_t rwkvq_actq_fp8(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes, int64_t ldc,
                       float* amax, float* scale, int32_t div_mode, uint32_t flags, void* stream) {
    RWKVQ_REQUIRE(codes && amax, RWKVQ_E_BADARG, "actq_fp8: null output");
    RWKVQ_REQUIRE(ldc >= K, RWKVQ_E_SHAPE, "actq_fp8: ldc=%lld < K", (long long)ldc);
    cudaStream_t st = (cudaStream_t)stream;
    const int after = (flags & RWKVQ_FLAG_AMAX_AFTER_BF16) ? 1 : 0, from_bf16 = (flags & RWKVQ_FLAG_QUANT_FROM_BF16) ? 1 : 0;
    Prep3Args a{};
    a.x[0] = x; a.amax = amax;
    int32_t rc = launch_prep(a, 1, x_dtype, M, K, ldx, K, div_mode, st, after);
    if (rc != RWKVQ_OK) return rc;
    if (M == 0 || K == 0) {   // scale = 0/448
        if (scale && cudaMemsetAsync(scale, 0, sizeof(float), st) != cudaSuccess) return check_launch("actq_fp8 memset");
        return RWKVQ_OK;
    }
    const bool vec = (K % 8 == 0) && (ldx % 8 == 0) && aligned16(x) && (ldc % 8 == 0) && ((uintptr_t)codes % 8 == 0);
    dim3 grid((unsigned)M, (unsigned)((K + kSegElems - 1) / kSegElems));
#define RWKVQ_Q(DT, V) quant_fp8_kernel<DT, V><<<grid, kThreads, 0, st>>>(x, codes, scale, amax, K, ldx, ldc, div_mode, from_bf16)
    if (x_dtype == RWKVQ_F16) { if (vec) RWKVQ_Q(RWKVQ_F16, true); else RWKVQ_Q(RWKVQ_F16, false); }
    else                      { if (vec) RWKVQ_Q(RWKVQ_BF16, true); else RWKVQ_Q(RWKVQ_BF16, false); }
#undef RWKVQ_Q
    return check_launch("actq_fp8");
}

int32_t rwkvq_prep_x_fp8(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes, int64_t ldc,
                         float* scale, float* amax_scratch, void* stream) {
    RWKVQ_REQUIRE(scale != nullptr, RWKVQ_E_BADARG, "prep_x_fp8: scale is null");
    return rwkvq_actq_fp8(x, x_dtype, M, K, ldx, codes, ldc, amax_scratch, scale, RWKVQ_DIV_TORCH, 0u, stream);
}

static int32_t launch_quant_int8(const QInt8Args& qa, int nt, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, int64_t ldc,
                                 int32_t div_mode, cudaStream_t st, const char* who) {
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, x_dtype);
    RWKVQ_REQUIRE(div_mode == RWKVQ_DIV_IEEE || div_mode == RWKVQ_DIV_FULL, RWKVQ_E_BADARG, "%s: div_mode %d", who, div_mode);
    RWKVQ_REQUIRE(M >= 0 && K >= 0 && ldx >= K && ldc >= K, RWKVQ_E_SHAPE, "%s: M=%lld K=%lld", who, (long long)M, (long long)K);
    bool vec = (K % 8 == 0) && (ldx % 8 == 0) && (ldc % 8 == 0);
    for (int t = 0; t < nt; ++t) {
        RWKVQ_REQUIRE(qa.x[t] && qa.codes[t] && qa.scales[t], RWKVQ_E_BADARG, "%s: null pointer", who);
        vec = vec && aligned16(qa.x[t]) && ((uintptr_t)qa.codes[t] % 8 == 0);
    }
    if (M == 0) return RWKVQ_OK;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)M, (unsigned)nt);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl() ? 1 : 0;
    const int dm = div_mode;
    cudaError_t e;
    const bool keep = vec && K <= (int64_t)kThreads * 8 * 8 && M * nt <= 4 * (int64_t)sm_count();     // few rows: one read, registers
#define RWKVQ_Q(DT, V, KP) e = cudaLaunchKernelEx(&cfg, quant_int8_kernel<DT, V, KP>, qa, K, ldx, ldc, dm)
    if (x_dtype == RWKVQ_F16) { if (keep) RWKVQ_Q(RWKVQ_F16, true, true); else if (vec) RWKVQ_Q(RWKVQ_F16, true, false); else RWKVQ_Q(RWKVQ_F16, false, false); }
    else                      { if (keep) RWKVQ_Q(RWKVQ_BF16, true, true); else if (vec) RWKVQ_Q(RWKVQ_BF16, true, false); else RWKVQ_Q(RWKVQ_BF16, false, false); }
#undef RWKVQ_Q
    if (e != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
    }
    return check_launch(who);
}

int32_t rwkvq_prep_x_int8(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* codes, int64_t ldc,
                          float* scales, int32_t div_mode, void* stream) {
    QInt8Args qa{};
    qa.x[0] = x; qa.codes[0] = codes; qa.scales[0] = scales;
    return launch_quant_int8(qa, 1, x_dtype, M, K, ldx, ldc, div_mode, (cudaStream_t)stream, "prep_x_int8");
}

int32_t rwkvq_prep3_x_int8(const void* xr, const void* xk, const void* xv, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx,
                           int8_t* codes_r, int8_t* codes_k, int8_t* codes_v, int64_t ldc, float* scales_r, float* scales_k,
                           float* scales_v, int32_t div_mode, void* stream) {
    QInt8Args qa{};
    qa.x[0] = xr; qa.x[1] = xk; qa.x[2] = xv; qa.codes[0] = codes_r; qa.codes[1] = codes_k; qa.codes[2] = codes_v;
    qa.scales[0] = scales_r; qa.scales[1] = scales_k; qa.scales[2] = scales_v;
    return launch_quant_int8(qa, 3, x_dtype, M, K, ldx, ldc, div_mode, (cudaStream_t)stream, "prep3_x_int8");
}

int64_t rwkvq_actq_fp8_fused_scratch_bytes(void) { return (kFusedEpochWord + 32) * 4; }

static int32_t launch_actq_fused(ActqArgs a, int nt, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, int64_t ldc, void* scratch,
                                 int64_t scratch_bytes, int32_t* status, int32_t div_mode, uint32_t flags, cudaStream_t st, const char* who) {
    RWKVQ_REQUIRE(scratch != nullptr && a.amax_out != nullptr, RWKVQ_E_BADARG, "%s: null pointer", who);
    for (int t = 0; t < nt; ++t) {
        RWKVQ_REQUIRE(a.x[t] && a.codes[t], RWKVQ_E_BADARG, "%s: null pointer (tensor %d)", who, t);
        RWKVQ_REQUIRE(aligned16(a.x[t]) && ((uintptr_t)a.codes[t] & 7) == 0, RWKVQ_E_ALIGN, "%s: rows must be 16-byte (x) / 8-byte (codes) aligned", who);
    }
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, x_dtype);
    RWKVQ_REQUIRE(div_mode == RWKVQ_DIV_IEEE || div_mode == RWKVQ_DIV_FULL || div_mode == RWKVQ_DIV_TORCH, RWKVQ_E_BADARG, "%s: div_mode %d", who, div_mode);
    RWKVQ_REQUIRE(M > 0 && K > 0 && K % 8 == 0 && M < (1 << 30), RWKVQ_E_SHAPE, "%s: M=%lld K=%lld (K must be a multiple of 8)", who, (long long)M, (long long)K);
    RWKVQ_REQUIRE(ldx % 8 == 0 && ldx >= K && ldc % 8 == 0 && ldc >= K, RWKVQ_E_ALIGN, "%s: rows must be 16-byte (x) / 8-byte (codes) aligned", who);
    RWKVQ_REQUIRE(scratch_bytes >= rwkvq_actq_fp8_fused_scratch_bytes() && ((uintptr_t)scratch & 3) == 0, RWKVQ_E_WORKSPACE,
                  "%s: scratch of %lld bytes needed", who, (long long)rwkvq_actq_fp8_fused_scratch_bytes());
    a.nt = nt;
    a.cpt = (int)std::min<int64_t>(M, std::min<int64_t>(kFusedMaxCtas, 2 * (int64_t)sm_count()) / nt);
    a.after_bf16 = (flags & RWKVQ_FLAG_AMAX_AFTER_BF16) ? 1 : 0;
    a.from_bf16 = (flags & RWKVQ_FLAG_QUANT_FROM_BF16) ? 1 : 0;
    a.M = (int)M; a.K = (int)K; a.ldx = ldx; a.ldc = ldc; a.div_mode = div_mode; a.status = status ? status : device_status_ptr();
    a.slots = reinterpret_cast<float*>(scratch);
    a.flags = reinterpret_cast<uint32_t*>(scratch) + kFusedMaxCtas;
    a.wait_ns = wait_limit_ns();
    const char* small_env = std::getenv("RWKVQ_ACTQ_SMALL_MAX");         // read per call: a test switches forms in one process
    const int64_t small_max = small_env ? std::atoll(small_env) : (int64_t)8 * 8 * kSmallThreads;
    if (M * (K / 8) <= std::min<int64_t>(small_max, (int64_t)8 * 8 * kSmallThreads) && K / 8 < 65536) {
        // decode-sized block: a cluster of CTAs per tensor (about 4 vectors per thread), no grid rendezvous, programmatic
        // dependent launch (the scratch is not touched)
        static const int64_t light_max = std::getenv("RWKVQ_ACTQ_LIGHT_MAX") ? std::atoll(std::getenv("RWKVQ_ACTQ_LIGHT_MAX")) : 8 * 8 * kSmallThreadsLight;
        const int threads = M * (K / 8) <= light_max ? kSmallThreadsLight : kSmallThreads;
        int cluster = 1;
        while (cluster < 8 && M * (K / 8) > (int64_t)cluster * 4 * threads) cluster <<= 1;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)(nt * cluster));
        cfg.blockDim = dim3((unsigned)threads);
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)cluster;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = use_pdl() ? 2 : 1;
        const cudaError_t e = x_dtype == RWKVQ_F16 ? cudaLaunchKernelEx(&cfg, actq_fp8_small_kernel<RWKVQ_F16>, a)
                                                   : cudaLaunchKernelEx(&cfg, actq_fp8_small_kernel<RWKVQ_BF16>, a);
        if (e != cudaSuccess) {
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
        }
        return check_launch(who);
    }
    const char* two_env = std::getenv("RWKVQ_ACTQ_TWO_MAX");
    const int64_t two_max = two_env ? std::atoll(two_env) : kTwoMaxVectors;
    if (M * (K / 8) <= two_max) {
        // mid-sized block: abs-max pass and codes pass as two plain launches chained by programmatic dependent launch
        const int kv = (int)(K / 8);
        int cpr = 1;                                     // CTAs per row: about two CTAs per SM in all, 256+ vectors each
        while ((int64_t)M * cpr * nt < 2 * (int64_t)sm_count() && cpr * 2 * kTwoThreads <= kv) cpr <<= 1;
        const int rows = (int)std::min<int64_t>(M, std::max<int64_t>(1, 4 * (int64_t)sm_count() / (cpr * nt)));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)(rows * cpr), (unsigned)nt);
        cfg.blockDim = dim3(kTwoThreads);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = use_pdl() ? 1 : 0;
        cudaError_t e = x_dtype == RWKVQ_F16 ? cudaLaunchKernelEx(&cfg, actq_two_amax_kernel<RWKVQ_F16>, a, cpr)
                                             : cudaLaunchKernelEx(&cfg, actq_two_amax_kernel<RWKVQ_BF16>, a, cpr);
        if (e == cudaSuccess)
            e = x_dtype == RWKVQ_F16 ? cudaLaunchKernelEx(&cfg, actq_two_codes_kernel<RWKVQ_F16>, a, cpr)
                                     : cudaLaunchKernelEx(&cfg, actq_two_codes_kernel<RWKVQ_BF16>, a, cpr);
        if (e != cudaSuccess) {
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
        }
        g_launches.fetch_add(1, std::memory_order_relaxed);         // two launches: check_launch counts the other one
        return check_launch(who);
    }
    void* args[] = {(void*)&a};
    const bool keep = K / 8 <= kFusedThreads && M <= 8 * (int64_t)a.cpt;
    const void* fn = x_dtype == RWKVQ_F16
                         ? (keep ? (const void*)actq_fp8_fused_kernel<RWKVQ_F16, true> : (const void*)actq_fp8_fused_kernel<RWKVQ_F16, false>)
                         : (keep ? (const void*)actq_fp8_fused_kernel<RWKVQ_BF16, true> : (const void*)actq_fp8_fused_kernel<RWKVQ_BF16, false>);
    const cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(a.cpt * nt), dim3(kFusedThreads), args, 0, st);
    if (e != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
    }
    return check_launch(who);
}

int32_t rwkvq_actq_fp8_fused(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes, int64_t ldc,
                             float* amax, float* scale, void* scratch, int64_t scratch_bytes, int32_t* status, int32_t div_mode,
                             uint32_t flags, void* stream) {
    ActqArgs a{};
    a.x[0] = x; a.codes[0] = codes; a.amax_out = amax; a.scale_out[0] = scale;
    return launch_actq_fused(a, 1, x_dtype, M, K, ldx, ldc, scratch, scratch_bytes, status, div_mode, flags, (cudaStream_t)stream, "actq_fp8_fused");
}

int32_t rwkvq_actq_fp8_fused3(const void* xr, const void* xk, const void* xv, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx,
                              uint8_t* codes_r, uint8_t* codes_k, uint8_t* codes_v, int64_t ldc, float* amax3, void* scratch,
                              int64_t scratch_bytes, int32_t* status, int32_t div_mode, uint32_t flags, void* stream) {
    ActqArgs a{};
    a.x[0] = xr; a.x[1] = xk; a.x[2] = xv; a.codes[0] = codes_r; a.codes[1] = codes_k; a.codes[2] = codes_v; a.amax_out = amax3;
    return launch_actq_fused(a, 3, x_dtype, M, K, ldx, ldc, scratch, scratch_bytes, status, div_mode, flags, (cudaStream_t)stream, "actq_fp8_fused3");
}


void rwkvq_set_wait_limit_us(int64_t microseconds) { wait_limit_override().store(microseconds > 0 ? microseconds : -1); }

int32_t rwkvq_actq_fp8_given(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, uint8_t* codes, int64_t ldc, float* amax_out,
                             float* scale_out, void* ffn_scratch, int32_t div_mode, uint32_t flags, void* stream) {
    const char* who = "actq_fp8_given";
    RWKVQ_REQUIRE(x && codes && amax_out && ffn_scratch, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, x_dtype);
    RWKVQ_REQUIRE(div_mode == RWKVQ_DIV_IEEE || div_mode == RWKVQ_DIV_FULL || div_mode == RWKVQ_DIV_TORCH, RWKVQ_E_BADARG, "%s: div_mode %d", who, div_mode);
    RWKVQ_REQUIRE(M > 0 && K > 0 && K % 8 == 0 && M < (1 << 30), RWKVQ_E_SHAPE, "%s: M=%lld K=%lld (K must be a multiple of 8)", who, (long long)M, (long long)K);
    RWKVQ_REQUIRE(aligned16(x) && ldx % 8 == 0 && ldx >= K && ldc % 8 == 0 && ldc >= K && ((uintptr_t)codes & 7) == 0 && ((uintptr_t)ffn_scratch & 7) == 0,
                  RWKVQ_E_ALIGN, "%s: rows must be 16-byte (x) / 8-byte (codes, scratch) aligned", who);
    const int64_t nvec = M * (K / 8);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)std::min<int64_t>((nvec + kThreads * 4 - 1) / (kThreads * 4), 8 * (int64_t)sm_count()));
    cfg.blockDim = dim3(kThreads);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl() ? 1 : 0;
    const int m = (int)M, dm = div_mode, fb = (flags & RWKVQ_FLAG_QUANT_FROM_BF16) ? 1 : 0;
    float* ffn = reinterpret_cast<float*>(ffn_scratch);
    const cudaError_t e = x_dtype == RWKVQ_F16
        ? cudaLaunchKernelEx(&cfg, quant_fp8_given_kernel<RWKVQ_F16>, x, codes, amax_out, scale_out, ffn, m, K, ldx, ldc, dm, fb)
        : cudaLaunchKernelEx(&cfg, quant_fp8_given_kernel<RWKVQ_BF16>, x, codes, amax_out, scale_out, ffn, m, K, ldx, ldc, dm, fb);
    if (e != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
    }
    return check_launch(who);
}

int32_t rwkvq_actq_int8_given(const void* x, int32_t x_dtype, int64_t M, int64_t K, int64_t ldx, int8_t* codes, int64_t ldc, float* scales,
                              float* row_max, int32_t div_mode, void* stream) {
    const char* who = "actq_int8_given";
    RWKVQ_REQUIRE(x && codes && scales && row_max, RWKVQ_E_BADARG, "%s: null pointer", who);
    RWKVQ_REQUIRE(x_dtype == RWKVQ_F16 || x_dtype == RWKVQ_BF16, RWKVQ_E_BADARG, "%s: x_dtype %d", who, x_dtype);
    RWKVQ_REQUIRE(div_mode == RWKVQ_DIV_IEEE || div_mode == RWKVQ_DIV_FULL, RWKVQ_E_BADARG, "%s: div_mode %d", who, div_mode);
    RWKVQ_REQUIRE(M > 0 && K > 0 && K % 8 == 0 && M < (1 << 30), RWKVQ_E_SHAPE, "%s: M=%lld K=%lld (K must be a multiple of 8)", who, (long long)M, (long long)K);
    RWKVQ_REQUIRE(aligned16(x) && ldx % 8 == 0 && ldx >= K && ldc % 8 == 0 && ldc >= K && ((uintptr_t)codes & 7) == 0 && ((uintptr_t)row_max & 3) == 0,
                  RWKVQ_E_ALIGN, "%s: rows must be 16-byte (x) / 8-byte (codes) aligned", who);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)M);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl() ? 1 : 0;
    const int dm = div_mode;
    const cudaError_t e = x_dtype == RWKVQ_F16
        ? cudaLaunchKernelEx(&cfg, quant_int8_given_kernel<RWKVQ_F16>, x, codes, scales, row_max, K, ldx, ldc, dm)
        : cudaLaunchKernelEx(&cfg, quant_int8_given_kernel<RWKVQ_BF16>, x, codes, scales, row_max, K, ldx, ldc, dm);
    if (e != cudaSuccess) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return fail(RWKVQ_E_LAUNCH, "%s: %s", who, cudaGetErrorString(e));
    }
    return check_launch(who);
}

int32_t rwkvq_device_status(int32_t* host_status, int32_t clear) {
    RWKVQ_REQUIRE(host_status != nullptr, RWKVQ_E_BADARG, "device_status: null pointer");
    int* p = device_status_ptr();
    RWKVQ_REQUIRE(p != nullptr, RWKVQ_E_LAUNCH, "device_status: the status word's address is not available");
    cudaError_t e = cudaMemcpy(host_status, p, sizeof(int32_t), cudaMemcpyDeviceToHost);
    RWKVQ_REQUIRE(e == cudaSuccess, RWKVQ_E_LAUNCH, "device_status: %s", cudaGetErrorString(e));
    if (clear && *host_status != 0) {
        e = cudaMemset(p, 0, sizeof(int32_t));
        RWKVQ_REQUIRE(e == cudaSuccess, RWKVQ_E_LAUNCH, "device_status: %s", cudaGetErrorString(e));
    }
    return RWKVQ_OK;
}

int32_t rwkvq_selftest_timeout(int32_t* status, void* scratch4, int64_t limit_us, int32_t mode, void* stream) {
    RWKVQ_REQUIRE(status != nullptr && scratch4 != nullptr, RWKVQ_E_BADARG, "selftest_timeout: null pointer");
    RWKVQ_REQUIRE(limit_us > 0 && limit_us <= 1000000 && (mode == 0 || mode == 1), RWKVQ_E_BADARG, "selftest_timeout: limit_us in (0, 1e6], mode 0 or 1");
    selftest_timeout_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(status, reinterpret_cast<uint32_t*>(scratch4), (unsigned long long)limit_us * 1000ull, mode);
    return check_launch("selftest_timeout");
}

}  // extern "C"
