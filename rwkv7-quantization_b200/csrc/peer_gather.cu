// All-gather along the output features for a column-split projection, written for NVLink peer memory.
//
// Every rank holds one buffer OUT [M, N] that its peers can address (exchanged once, e.g. by CUDA IPC).  A rank's
// projection writes its own N/world columns straight into OUT (the GEMM entry points take a leading dimension), then
//   rwkvq_peer_signal        publishes "my columns of call `epoch` are complete" in every peer's flag array
//                            (system-scope release after a system-scope fence), and
//   rwkvq_allgather_cols_pull waits -- bounded -- for each peer's flag and copies that peer's columns out of the peer's
//                            OUT into the local OUT with plain 16-byte peer loads: the result lands in its final
//                            [M, N] layout, no staging buffer and no transposing copy.
// Waits are bounded by the library's wait limit; a rank that never signals leaves RWKVQ_E_TIMEOUT in the status word
// and the kernel returns.  No TMA and no multicast is used on peer memory: ordinary loads and stores only.
#include <algorithm>
#include <cstring>

#include "common.cuh"

namespace rwkvq {

constexpr int kMaxPeers = 16;

struct PeerPtrs {
    void* p[kMaxPeers];
};

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// flags[r] of rank q's flag array = the last epoch rank r has completed.  One thread per peer.
__global__ void peer_signal_kernel(PeerPtrs flag_arrays, int rank, int world, uint32_t epoch) {
    __threadfence_system();                                   // this rank's earlier writes to its OUT are visible system-wide
    if ((int)threadIdx.x < world) st_release_sys_u32(reinterpret_cast<uint32_t*>(flag_arrays.p[threadIdx.x]) + rank, epoch);
}

// Bounded wait for *p == want at system scope (the writer is another GPU).
__device__ __forceinline__ bool wait_peer_flag(const uint32_t* p, uint32_t want, unsigned long long limit_ns) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
        if (ld_acquire_sys_u32(p) == want) return true;
        __nanosleep(200);
    }
    const unsigned long long t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            if (ld_acquire_sys_u32(p) == want) return true;
            __nanosleep(500);
        }
        if (global_ns() - t0 > limit_ns) return false;
    }
}

// grid: (chunks of rows, world - 1 sources).  Source s (skipping this rank) -> its columns [s*nl, (s+1)*nl) of every row.
__global__ void __launch_bounds__(256) allgather_cols_pull_kernel(PeerPtrs outs, const uint32_t* my_flags, uint32_t epoch, int rank, int world,
                                                                   int M, int nl, int64_t ld, int rows_per_cta, int* status,
                                                                   unsigned long long wait_ns) {
    __shared__ int s_ok;
    const int src = (int)blockIdx.y + ((int)blockIdx.y >= rank ? 1 : 0);
    if (threadIdx.x == 0) {
        s_ok = wait_peer_flag(my_flags + src, epoch, wait_ns) ? 1 : 0;
        if (!s_ok && status) atomicExch(status, RWKVQ_E_TIMEOUT);
    }
    __syncthreads();
    if (!s_ok) return;
    const __half* from = reinterpret_cast<const __half*>(outs.p[src]) + (int64_t)src * nl;
    __half* to = reinterpret_cast<__half*>(outs.p[rank]) + (int64_t)src * nl;
    const int r0 = blockIdx.x * rows_per_cta, r1 = min(M, r0 + rows_per_cta);
    const int vec = nl >> 3;                                  // 16-byte vectors per row slice
    for (int r = r0; r < r1; ++r) {
        const uint4* f = reinterpret_cast<const uint4*>(from + (int64_t)r * ld);
        uint4* t = reinterpret_cast<uint4*>(to + (int64_t)r * ld);
        for (int i = threadIdx.x; i < vec; i += 4 * blockDim.x) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (i + j * (int)blockDim.x < vec) {
                    const uint4* p = f + i + j * blockDim.x;
                    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(v[j].x), "=r"(v[j].y), "=r"(v[j].z), "=r"(v[j].w) : "l"(p) : "memory");
                }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (i + j * (int)blockDim.x < vec) t[i + j * blockDim.x] = v[j];
        }
    }
}

// Receiver side of a projection that PUSHES its result to the peers: wait, bounded, until every other rank has
// published `epoch`.  One thread per source rank.
__global__ void peer_wait_kernel(const uint32_t* my_flags, uint32_t epoch, int rank, int world, int* status, unsigned long long wait_ns) {
    const int src = (int)threadIdx.x;
    if (src < world && src != rank && !wait_peer_flag(my_flags + src, epoch, wait_ns) && status) atomicExch(status, RWKVQ_E_TIMEOUT);
}

}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

/* Make memory of `peer_device` addressable from kernels of the current device (cudaDeviceEnablePeerAccess; already
 * enabled counts as success).  RWKVQ_E_ARCH if the two devices cannot reach each other. */
int32_t rwkvq_enable_peer_access(int32_t peer_device) {
    int dev = 0, can = 0;
    cudaError_t e = cudaGetDevice(&dev);
    RWKVQ_REQUIRE(e == cudaSuccess, RWKVQ_E_LAUNCH, "enable_peer_access: %s", cudaGetErrorString(e));
    if (dev == peer_device) return RWKVQ_OK;
    e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
    RWKVQ_REQUIRE(e == cudaSuccess && can, RWKVQ_E_ARCH, "enable_peer_access: device %d cannot address device %d", dev, peer_device);
    e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return RWKVQ_OK;
    }
    RWKVQ_REQUIRE(e == cudaSuccess, RWKVQ_E_LAUNCH, "enable_peer_access: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

/* Set-up calls of the peer buffers (the only entry points of this library that allocate; not for the serving loop).
 * rwkvq_peer_alloc: `bytes` of zeroed device memory on the current device plus its 64-byte CUDA IPC handle, to be sent
 * to the other ranks.  rwkvq_peer_open: maps another process's buffer from its handle, with THIS process's device
 * current, so that kernels of this device can address it (peer access between the two devices is set up by the open).
 * rwkvq_peer_close / rwkvq_peer_free undo them. */
int32_t rwkvq_peer_alloc(int64_t bytes, void** ptr_out, void* handle64_out) {
    RWKVQ_REQUIRE(bytes > 0 && ptr_out && handle64_out, RWKVQ_E_BADARG, "peer_alloc: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 bytes");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    RWKVQ_REQUIRE(e == cudaSuccess, RWKVQ_E_LAUNCH, "peer_alloc: cudaMalloc(%lld): %s", (long long)bytes, cudaGetErrorString(e));
    e = cudaMemset(p, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64_out), p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(RWKVQ_E_LAUNCH, "peer_alloc: %s", cudaGetErrorString(e));
    }
    *ptr_out = p;
    return RWKVQ_OK;
}

int32_t rwkvq_peer_open(const void* handle64, void** ptr_out) {
    RWKVQ_REQUIRE(handle64 && ptr_out, RWKVQ_E_BADARG, "peer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    RWKVQ_REQUIRE(e == cudaSuccess && p != nullptr, RWKVQ_E_LAUNCH, "peer_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    *ptr_out = p;
    return RWKVQ_OK;
}

int32_t rwkvq_peer_close(void* ptr) {
    const cudaError_t e = cudaIpcCloseMemHandle(ptr);
    RWKVQ_REQUIRE(e == cudaSuccess, RWKVQ_E_LAUNCH, "peer_close: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

int32_t rwkvq_peer_free(void* ptr) {
    const cudaError_t e = cudaFree(ptr);
    RWKVQ_REQUIRE(e == cudaSuccess, RWKVQ_E_LAUNCH, "peer_free: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

int32_t rwkvq_peer_signal(void* const* flag_arrays, int32_t rank, int32_t world, uint32_t epoch, void* stream) {
    RWKVQ_REQUIRE(flag_arrays != nullptr && world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, RWKVQ_E_BADARG,
                  "peer_signal: rank %d of %d", rank, world);
    PeerPtrs pp{};
    for (int i = 0; i < world; ++i) {
        RWKVQ_REQUIRE(flag_arrays[i] != nullptr && ((uintptr_t)flag_arrays[i] & 3) == 0, RWKVQ_E_BADARG, "peer_signal: flag array %d", i);
        pp.p[i] = flag_arrays[i];
    }
    peer_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pp, rank, world, epoch);
    return check_launch("peer_signal");
}

/* Wait on `stream` until flags[r] == epoch for every r != rank (the other ranks' pushed columns of this call are in
 * this rank's buffer); a rank that never signals leaves RWKVQ_E_TIMEOUT in *status after the wait limit. */
int32_t rwkvq_peer_wait(const uint32_t* my_flags, uint32_t epoch, int32_t rank, int32_t world, int32_t* status, void* stream) {
    RWKVQ_REQUIRE(my_flags != nullptr && world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, RWKVQ_E_BADARG, "peer_wait: rank %d of %d", rank, world);
    if (world == 1) return RWKVQ_OK;
    peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(my_flags, epoch, rank, world, status ? status : device_status_ptr(), wait_limit_ns());
    return check_launch("peer_wait");
}

int32_t rwkvq_allgather_cols_pull(void* const* outs, const uint32_t* my_flags, uint32_t epoch, int32_t rank, int32_t world, int64_t M,
                                  int64_t n_local, int64_t ld, int32_t* status, void* stream) {
    const char* who = "allgather_cols_pull";
    RWKVQ_REQUIRE(outs != nullptr && my_flags != nullptr && world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, RWKVQ_E_BADARG,
                  "%s: rank %d of %d", who, rank, world);
    RWKVQ_REQUIRE(M >= 0 && M < (1 << 30) && n_local > 0 && n_local % 8 == 0 && ld >= n_local * world && ld % 8 == 0, RWKVQ_E_SHAPE,
                  "%s: M=%lld n_local=%lld ld=%lld (slices of a multiple of 8 columns, 16-byte aligned rows)", who, (long long)M,
                  (long long)n_local, (long long)ld);
    PeerPtrs pp{};
    for (int i = 0; i < world; ++i) {
        RWKVQ_REQUIRE(outs[i] != nullptr && aligned16(outs[i]), RWKVQ_E_ALIGN, "%s: buffer of rank %d must be 16-byte aligned", who, i);
        pp.p[i] = outs[i];
    }
    if (M == 0 || world == 1) return RWKVQ_OK;
    // enough CTAs to keep the links busy, each with whole rows: about 64 KB per CTA
    int rows_per_cta = (int)std::max<int64_t>(1, 65536 / (n_local * 2));
    int64_t chunks = (M + rows_per_cta - 1) / rows_per_cta;
    const int64_t want = std::max<int64_t>(1, 4 * (int64_t)sm_count() / (world - 1));
    if (chunks > want) {
        rows_per_cta = (int)((M + want - 1) / want);
        chunks = (M + rows_per_cta - 1) / rows_per_cta;
    }
    allgather_cols_pull_kernel<<<dim3((unsigned)chunks, (unsigned)(world - 1)), 256, 0, (cudaStream_t)stream>>>(
        pp, my_flags, epoch, rank, world, (int)M, (int)n_local, ld, rows_per_cta, status ? status : device_status_ptr(), wait_limit_ns());
    return check_launch(who);
}

}  // extern "C"
