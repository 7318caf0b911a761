// All-gather of the ranks' output blocks by plain stores into the peers' memory over NVLink / NVSwitch, one kernel per
// rank (one process per GPU), plus the two calls that make a device allocation of another process addressable here
// (CUDA IPC).  The reference has no multi-device path; this replaces the one NCCL all-gather at the end of the
// batch-sharded encoder (daceml_b200/distributed.py), whose launch and protocol cost more than its bytes at 8 MB per rank.
//
// Every rank owns a `gathered` buffer ([world][bytes_per_rank]) and 64 flag words, both mapped into every other rank's
// process.  One launch per rank and epoch e (a counter kept in the rank's own flag words, so a CUDA graph can replay
// the launch):
//   1. entered: CTA 0 writes e into flag word [rank] of every peer; every CTA waits until all peers have written e into
//      its own words - a peer that has entered e has finished, in stream order, whatever read its gathered buffer before;
//   2. push: every 16-byte packet of the local block is read once and stored into slot [rank] of every gathered buffer
//      (the local one included);
//   3. done: the CTA that finishes last writes e into flag word [16 + rank] of every peer and waits for the peers' e in
//      its own: when the kernel completes, this rank's gathered buffer holds every block.
// No load from peer memory, no multicast, no TMA: peer traffic is st.global of 16 bytes.  Flags are written with
// st.release.sys after __threadfence_system() and read with ld.acquire.sys.  Every wait is bounded (1 s); a wait that
// runs out records DEV_TIMEOUT_PEER in the context's status word and the kernel runs to its end without spinning again.
#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200ml {

namespace {

constexpr int PEER_THREADS = 512;
constexpr int PEER_UNROLL = 4;
constexpr int FLAG_ENTERED = 0, FLAG_DONE = 16, FLAG_EPOCH = 32, FLAG_ARRIVALS = 33;

struct PeerArgs {
    int32_t rank, world;
    int64_t packets;  // 16-byte packets per rank block
    const uint4* src;
    uint4* gathered[B200ML_MAX_PEERS];
    uint32_t* flags[B200ML_MAX_PEERS];
    int32_t* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Waits until *word has reached `epoch` (wrap-safe); false after kWaitLimitNs.
__device__ __forceinline__ bool wait_flag(const uint32_t* word, uint32_t epoch) {
    if (static_cast<int32_t>(ld_acquire_sys(word) - epoch) >= 0) return true;
    const uint64_t t0 = ptx::global_timer_ns();
    while (true) {
        for (int i = 0; i < 64; ++i) {
            if (static_cast<int32_t>(ld_acquire_sys(word) - epoch) >= 0) return true;
            __nanosleep(40);
        }
        if (ptx::global_timer_ns() - t0 > ptx::kWaitLimitNs) return false;
    }
}

__global__ void __launch_bounds__(PEER_THREADS) peer_allgather_kernel(const PeerArgs a) {
    __shared__ int s_ok, s_last;
    pdl_launch_dependents();
    pdl_wait();  // the block to send comes from the kernel before this one
    uint32_t* mine = a.flags[a.rank];
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(mine + FLAG_EPOCH) + 1;  // written by the previous launch
    const int t = threadIdx.x;
    if (t == 0) s_ok = 1;
    __syncthreads();
    // 1. entered
    if (t < a.world && t != a.rank) {
        if (blockIdx.x == 0) st_release_sys(a.flags[t] + FLAG_ENTERED + a.rank, epoch);
        if (!wait_flag(mine + FLAG_ENTERED + t, epoch)) {
            atomicExch(a.status, DEV_TIMEOUT_PEER);
            s_ok = 0;
        }
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    // 2. push: a packet is read once and stored world times
    if (ok) {
        const int64_t stride = static_cast<int64_t>(gridDim.x) * PEER_THREADS;
        const int64_t slot = static_cast<int64_t>(a.rank) * a.packets;
        for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * PEER_THREADS + t; i0 < a.packets; i0 += stride * PEER_UNROLL) {
            uint4 v[PEER_UNROLL];
#pragma unroll
            for (int u = 0; u < PEER_UNROLL; ++u) {
                const int64_t i = i0 + u * stride;
                if (i < a.packets) v[u] = __ldg(a.src + i);
            }
            for (int p = 0; p < a.world; ++p) {
                uint4* dst = a.gathered[p] + slot;
#pragma unroll
                for (int u = 0; u < PEER_UNROLL; ++u) {
                    const int64_t i = i0 + u * stride;
                    if (i < a.packets) dst[i] = v[u];
                }
            }
        }
    }
    // 3. done
    __threadfence_system();
    __syncthreads();
    if (t == 0) s_last = atomicAdd(mine + FLAG_ARRIVALS, 1u) == gridDim.x - 1 ? 1 : 0;
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        if (t < a.world && t != a.rank) {
            st_release_sys(a.flags[t] + FLAG_DONE + a.rank, epoch);
            if (ok && !wait_flag(mine + FLAG_DONE + t, epoch)) atomicExch(a.status, DEV_TIMEOUT_PEER);
        }
        __syncthreads();
        if (t == 0) {
            mine[FLAG_ARRIVALS] = 0;
            mine[FLAG_EPOCH] = epoch;
        }
    }
}

int peer_ctas() {
    static const int n = [] {
        const char* e = getenv("B200ML_PEER_CTAS");
        const int v = e ? atoi(e) : 0;
        return v > 0 && v <= 1024 ? v : 48;
    }();
    return n;
}

}  // namespace

int peer_allgather(const b200ml_ctx* ctx, const b200ml_peer_group* g, const void* src, int64_t bytes_per_rank, cudaStream_t stream) {
    B200ML_REQUIRE(g && g->world >= 1 && g->world <= B200ML_MAX_PEERS && g->rank >= 0 && g->rank < g->world,
                   "peer_allgather: bad rank %d of %d (at most %d ranks)", g ? g->rank : -1, g ? g->world : -1, B200ML_MAX_PEERS);
    B200ML_REQUIRE(bytes_per_rank >= 0 && bytes_per_rank % 16 == 0 && aligned16(src), "peer_allgather: the block must be 16-byte aligned and a multiple of 16 bytes");
    PeerArgs a{};
    a.rank = g->rank;
    a.world = g->world;
    a.packets = bytes_per_rank / 16;
    a.src = static_cast<const uint4*>(src);
    for (int r = 0; r < g->world; ++r) {
        B200ML_REQUIRE(g->gathered[r] && g->flags[r] && aligned16(g->gathered[r]), "peer_allgather: rank %d's buffers are not mapped", r);
        a.gathered[r] = static_cast<uint4*>(g->gathered[r]);
        a.flags[r] = static_cast<uint32_t*>(g->flags[r]);
    }
    a.status = ctx->status_dev;
    int64_t want = ceil_div(a.packets, static_cast<int64_t>(PEER_THREADS) * PEER_UNROLL);
    const int grid = static_cast<int>(want < 1 ? 1 : (want < peer_ctas() ? want : peer_ctas()));
    B200ML_CUDA(launch_pdl(peer_allgather_kernel, dim3(grid), dim3(PEER_THREADS), 0, stream, a));
    return check_launch("peer_allgather");
}

// The handle of the allocation that holds `ptr` and ptr's offset inside it, for another process on this box.
int ipc_export(const b200ml_ctx* ctx, const void* ptr, void* handle64, int64_t* offset) {
    B200ML_REQUIRE(ptr && handle64 && offset, "ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    B200ML_REQUIRE(ctx->mem_get_address_range, "ipc_export: cuMemGetAddressRange is not available");
    CUdeviceptr base = 0;
    size_t size = 0;
    using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
    CUresult r = reinterpret_cast<RangeFn>(ctx->mem_get_address_range)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
    if (r != CUDA_SUCCESS) return fail(B200ML_ERR_CUDA, "ipc_export: cuMemGetAddressRange failed with CUresult %d", (int)r);
    cudaIpcMemHandle_t h;
    B200ML_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
    memcpy(handle64, &h, 64);
    *offset = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
    return B200ML_OK;
}

// Maps another process's allocation into this one (peer access from the current device is enabled as needed).
int ipc_open(const b200ml_ctx*, const void* handle64, int64_t offset, void** ptr) {
    B200ML_REQUIRE(handle64 && ptr && offset >= 0, "ipc_open: bad argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* base = nullptr;
    B200ML_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = static_cast<uint8_t*>(base) + offset;
    return B200ML_OK;
}

int ipc_close(const b200ml_ctx*, void* ptr, int64_t offset) {
    if (!ptr) return B200ML_OK;
    B200ML_CUDA(cudaIpcCloseMemHandle(static_cast<uint8_t*>(ptr) - offset));
    return B200ML_OK;
}

}  // namespace b200ml

extern "C" int b200ml_peer_allgather(b200ml_ctx* ctx, const b200ml_peer_group* group, const void* src, int64_t bytes_per_rank,
                                     b200ml_stream stream) {
    using namespace b200ml;
    if (ctx == nullptr) return fail(B200ML_ERR_INVALID, "peer_allgather: null context");
    DeviceGuard guard(ctx->device);
    return peer_allgather(ctx, group, src, bytes_per_rank, static_cast<cudaStream_t>(stream));
}
extern "C" int b200ml_ipc_export(b200ml_ctx* ctx, const void* ptr, void* handle64, int64_t* offset) {
    using namespace b200ml;
    if (ctx == nullptr) return fail(B200ML_ERR_INVALID, "ipc_export: null context");
    DeviceGuard guard(ctx->device);
    return ipc_export(ctx, ptr, handle64, offset);
}
extern "C" int b200ml_ipc_open(b200ml_ctx* ctx, const void* handle64, int64_t offset, void** ptr) {
    using namespace b200ml;
    if (ctx == nullptr) return fail(B200ML_ERR_INVALID, "ipc_open: null context");
    DeviceGuard guard(ctx->device);
    return ipc_open(ctx, handle64, offset, ptr);
}
extern "C" int b200ml_ipc_close(b200ml_ctx* ctx, void* ptr, int64_t offset) {
    using namespace b200ml;
    if (ctx == nullptr) return fail(B200ML_ERR_INVALID, "ipc_close: null context");
    DeviceGuard guard(ctx->device);
    return ipc_close(ctx, ptr, offset);
}
