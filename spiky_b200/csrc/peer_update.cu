// Data-parallel SGD step over peer memory: gradient reduction, table update and broadcast of the updated tables in
// one kernel (no reference counterpart: the reference trains on one device).
//
// Every rank keeps its dense table gradient and its tables in buffers the other ranks of the node have mapped
// (CUDA IPC; NVLink / NVSwitch carries the accesses).  Rank r owns the slice [begin, end) of the tables: its kernel
// loads that slice of every rank's gradient (its own from HBM, the others as peer loads), sums them in rank order,
// applies  w <- w - scale * sum  to its own copy and stores the new values into every rank's tables (peer stores).
// Bytes over the links per rank: (G-1)/G of the tables in, the same out, in both directions at once - what a ring
// all-reduce moves in two phases, but single hop, with the optimiser pass folded in and no staging buffers.  Every
// element is computed by exactly one rank, so the replicas stay bit-identical.
//
// The kernel waits on nothing: the caller orders it after every rank's gradient is complete and orders the next
// reader of the tables after every rank's kernel (stream-ordered barriers of the process group, see
// spiky_b200/data_parallel.py PeerTableUpdate).
#include <string.h>

#include "lutb_common.cuh"

namespace lutb {
namespace {

constexpr int kMaxPeerRanks = LUTB_MAX_PEER_RANKS;
constexpr int kPeerThreads = 256;

struct PeerArgs {
    const float *grad[kMaxPeerRanks];
    float *weights[kMaxPeerRanks];
    int n_ranks;
    int rank;
    int64_t begin, end;  // the slice this rank owns, in floats
    float scale;
};

__device__ __forceinline__ float4 load_stream(const float4 *p) { return __ldcs(p); }
__device__ __forceinline__ void store_stream(float4 *p, float4 v) { __stcs(p, v); }

// explicit multiply then subtract (no contraction into an FMA): the result is the fp32 expression  w - scale * g
__device__ __forceinline__ float sgd(float w, float g, float scale) { return __fsub_rn(w, __fmul_rn(scale, g)); }

// N > 0: number of ranks known at compile time; N == 0: any number of ranks up to kMaxPeerRanks.  A thread handles U
// 16-byte elements per trip, a block stride apart, and issues all N * U gradient loads before it uses any: a peer load
// takes microseconds over NVLink, so the link is only kept busy by the bytes in flight (threads x N x U x 16), and one
// block of 256 threads per SM (half of its registers at most) leaves the rest of the SM to the backward kernels this update overlaps with.
template <int N, int U>
__global__ void __launch_bounds__(kPeerThreads) peer_sgd_kernel(const PeerArgs a) {
    const int n = N > 0 ? N : a.n_ranks;
    // 16-byte body: buffers are 256-byte aligned allocations, so float index multiples of 4 are aligned everywhere
    const int64_t v0 = (a.begin + 3) >> 2, v1 = a.end >> 2;
    const int64_t stride = (int64_t)gridDim.x * kPeerThreads;
    const float *own_w = a.weights[a.rank];
    for (int64_t i0 = v0 + (int64_t)blockIdx.x * kPeerThreads + threadIdx.x; i0 < v1; i0 += stride * U) {
        float4 acc[U], w[U];
        if (N > 0) {
            float4 g[N > 0 ? N : 1][U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t i = i0 + u * stride;
                if (i < v1) {
#pragma unroll
                    for (int r = 0; r < N; ++r) g[r][u] = load_stream(reinterpret_cast<const float4 *>(a.grad[r]) + i);
                    w[u] = *(reinterpret_cast<const float4 *>(own_w) + i);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                acc[u] = g[0][u];
#pragma unroll
                for (int r = 1; r < N; ++r) {
                    acc[u].x += g[r][u].x;
                    acc[u].y += g[r][u].y;
                    acc[u].z += g[r][u].z;
                    acc[u].w += g[r][u].w;
                }
            }
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t i = i0 + u * stride;
                if (i < v1) {
                    acc[u] = load_stream(reinterpret_cast<const float4 *>(a.grad[0]) + i);
                    for (int r = 1; r < n; ++r) {
                        const float4 g = load_stream(reinterpret_cast<const float4 *>(a.grad[r]) + i);
                        acc[u].x += g.x;
                        acc[u].y += g.y;
                        acc[u].z += g.z;
                        acc[u].w += g.w;
                    }
                    w[u] = *(reinterpret_cast<const float4 *>(own_w) + i);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i < v1) {
                float4 v = w[u];
                v.x = sgd(v.x, acc[u].x, a.scale);
                v.y = sgd(v.y, acc[u].y, a.scale);
                v.z = sgd(v.z, acc[u].z, a.scale);
                v.w = sgd(v.w, acc[u].w, a.scale);
                if (N > 0) {
#pragma unroll
                    for (int r = 0; r < N; ++r) store_stream(reinterpret_cast<float4 *>(a.weights[r]) + i, v);
                } else {
                    for (int r = 0; r < n; ++r) store_stream(reinterpret_cast<float4 *>(a.weights[r]) + i, v);
                }
            }
        }
    }
    // ragged ends of the slice (at most 3 floats each side), one thread per element
    if (blockIdx.x == 0) {
        const int64_t body0 = min(v0 << 2, a.end), body1 = max(v1 << 2, body0);
        const int64_t head = body0 - a.begin, tail = a.end - body1;
        if ((int64_t)threadIdx.x < head + tail) {
            const int64_t e = (int64_t)threadIdx.x < head ? a.begin + threadIdx.x : body1 + (threadIdx.x - head);
            float acc = a.grad[0][e];
            for (int r = 1; r < n; ++r) acc += a.grad[r][e];
            const float w = sgd(own_w[e], acc, a.scale);
            for (int r = 0; r < n; ++r) a.weights[r][e] = w;
        }
    }
}

// elements per thread and trip: 16 gradient loads of 16 bytes in flight per thread up to 8 ranks
constexpr int unroll_of(int n) { return n == 0 ? 1 : (n <= 4 ? 4 : 2); }

// ---- barrier over the ranks, through flags in peer memory.  Every rank owns an array of one 64-bit flag per rank.
// Thread r of the (single) block stores the epoch into this rank's slot of rank r's array (release, system scope: the
// stores of the kernels launched before it on the stream are visible to whoever reads the flag) and then polls rank r's
// slot of its own array until it holds the epoch (acquire).  Epochs only grow, so nothing is ever reset.  The wait is
// bounded by the SM clock; a wait that runs out is counted (lutb_device_wait_errors) and the kernel returns.
constexpr long long kBarrierLimitCycles = 4000ll * 1000ll * 1000ll;   // about two seconds of SM clock

__device__ int g_peer_wait_errors = 0;

struct BarrierArgs {
    unsigned long long *flags[kMaxPeerRanks];
    int n_ranks;
    int rank;
    unsigned long long epoch;
};

__global__ void peer_barrier_kernel(const BarrierArgs a) {
    const int r = threadIdx.x;
    if (r >= a.n_ranks) return;
    unsigned long long *out = a.flags[r] + a.rank;
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(out), "l"(a.epoch) : "memory");
    const unsigned long long *in = a.flags[a.rank] + r;
    const long long t0 = clock64();
    for (;;) {
        unsigned long long seen;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(in) : "memory");
        if (seen >= a.epoch) break;
        if (clock64() - t0 > kBarrierLimitCycles) {
            atomicAdd(&g_peer_wait_errors, 1);
            break;
        }
    }
}

template <int N>
void launch(const PeerArgs &a, int64_t vecs, cudaStream_t stream) {
    constexpr int U = unroll_of(N);
    const int64_t want = (vecs + (int64_t)kPeerThreads * U - 1) / ((int64_t)kPeerThreads * U);
    const int blocks = (int)max((int64_t)1, min((int64_t)device_info().sm_count, want));
    peer_sgd_kernel<N, U><<<blocks, kPeerThreads, 0, stream>>>(a);
}

}  // namespace

int peer_wait_errors(int *count_out) {
    LUTB_CUDA(cudaMemcpyFromSymbol(count_out, g_peer_wait_errors, sizeof(int)));
    return LUTB_OK;
}

}  // namespace lutb

using namespace lutb;

extern "C" {

int lutb_peer_alloc(size_t bytes, void **ptr_out, unsigned char *handle_out) {
    LUTB_REQUIRE(ptr_out && handle_out && bytes > 0, LUTB_ERR_NULL, "lutb_peer_alloc: null argument or zero size");
    static_assert(sizeof(cudaIpcMemHandle_t) == LUTB_PEER_HANDLE_BYTES, "handle size");
    void *p = nullptr;
    LUTB_CUDA(cudaMalloc(&p, bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        set_error("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    memcpy(handle_out, &h, sizeof(h));
    *ptr_out = p;
    return LUTB_OK;
}

int lutb_peer_free(void *ptr) {
    if (ptr) LUTB_CUDA(cudaFree(ptr));
    return LUTB_OK;
}

int lutb_peer_open(const unsigned char *handle, void **ptr_out) {
    LUTB_REQUIRE(handle && ptr_out, LUTB_ERR_NULL, "lutb_peer_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    LUTB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr_out = p;
    return LUTB_OK;
}

int lutb_peer_close(void *ptr) {
    if (ptr) LUTB_CUDA(cudaIpcCloseMemHandle(ptr));
    return LUTB_OK;
}

int lutb_peer_barrier(int32_t n_ranks, int32_t rank, void *const *flags, uint64_t epoch, void *stream) {
    LUTB_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeerRanks, LUTB_ERR_SHAPE, "lutb_peer_barrier: 1 <= n_ranks <= %d",
                 kMaxPeerRanks);
    LUTB_REQUIRE(rank >= 0 && rank < n_ranks && flags, LUTB_ERR_SHAPE, "lutb_peer_barrier: bad rank or null");
    LUTB_REQUIRE(epoch > 0, LUTB_ERR_SHAPE, "lutb_peer_barrier: epochs start at 1 (the flags start at 0)");
    BarrierArgs a{};
    for (int r = 0; r < n_ranks; ++r) {
        LUTB_REQUIRE(flags[r] && ((uintptr_t)flags[r] & 7) == 0, LUTB_ERR_ALIGN, "lutb_peer_barrier: flag array of rank %d", r);
        a.flags[r] = static_cast<unsigned long long *>(flags[r]);
    }
    a.n_ranks = n_ranks;
    a.rank = rank;
    a.epoch = epoch;
    cudaStream_t s = (cudaStream_t)stream;
    KernelScope scope(K_PEER_BARRIER, s);
    peer_barrier_kernel<<<1, 32, 0, s>>>(a);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

int lutb_peer_sgd_update(int32_t n_ranks, int32_t rank, const float *const *grads, float *const *weights,
                         int64_t begin, int64_t end, float scale, void *stream) {
    LUTB_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeerRanks, LUTB_ERR_SHAPE, "lutb_peer_sgd_update: 1 <= n_ranks <= %d",
                 kMaxPeerRanks);
    LUTB_REQUIRE(rank >= 0 && rank < n_ranks && grads && weights, LUTB_ERR_SHAPE, "lutb_peer_sgd_update: bad rank or null");
    LUTB_REQUIRE(begin >= 0 && end >= begin, LUTB_ERR_SHAPE, "lutb_peer_sgd_update: bad slice [%lld, %lld)",
                 (long long)begin, (long long)end);
    PeerArgs a{};
    for (int r = 0; r < n_ranks; ++r) {
        LUTB_REQUIRE(grads[r] && weights[r], LUTB_ERR_NULL, "lutb_peer_sgd_update: null buffer of rank %d", r);
        LUTB_REQUIRE(((uintptr_t)grads[r] & 15) == 0 && ((uintptr_t)weights[r] & 15) == 0, LUTB_ERR_ALIGN,
                     "lutb_peer_sgd_update: buffers must be 16-byte aligned");
        a.grad[r] = grads[r];
        a.weights[r] = weights[r];
    }
    if (end == begin) return LUTB_OK;
    a.n_ranks = n_ranks;
    a.rank = rank;
    a.begin = begin;
    a.end = end;
    a.scale = scale;
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t vecs = (end - begin + 3) / 4;
    KernelScope scope(K_PEER_SGD_UPDATE, s);
    switch (n_ranks) {
        case 1: launch<1>(a, vecs, s); break;
        case 2: launch<2>(a, vecs, s); break;
        case 3: launch<3>(a, vecs, s); break;
        case 4: launch<4>(a, vecs, s); break;
        case 5: launch<5>(a, vecs, s); break;
        case 6: launch<6>(a, vecs, s); break;
        case 7: launch<7>(a, vecs, s); break;
        case 8: launch<8>(a, vecs, s); break;
        default: launch<0>(a, vecs, s); break;
    }
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

}  // extern "C"
