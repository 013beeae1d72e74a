// Data-parallel SGD step over peer memory: gradient reduction, table update and broadcast of the updated tables in
// one kernel (no reference counterpart: the reference trains on one device).
//
// Every rank keeps its dense table gradient and its tables in buffers the other ranks of the node have mapped
// (CUDA IPC; NVLink / NVSwitch carries the accesses).  Rank r owns the slice [begin, end) of the tables: its kernel
// fetches that slice of every rank's gradient (its own from HBM, the others over the links), sums them in rank order,
// applies  w <- w - scale * sum  to its own copy and stores the new values into every rank's tables (peer stores).
// Bytes over the links: a rank fetches (G-1)/G of the gradient bytes and stores (G-1)/G of the table bytes, and serves
// as much to the others: 2 (G-1)/G of the table bytes per GPU and direction, what a ring all-reduce moves in two
// phases, but single hop, with the optimiser pass folded in and no staging buffers.  Every element is computed by
// exactly one rank, so the replicas stay bit-identical.
//
// The update kernel waits on no other rank: the caller orders it after every rank's gradient is complete and orders
// the next reader of the tables after every rank's kernel (lutb_peer_barrier below, or a collective of the process
// group; see spiky_b200/data_parallel.py PeerTableUpdate).
#include <string.h>

#include "lutb_common.cuh"
#include "mbarrier.cuh"

namespace lutb {
namespace {

constexpr int kMaxPeerRanks = LUTB_MAX_PEER_RANKS;

struct PeerArgs {
    const float *grad[kMaxPeerRanks];
    float *weights[kMaxPeerRanks];
    int n_ranks;
    int rank;
    int64_t begin, end;  // the slice this rank owns, in floats
    float scale;
};

// The body of the slice is cut into pieces of kPieceFloats (1024 floats; 512 beyond 8 ranks); piece c belongs to block
// c % gridDim.x (one block per SM).  A producer warp streams, per piece, the n gradient pieces (the other ranks' over NVLink, this rank's from HBM) and the
// piece of this rank's tables into one stage of a shared-memory ring with bulk copies (cp.async.bulk + mbarrier
// transaction counts): a peer access takes microseconds, so the link is only kept busy by the bytes in flight, and the
// copy engine holds a whole ring of them per SM without occupying registers or warps.  Eight consumer warps add the
// gradient pieces in rank order, apply the step and store the result into every rank's tables (plain 16-byte stores:
// peer stores are posted, nothing waits for them).  One block of 288 threads per SM leaves most of the SM to the
// backward kernels this update overlaps with.  Every wait is bounded; a wait that runs out is counted
// (lutb_device_wait_errors), the block stops taking pieces and leaves after a bounded wait for its copies in flight.
constexpr int kPeerConsumerWarps = 8;
constexpr int kPeerThreads = (kPeerConsumerWarps + 1) * 32;
constexpr int kPeerMaxStages = 16;
constexpr size_t kPeerRingBytes = 128 * 1024;   // half of the SM's shared memory: the rest stays L1 for the kernels beside it

__device__ int g_peer_wait_errors = 0;

__device__ __forceinline__ void store_stream(float4 *p, float4 v) { __stcs(p, v); }

// explicit multiply then subtract (no contraction into an FMA): the result is the fp32 expression  w - scale * g
__device__ __forceinline__ float sgd(float w, float g, float scale) { return __fsub_rn(w, __fmul_rn(scale, g)); }

__global__ void __launch_bounds__(kPeerThreads) peer_sgd_kernel(const PeerArgs a, int n_stages, int kPieceFloats) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int n = a.n_ranks;
    const int stage_floats = (n + 1) * kPieceFloats;   // n gradient pieces, then the piece of the tables
    float *ring = reinterpret_cast<float *>(smem);
    unsigned char *tail = smem + (size_t)n_stages * stage_floats * sizeof(float);
    const uint32_t full0 = smem_u32(tail), empty0 = full0 + 8 * kPeerMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tail + 16 * kPeerMaxStages);
    if (threadIdx.x == 0) {
        for (int st = 0; st < n_stages; st++) {
            mbar_init(full0 + 8 * st, 1);                       // the producer's arrive + the copies' bytes
            mbar_init(empty0 + 8 * st, kPeerConsumerWarps);     // one arrive per consumer warp
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    // 16-byte body of the slice: buffers are 256-byte aligned allocations, so float indices that are multiples of 4 are
    // 16-byte aligned in every rank's buffer
    const int64_t f0 = ((a.begin + 3) >> 2) << 2, f1 = (a.end >> 2) << 2;
    const int64_t n_pieces = f1 > f0 ? (f1 - f0 + kPieceFloats - 1) / kPieceFloats : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t slot = 0, phase = 0;

    if (warp == kPeerConsumerWarps) {
        // ---- producer
        uint32_t issued = 0;
        bool ok = true;
        for (int64_t c = blockIdx.x; c < n_pieces && ok; c += gridDim.x) {
            // a fresh barrier passes the wait for parity 1, so the first round does not wait
            if (!mbar_wait(empty0 + 8 * slot, phase ^ 1u) || *abort_flag) { ok = false; break; }
            if (lane == 0) {
                const int64_t e0 = f0 + c * kPieceFloats;
                const uint32_t bytes = (uint32_t)(min((int64_t)kPieceFloats, f1 - e0) * 4);
                float *dst = ring + (size_t)slot * stage_floats;
                mbar_arrive_expect_tx(full0 + 8 * slot, bytes * (uint32_t)(n + 1));
                // the other ranks' pieces first: they take longest
                for (int k = 1; k <= n; k++) {
                    const int r = (a.rank + k) % n;
                    bulk_copy_g2s(smem_u32(dst + (size_t)r * kPieceFloats), a.grad[r] + e0, bytes, full0 + 8 * slot);
                }
                bulk_copy_g2s(smem_u32(dst + (size_t)n * kPieceFloats), a.weights[a.rank] + e0, bytes, full0 + 8 * slot);
            }
            __syncwarp();
            if (++slot == (uint32_t)n_stages) { slot = 0; phase ^= 1u; }
            issued++;
        }
        if (!ok) {
            if (lane == 0) { atomicAdd(&g_peer_wait_errors, 1); *abort_flag = 1; }
            // the block is leaving early: give the copies still in flight a bounded time to land
            const uint32_t back = min(issued, (uint32_t)n_stages);
            for (uint32_t k = 0; k < back; k++) {
                const uint32_t item = issued - 1 - k;
                if (!mbar_wait(full0 + 8 * (item % n_stages), (item / n_stages) & 1u)) break;
            }
        }
    } else {
        // ---- consumers: warp w takes the 16-byte elements w, w + 8, ... of every 32-element row of the piece
        for (int64_t c = blockIdx.x; c < n_pieces; c += gridDim.x) {
            if (*abort_flag) break;
            if (!mbar_wait(full0 + 8 * slot, phase)) {
                if (lane == 0) { atomicAdd(&g_peer_wait_errors, 1); *abort_flag = 1; }
                break;
            }
            const int64_t e0 = f0 + c * kPieceFloats;
            const int vecs = (int)(min((int64_t)kPieceFloats, f1 - e0) >> 2);
            const float4 *src = reinterpret_cast<const float4 *>(ring + (size_t)slot * stage_floats);
            for (int v = warp * 32 + lane; v < vecs; v += kPeerConsumerWarps * 32) {
                float4 acc = src[v];
                for (int r = 1; r < n; r++) {
                    const float4 g = src[r * (kPieceFloats / 4) + v];
                    acc.x += g.x;
                    acc.y += g.y;
                    acc.z += g.z;
                    acc.w += g.w;
                }
                float4 w = src[n * (kPieceFloats / 4) + v];
                w.x = sgd(w.x, acc.x, a.scale);
                w.y = sgd(w.y, acc.y, a.scale);
                w.z = sgd(w.z, acc.z, a.scale);
                w.w = sgd(w.w, acc.w, a.scale);
                const int64_t i = (e0 >> 2) + v;
                for (int r = 0; r < n; r++) store_stream(reinterpret_cast<float4 *>(a.weights[r]) + i, w);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * slot);
            if (++slot == (uint32_t)n_stages) { slot = 0; phase ^= 1u; }
        }
        // ragged ends of the slice (at most 3 floats each side), one thread per element
        if (blockIdx.x == 0 && warp == 0) {
            const int64_t body0 = min(f0, a.end), body1 = max(f1, body0);
            const int64_t head = body0 - a.begin, tail_n = a.end - body1;
            if ((int64_t)lane < head + tail_n) {
                const int64_t e = (int64_t)lane < head ? a.begin + lane : body1 + (lane - head);
                float acc = a.grad[0][e];
                for (int r = 1; r < n; ++r) acc += a.grad[r][e];
                const float w = sgd(a.weights[a.rank][e], acc, a.scale);
                for (int r = 0; r < n; ++r) a.weights[r][e] = w;
            }
        }
    }
}

// ---- broadcast of a local byte range into the same place of every rank's buffer (peer stores are posted: nothing
// waits for them, so a modest grid fills the outgoing links and leaves most of the SMs to the kernels beside it).
struct BroadcastArgs {
    unsigned char *dst[kMaxPeerRanks];
    const unsigned char *src;
    int n_ranks;
    int64_t offset, bytes;   // dst[r] + offset .. + bytes  <-  src .. + bytes
};

constexpr int kBroadcastThreads = 256;
constexpr int kBroadcastUnroll = 8;   // 128 bytes of local loads in flight per thread: the source side must not be the limit

__global__ void __launch_bounds__(kBroadcastThreads) peer_broadcast_kernel(const BroadcastArgs a) {
    // 16-byte body where source and destinations are aligned alike, single bytes at the two ends (and everywhere when
    // they are not: callers keep offsets 16-byte aligned)
    const uintptr_t s0 = reinterpret_cast<uintptr_t>(a.src);
    bool same = true;
    for (int r = 0; r < a.n_ranks; r++) same = same && (((reinterpret_cast<uintptr_t>(a.dst[r]) + a.offset) ^ s0) & 15) == 0;
    int64_t head = same ? (int64_t)((16 - (s0 & 15)) & 15) : a.bytes;
    if (head > a.bytes) head = a.bytes;
    const int64_t vecs = (a.bytes - head) >> 4;
    const int64_t tail0 = head + (vecs << 4);
    const int64_t tid = (int64_t)blockIdx.x * kBroadcastThreads + threadIdx.x, stride = (int64_t)gridDim.x * kBroadcastThreads;
    const uint4 *src4 = reinterpret_cast<const uint4 *>(a.src + head);
    for (int64_t i0 = tid; i0 < vecs; i0 += stride * kBroadcastUnroll) {
        uint4 v[kBroadcastUnroll];
#pragma unroll
        for (int u = 0; u < kBroadcastUnroll; u++) {
            const int64_t i = i0 + u * stride;
            if (i < vecs) v[u] = __ldcs(src4 + i);
        }
#pragma unroll
        for (int u = 0; u < kBroadcastUnroll; u++) {
            const int64_t i = i0 + u * stride;
            if (i < vecs)
                for (int r = 0; r < a.n_ranks; r++) __stcs(reinterpret_cast<uint4 *>(a.dst[r] + a.offset + head) + i, v[u]);
        }
    }
    // the ends: at most 15 bytes each in the aligned case
    for (int64_t e = tid; e < head + (a.bytes - tail0); e += stride) {
        const int64_t b = e < head ? e : tail0 + (e - head);
        const unsigned char c = a.src[b];
        for (int r = 0; r < a.n_ranks; r++) a.dst[r][a.offset + b] = c;
    }
}

// ---- barrier over the ranks, through flags in peer memory.  Every rank owns an array of one 64-bit flag per rank.
// Thread r of the (single) block stores the epoch into this rank's slot of rank r's array (release, system scope: the
// stores of the kernels launched before it on the stream are visible to whoever reads the flag) and then polls rank r's
// slot of its own array until it holds the epoch (acquire).  Epochs only grow, so nothing is ever reset.  The wait is
// bounded by the SM clock; a wait that runs out is counted (lutb_device_wait_errors) and the kernel returns.
constexpr long long kBarrierLimitCycles = 4000ll * 1000ll * 1000ll;   // about two seconds of SM clock

struct BarrierArgs {
    unsigned long long *flags[kMaxPeerRanks];
    int n_ranks;
    int rank;
    unsigned long long epoch;
};

__global__ void peer_barrier_kernel(const BarrierArgs a) {
    const int r = threadIdx.x;
    // epoch 0: the epoch is this rank's own count of barriers on these flags, kept in device memory behind the rank
    // slots of its array (the launch carries no changing argument, so it may be replayed from a CUDA graph)
    __shared__ unsigned long long epoch_s;
    if (r == 0) {
        unsigned long long e = a.epoch;
        if (e == 0) {
            unsigned long long *counter = a.flags[a.rank] + kMaxPeerRanks;
            e = *counter + 1;
            *counter = e;
        }
        epoch_s = e;
    }
    __syncthreads();
    const unsigned long long epoch = epoch_s;
    if (r >= a.n_ranks) return;
    unsigned long long *out = a.flags[r] + a.rank;
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(out), "l"(epoch) : "memory");
    const unsigned long long *in = a.flags[a.rank] + r;
    const long long t0 = clock64();
    for (;;) {
        unsigned long long seen;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(in) : "memory");
        if (seen >= epoch) break;
        if (clock64() - t0 > kBarrierLimitCycles) {
            atomicAdd(&g_peer_wait_errors, 1);
            break;
        }
    }
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

int lutb_peer_broadcast(int32_t n_ranks, void *const *dst, int64_t dst_offset, const void *src, int64_t bytes,
                        void *stream) {
    LUTB_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeerRanks && dst, LUTB_ERR_SHAPE, "lutb_peer_broadcast: 1 <= n_ranks <= %d",
                 kMaxPeerRanks);
    LUTB_REQUIRE(dst_offset >= 0 && bytes >= 0 && (src || bytes == 0), LUTB_ERR_SHAPE, "lutb_peer_broadcast: bad range");
    if (bytes == 0) return LUTB_OK;
    BroadcastArgs a{};
    for (int r = 0; r < n_ranks; ++r) {
        LUTB_REQUIRE(dst[r], LUTB_ERR_NULL, "lutb_peer_broadcast: null buffer %d", r);
        a.dst[r] = static_cast<unsigned char *>(dst[r]);
    }
    a.src = static_cast<const unsigned char *>(src);
    a.n_ranks = n_ranks;
    a.offset = dst_offset;
    a.bytes = bytes;
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t per_block = (int64_t)kBroadcastThreads * kBroadcastUnroll * 16;
    const int64_t want = (bytes + per_block - 1) / per_block;
    // half of the SMs, one block each: with 37 blocks and 64 bytes per thread the copy ran at 570 GB/s, limited by the
    // local loads in flight (600 KB against a latency of about a microsecond)
    const int blocks = (int)max((int64_t)1, min((int64_t)max(device_info().sm_count / 2, 1), want));
    KernelScope scope(K_PEER_BROADCAST, s);
    peer_broadcast_kernel<<<blocks, kBroadcastThreads, 0, s>>>(a);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

int lutb_peer_copy(void *dst, const void *src, size_t bytes, void *stream) {
    LUTB_REQUIRE((dst && src) || bytes == 0, LUTB_ERR_NULL, "lutb_peer_copy: null pointer");
    if (bytes == 0) return LUTB_OK;
    // a plain asynchronous copy: between this GPU's memory and a mapped buffer of another it runs on a copy engine
    // over NVLink and occupies no SM
    LUTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return LUTB_OK;
}

int lutb_peer_barrier(int32_t n_ranks, int32_t rank, void *const *flags, uint64_t epoch, void *stream) {
    LUTB_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeerRanks, LUTB_ERR_SHAPE, "lutb_peer_barrier: 1 <= n_ranks <= %d",
                 kMaxPeerRanks);
    LUTB_REQUIRE(rank >= 0 && rank < n_ranks && flags, LUTB_ERR_SHAPE, "lutb_peer_barrier: bad rank or null");
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
    // as many stages as fit the ring: the bytes in flight per SM
    const int kPieceFloats = n_ranks <= 8 ? 1024 : 512;
    const size_t stage_bytes = (size_t)(n_ranks + 1) * kPieceFloats * sizeof(float);
    int n_stages = (int)(kPeerRingBytes / stage_bytes);
    if (n_stages > kPeerMaxStages) n_stages = kPeerMaxStages;
    LUTB_REQUIRE(n_stages >= 2, LUTB_ERR_SHAPE, "lutb_peer_sgd_update: too many ranks for the shared-memory ring");
    const size_t smem = (size_t)n_stages * stage_bytes + 16 * kPeerMaxStages + 16;
    // once per device, so that later launches (stream capture included) are launches only
    static unsigned long long attr_done = 0;
    const int dev = device_info().device;
    if (dev >= 64 || !((attr_done >> dev) & 1ull)) {
        LUTB_CUDA(cudaFuncSetAttribute(peer_sgd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(kPeerRingBytes + 16 * kPeerMaxStages + 16)));
        if (dev < 64) attr_done |= 1ull << dev;
    }
    const int64_t pieces = (vecs * 4 + kPieceFloats - 1) / kPieceFloats;
    const int blocks = (int)max((int64_t)1, min((int64_t)device_info().sm_count, pieces));
    peer_sgd_kernel<<<blocks, kPeerThreads, smem, s>>>(a, n_stages, kPieceFloats);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

}  // extern "C"
