// Ordered stream compaction of a dense 32-bit array into (index, value) lists: the step the Sparse gradient policy
// runs on the dense table gradient after every backward pass.
//
// Replaces DenseToSparseConverterNative (spiky_cuda/torch_utils/torch_utils.cu:11-340; kernels count_nonzero and
// densify, densify_new in spiky_cuda/torch_utils/torch_utils_kernels_logic.proto:1-131, 133-179, 181-324).  The reference appends through one global
// atomic counter, so its output order depends on scheduling; here the positions come from a two-level prefix sum
// (per-tile counts, one scan over the tiles, ballot ranks inside a tile), which makes the lists sorted by index and
// identical from run to run.  Bit patterns are compared, not values: -0.0f counts as non-zero like in the reference.
#include "lutb_common.cuh"

namespace lutb {

constexpr int kTileThreads = 256;
constexpr int kTileWords = kTileThreads * 8;  // two 16-byte loads per thread

__device__ __forceinline__ void load_tile_words(const uint32_t *__restrict__ src, int64_t n, int64_t tile, bool vec,
                                                uint32_t (&w)[8]) {
    // thread t owns words [t * 8, t * 8 + 8) of the tile, so ranks inside a thread follow index order
    const int64_t first = tile * kTileWords + (int64_t)threadIdx.x * 8;
    if (vec && first + 8 <= n) {
        const uint4 a = __ldg(reinterpret_cast<const uint4 *>(src + first));
        const uint4 b = __ldg(reinterpret_cast<const uint4 *>(src + first) + 1);
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    } else {
#pragma unroll
        for (int e = 0; e < 8; e++) w[e] = first + e < n ? __ldg(src + first + e) : 0u;
    }
}

__device__ __forceinline__ int count_words(const uint32_t (&w)[8]) {
    int c = 0;
#pragma unroll
    for (int e = 0; e < 8; e++) c += w[e] != 0u;
    return c;
}

// block-wide exclusive prefix of one int per thread; returns the thread's offset, *total gets the block sum
__device__ __forceinline__ int block_exclusive(int v, int *total) {
    __shared__ int warp_sums[kTileThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    int before = 0, all = 0;
#pragma unroll
    for (int i = 0; i < kTileThreads / 32; i++) {
        const int s = warp_sums[i];
        if (i < warp) before += s;
        all += s;
    }
    __syncthreads();
    *total = all;
    return before + incl - v;
}

__global__ void __launch_bounds__(kTileThreads) d2s_tile_count_kernel(const uint32_t *__restrict__ src, int64_t n, bool vec,
                                                                     int32_t *__restrict__ tile_counts) {
    uint32_t w[8];
    load_tile_words(src, n, blockIdx.x, vec, w);
    int total;
    block_exclusive(count_words(w), &total);
    if (threadIdx.x == 0) tile_counts[blockIdx.x] = total;
}

// One block scans the tile counts into starting positions (int64) and publishes the grand total.
__global__ void __launch_bounds__(kTileThreads) d2s_scan_tiles_kernel(const int32_t *__restrict__ tile_counts, int64_t n_tiles,
                                                                     int64_t *__restrict__ tile_starts,
                                                                     int64_t *__restrict__ total_out) {
    __shared__ int64_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int64_t base = 0; base < n_tiles; base += kTileThreads) {
        const int64_t i = base + threadIdx.x;
        const int v = i < n_tiles ? tile_counts[i] : 0;
        int total;
        const int off = block_exclusive(v, &total);
        if (i < n_tiles) tile_starts[i] = carry + off;
        __syncthreads();
        if (threadIdx.x == 0) carry += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) *total_out = carry;
}

__global__ void __launch_bounds__(kTileThreads) d2s_scatter_kernel(uint32_t *__restrict__ src, int64_t n, bool vec,
                                                                  const int64_t *__restrict__ tile_starts,
                                                                  int64_t *__restrict__ indices, uint32_t *__restrict__ values,
                                                                  int64_t capacity, int erase) {
    uint32_t w[8];
    load_tile_words(src, n, blockIdx.x, vec, w);
    const int mine = count_words(w);
    int total;
    int64_t pos = tile_starts[blockIdx.x] + block_exclusive(mine, &total);
    if (mine == 0) return;
    const int64_t first = (int64_t)blockIdx.x * kTileWords + (int64_t)threadIdx.x * 8;
#pragma unroll
    for (int e = 0; e < 8; e++) {
        if (w[e] != 0u) {
            if (pos < capacity) { indices[pos] = first + e; values[pos] = w[e]; }
            pos++;
        }
    }
    if (erase) {
        if (vec && first + 8 <= n) {
            reinterpret_cast<uint4 *>(src + first)[0] = make_uint4(0u, 0u, 0u, 0u);
            reinterpret_cast<uint4 *>(src + first)[1] = make_uint4(0u, 0u, 0u, 0u);
        } else {
#pragma unroll
            for (int e = 0; e < 8; e++)
                if (first + e < n) src[first + e] = 0u;
        }
    }
}

static int64_t tiles_of(int64_t n) { return (n + kTileWords - 1) / kTileWords; }

}  // namespace lutb

using namespace lutb;

extern "C" size_t lutb_dense_to_sparse_workspace(int64_t n) {
    if (n <= 0) return 0;
    const size_t t = (size_t)tiles_of(n);
    return ((t * 4 + 255) & ~(size_t)255) + t * 8 + 256;
}

static int d2s_count_pass(const uint32_t *src, int64_t n, void *workspace, size_t workspace_bytes, int64_t *total_out,
                          int32_t **counts_out, int64_t **starts_out, cudaStream_t st) {
    LUTB_REQUIRE(src && total_out, LUTB_ERR_NULL, "a required pointer is NULL");
    LUTB_REQUIRE(n > 0, LUTB_ERR_SHAPE, "empty source");
    LUTB_REQUIRE((reinterpret_cast<uintptr_t>(src) & 3) == 0, LUTB_ERR_ALIGN, "source must be 4-byte aligned");
    const int64_t t = tiles_of(n);
    LUTB_REQUIRE(t <= 0x7FFFFFFF, LUTB_ERR_SHAPE, "source too large");
    LUTB_REQUIRE(workspace && workspace_bytes >= lutb_dense_to_sparse_workspace(n), LUTB_ERR_WORKSPACE,
                 "dense_to_sparse needs %zu bytes of workspace", lutb_dense_to_sparse_workspace(n));
    const uintptr_t base = (reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t)255;
    int32_t *counts = reinterpret_cast<int32_t *>(base);
    int64_t *starts = reinterpret_cast<int64_t *>(base + (((size_t)t * 4 + 255) & ~(size_t)255));
    const bool vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    {
        KernelScope scope(K_DENSE_TO_SPARSE, st);
        d2s_tile_count_kernel<<<(unsigned)t, kTileThreads, 0, st>>>(src, n, vec, counts);
    }
    LUTB_LAUNCH_CHECK();
    {
        KernelScope scope(K_DENSE_TO_SPARSE, st);
        d2s_scan_tiles_kernel<<<1, kTileThreads, 0, st>>>(counts, t, starts, total_out);
    }
    LUTB_LAUNCH_CHECK();
    if (counts_out) *counts_out = counts;
    if (starts_out) *starts_out = starts;
    return LUTB_OK;
}

extern "C" int lutb_count_nonzero_32(const void *source, int64_t n, int64_t *count_out, void *workspace,
                                     size_t workspace_bytes, void *stream) {
    return d2s_count_pass(static_cast<const uint32_t *>(source), n, workspace, workspace_bytes, count_out, nullptr, nullptr,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int lutb_dense_to_sparse_32(void *source, int64_t n, int64_t *indices, void *values, int64_t capacity,
                                       int64_t *count_out, int erase_input, void *workspace, size_t workspace_bytes,
                                       void *stream) {
    LUTB_REQUIRE(indices && values, LUTB_ERR_NULL, "a required pointer is NULL");
    LUTB_REQUIRE(capacity >= 0, LUTB_ERR_SHAPE, "negative capacity");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint32_t *src = static_cast<uint32_t *>(source);
    int32_t *counts = nullptr;
    int64_t *starts = nullptr;
    int rc = d2s_count_pass(src, n, workspace, workspace_bytes, count_out, &counts, &starts, st);
    if (rc) return rc;
    const bool vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    KernelScope scope(K_DENSE_TO_SPARSE, st);
    d2s_scatter_kernel<<<(unsigned)tiles_of(n), kTileThreads, 0, st>>>(src, n, vec, starts, indices,
                                                                       static_cast<uint32_t *>(values), capacity, erase_input);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}
