// Deterministic table gradient of the non-sequence fully connected layer: counting sort of the batch by
// selected row (per detector, stable) followed by a segmented reduce.  Every cell of dW receives its
// contributions in ascending sample order, one rounded fp32 addition each - the order of the reference's
// host loop (gather_w_gradients_non_seq_fc_logic, lut_runtime_kernels_logic.proto:1547-1585) - so the
// result does not depend on scheduling and has no atomics on floating-point data.
//
// Scratch layout (all int32): counts [Nt][T][nblk] (turned into exclusive offsets in place), then perm [Nt][B].
#include "lutb_common.cuh"
#include "fc_dw_sorted.cuh"

#include <mutex>

namespace lutb {

constexpr int kSortBlock = 1024;  // samples per (detector, block) histogram slice

// counts[t][row][k] = number of samples of block k that selected `row` in detector t
__global__ void dw_sort_count_kernel(const int32_t *__restrict__ idx, int32_t *__restrict__ counts, int64_t batch,
                                     int n_detectors, int table_rows, int nblk) {
    const int t = blockIdx.x, k = blockIdx.y;
    const int64_t b0 = (int64_t)k * kSortBlock, b1 = min(batch, b0 + kSortBlock);
    for (int64_t b = b0 + threadIdx.x; b < b1; b += blockDim.x) {
        const int32_t r = __ldg(idx + b * n_detectors + t);
        atomicAdd(counts + ((size_t)t * table_rows + r) * nblk + k, 1);
    }
}

// exclusive scan over the flattened (row, block) counters of one detector; one block per detector
__global__ void dw_sort_scan_kernel(int32_t *__restrict__ counts, int table_rows, int nblk) {
    __shared__ int32_t partial[1024];
    __shared__ int32_t carry;
    int32_t *c = counts + (size_t)blockIdx.x * table_rows * nblk;
    const int64_t n = (int64_t)table_rows * nblk;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int64_t base = 0; base < n; base += blockDim.x) {
        const int64_t i = base + threadIdx.x;
        const int32_t v = i < n ? c[i] : 0;
        partial[threadIdx.x] = v;
        __syncthreads();
        for (int off = 1; off < (int)blockDim.x; off <<= 1) {  // Hillis-Steele inclusive scan
            int32_t add = threadIdx.x >= off ? partial[threadIdx.x - off] : 0;
            __syncthreads();
            partial[threadIdx.x] += add;
            __syncthreads();
        }
        if (i < n) c[i] = carry + partial[threadIdx.x] - v;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry += partial[threadIdx.x];
        __syncthreads();
    }
}

// stable scatter: one warp per (detector, block) walks its samples in order, 32 at a time
__global__ void dw_sort_scatter_kernel(const int32_t *__restrict__ idx, const int32_t *__restrict__ offsets,
                                       int32_t *__restrict__ perm, int64_t batch, int n_detectors, int table_rows,
                                       int nblk) {
    extern __shared__ int32_t cursor[];  // [table_rows] next free slot of each row for this (detector, block)
    const int t = blockIdx.x, k = blockIdx.y, lane = threadIdx.x;
    for (int r = lane; r < table_rows; r += 32) cursor[r] = __ldg(offsets + ((size_t)t * table_rows + r) * nblk + k);
    __syncwarp();
    const int64_t b0 = (int64_t)k * kSortBlock, b1 = min(batch, b0 + kSortBlock);
    int32_t *out = perm + (size_t)t * batch;
    for (int64_t base = b0; base < b1; base += 32) {
        const int64_t b = base + lane;
        const bool valid = b < b1;
        const int32_t r = valid ? __ldg(idx + b * n_detectors + t) : -1 - lane;  // invalid lanes match nobody
        const unsigned same = __match_any_sync(0xffffffffu, r);
        const int rank = __popc(same & ((1u << lane) - 1u));
        const int leader = __ffs(same) - 1;
        int32_t start = 0;
        if (valid && lane == leader) { start = cursor[r]; cursor[r] = start + __popc(same); }
        start = __shfl_sync(0xffffffffu, start, leader);
        if (valid) out[start + rank] = (int32_t)b;
        __syncwarp();
    }
}

// segmented reduce: one warp per (detector, row); samples of the segment in ascending order
__global__ void __launch_bounds__(256) dw_sort_reduce_kernel(const float *__restrict__ dY, const int32_t *__restrict__ offsets,
                                                            const int32_t *__restrict__ perm, float *__restrict__ target,
                                                            int64_t batch, int n_outputs, int n_detectors, int table_rows,
                                                            int nblk, double lr) {
    const int lane = threadIdx.x & 31;
    const int64_t seg = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (seg >= (int64_t)n_detectors * table_rows) return;
    const int t = (int)(seg / table_rows);
    const int32_t begin = __ldg(offsets + seg * nblk);
    const int32_t end = (seg % table_rows == table_rows - 1) ? (int32_t)batch : __ldg(offsets + (seg + 1) * nblk);
    if (begin == end) return;
    const int32_t *list = perm + (size_t)t * batch;
    float *row = target + seg * n_outputs;
    for (int o = lane; o < n_outputs; o += 32) {
        float acc = row[o];
        for (int32_t s = begin; s < end; s++) {
            const double g = (double)__ldg(dY + (size_t)__ldg(list + s) * n_outputs + o);
            if (fabs(g) > kEps) acc += (float)(g * lr);
        }
        row[o] = acc;
    }
}

size_t fc_dw_sorted_workspace(int64_t batch, int n_detectors, int table_rows) {
    const int64_t nblk = (batch + kSortBlock - 1) / kSortBlock;
    return ((size_t)n_detectors * table_rows * nblk + (size_t)n_detectors * batch) * sizeof(int32_t);
}

int launch_fc_dw_sorted(const float *dY, const int32_t *idx, float *target, int64_t batch, int n_outputs,
                        int n_detectors, int table_rows, double lr, void *workspace, cudaStream_t stream,
                        bool clear_with_memset) {
    const int64_t nblk64 = (batch + kSortBlock - 1) / kSortBlock;
    LUTB_REQUIRE(nblk64 <= 65535, LUTB_ERR_SHAPE, "batch too large for the sorted table-gradient variant");
    LUTB_REQUIRE((size_t)table_rows * 4 <= 200 * 1024, LUTB_ERR_SHAPE, "table too large for the sorted table-gradient variant");
    const int nblk = (int)nblk64;
    int32_t *counts = static_cast<int32_t *>(workspace);
    int32_t *perm = counts + (size_t)n_detectors * table_rows * nblk;
    const size_t count_bytes = (size_t)n_detectors * table_rows * nblk * sizeof(int32_t);
    if (clear_with_memset) LUTB_CUDA(cudaMemsetAsync(counts, 0, count_bytes, stream));
    dim3 grid((unsigned)n_detectors, (unsigned)nblk);
    KernelScope scope(K_FC_WEIGHT_GRAD, stream);
    dw_sort_count_kernel<<<grid, 256, 0, stream>>>(idx, counts, batch, n_detectors, table_rows, nblk);
    LUTB_LAUNCH_CHECK();
    dw_sort_scan_kernel<<<(unsigned)n_detectors, 1024, 0, stream>>>(counts, table_rows, nblk);
    LUTB_LAUNCH_CHECK();
    const size_t smem = (size_t)table_rows * sizeof(int32_t);
    if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(dw_sort_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dw_sort_scatter_kernel<<<grid, 32, smem, stream>>>(idx, counts, perm, batch, n_detectors, table_rows, nblk);
    LUTB_LAUNCH_CHECK();
    const int64_t segs = (int64_t)n_detectors * table_rows;
    dw_sort_reduce_kernel<<<(unsigned)((segs + 7) / 8), 256, 0, stream>>>(dY, counts, perm, target, batch, n_outputs,
                                                                        n_detectors, table_rows, nblk, lr);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

// ------------------------------------------------------------------------------------------
// Built-in scratch for callers that cannot allocate device memory.  The array lives in the library's
// device image: every GPU that loads the library holds it until the process exits.
// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the address a
// kernel may use is obtained per device with cudaGetSymbolAddress.
// ------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[LUTB_STATIC_SCRATCH_BYTES];

static std::mutex g_scratch_mutex;
static void *g_scratch_ptr[64] = {nullptr};

int static_scratch(void **ptr) {
    int dev = 0;
    LUTB_CUDA(cudaGetDevice(&dev));
    LUTB_REQUIRE(dev >= 0 && dev < 64, LUTB_ERR_SHAPE, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void *p = nullptr;
        LUTB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));  // resolved for the current device
        g_scratch_ptr[dev] = p;
    }
    *ptr = g_scratch_ptr[dev];
    return LUTB_OK;
}

}  // namespace lutb
