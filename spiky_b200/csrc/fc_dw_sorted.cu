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
// Table gradient as a list of touched rows (Sparse gradient policy): after the counting sort a segment
// (detector, row) with at least one sample is a touched row.  A block of 1024 threads looks at 1024 consecutive
// segments: the touched ones are counted (block totals -> exclusive scan by one block -> base of every block), each
// gets its position in the list from a block-wide scan of the flags, and the block's 32 warps reduce the touched
// segments one by one, writing the row number and the row of sums at that position.  Rows come out in ascending
// (detector, row) order; every cell is summed in ascending sample order like the dense sorted variant.
// ------------------------------------------------------------------------------------------
constexpr int kRowsBlock = 1024;

__device__ __forceinline__ bool segment_touched(const int32_t *offsets, int64_t seg, int table_rows, int nblk, int64_t batch,
                                                int32_t *begin, int32_t *end) {
    *begin = __ldg(offsets + seg * nblk);
    *end = (seg % table_rows == table_rows - 1) ? (int32_t)batch : __ldg(offsets + (seg + 1) * nblk);
    return *begin != *end;
}

__global__ void __launch_bounds__(kRowsBlock) dw_rows_count_kernel(const int32_t *__restrict__ offsets, int64_t n_seg,
                                                                  int table_rows, int nblk, int64_t batch,
                                                                  int32_t *__restrict__ block_sums) {
    const int64_t seg = (int64_t)blockIdx.x * kRowsBlock + threadIdx.x;
    int32_t b, e;
    const bool touched = seg < n_seg && segment_touched(offsets, seg, table_rows, nblk, batch, &b, &e);
    const int n = __syncthreads_count(touched);
    if (threadIdx.x == 0) block_sums[blockIdx.x] = n;
}

// exclusive scan of the block totals in place; the grand total goes to count_out
__global__ void __launch_bounds__(1024) dw_rows_scan_kernel(int32_t *__restrict__ block_sums, int64_t n_blocks,
                                                           int64_t *__restrict__ count_out) {
    __shared__ int32_t partial[1024];
    __shared__ int64_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int64_t base = 0; base < n_blocks; base += 1024) {
        const int64_t i = base + threadIdx.x;
        const int32_t v = i < n_blocks ? block_sums[i] : 0;
        partial[threadIdx.x] = v;
        __syncthreads();
        for (int off = 1; off < 1024; off <<= 1) {
            const int32_t add = threadIdx.x >= off ? partial[threadIdx.x - off] : 0;
            __syncthreads();
            partial[threadIdx.x] += add;
            __syncthreads();
        }
        if (i < n_blocks) block_sums[i] = (int32_t)carry + partial[threadIdx.x] - v;
        __syncthreads();
        if (threadIdx.x == 1023) carry += partial[1023];
        __syncthreads();
    }
    if (threadIdx.x == 0) *count_out = carry;
}

__global__ void __launch_bounds__(kRowsBlock) dw_rows_emit_kernel(const float *__restrict__ dY, const int32_t *__restrict__ offsets,
                                                                 const int32_t *__restrict__ perm,
                                                                 const int32_t *__restrict__ block_base, int64_t n_seg,
                                                                 int64_t batch, int n_outputs, int table_rows, int nblk,
                                                                 double lr, int64_t capacity, int64_t *__restrict__ row_ids,
                                                                 float *__restrict__ values) {
    __shared__ int32_t warp_sums[32];
    __shared__ int32_t position[kRowsBlock];   // list position of a touched segment, -1 otherwise
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t seg0 = (int64_t)blockIdx.x * kRowsBlock;
    const int64_t seg = seg0 + threadIdx.x;
    int32_t b, e;
    const bool touched = seg < n_seg && segment_touched(offsets, seg, table_rows, nblk, batch, &b, &e);
    const unsigned mask = __ballot_sync(0xffffffffu, touched);
    if (lane == 0) warp_sums[warp] = __popc(mask);
    __syncthreads();
    int32_t before = __ldg(block_base + blockIdx.x);
    for (int w = 0; w < warp; w++) before += warp_sums[w];
    position[threadIdx.x] = touched ? before + __popc(mask & ((1u << lane) - 1u)) : -1;
    __syncthreads();
    for (int i = warp; i < kRowsBlock; i += 32) {
        const int32_t pos = position[i];
        if (pos < 0 || pos >= capacity) continue;   // warp-uniform
        const int64_t sg = seg0 + i;
        int32_t begin, end;
        segment_touched(offsets, sg, table_rows, nblk, batch, &begin, &end);
        const int32_t *list = perm + (size_t)(sg / table_rows) * batch;
        if (lane == 0) row_ids[pos] = sg;
        float *row = values + (size_t)pos * n_outputs;
        for (int o = lane; o < n_outputs; o += 32) {
            float acc = 0.f;
            for (int32_t s = begin; s < end; s++) {
                const double g = (double)__ldg(dY + (size_t)__ldg(list + s) * n_outputs + o);
                if (fabs(g) > kEps) acc += (float)(g * lr);
            }
            row[o] = acc;
        }
    }
}

size_t fc_dw_rows_workspace(int64_t batch, int n_detectors, int table_rows) {
    const int64_t n_blocks = ((int64_t)n_detectors * table_rows + kRowsBlock - 1) / kRowsBlock;
    const size_t sorted = (fc_dw_sorted_workspace(batch, n_detectors, table_rows) + 15) & ~(size_t)15;
    return sorted + (size_t)n_blocks * sizeof(int32_t);
}

int launch_fc_dw_rows(const float *dY, const int32_t *idx, int64_t batch, int n_outputs, int n_detectors, int table_rows,
                      double lr, int64_t *row_ids, float *values, int64_t capacity, int64_t *count_out, void *workspace,
                      cudaStream_t stream) {
    const int64_t nblk64 = (batch + kSortBlock - 1) / kSortBlock;
    LUTB_REQUIRE(nblk64 <= 65535, LUTB_ERR_SHAPE, "batch too large for the sorted table-gradient variant");
    LUTB_REQUIRE((size_t)table_rows * 4 <= 200 * 1024, LUTB_ERR_SHAPE, "table too large for the sorted table-gradient variant");
    const int nblk = (int)nblk64;
    int32_t *counts = static_cast<int32_t *>(workspace);
    int32_t *perm = counts + (size_t)n_detectors * table_rows * nblk;
    const size_t sorted = (fc_dw_sorted_workspace(batch, n_detectors, table_rows) + 15) & ~(size_t)15;
    int32_t *block_sums = reinterpret_cast<int32_t *>(static_cast<unsigned char *>(workspace) + sorted);
    LUTB_CUDA(cudaMemsetAsync(counts, 0, (size_t)n_detectors * table_rows * nblk * sizeof(int32_t), stream));
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
    const int64_t n_seg = (int64_t)n_detectors * table_rows;
    const int64_t n_blocks = (n_seg + kRowsBlock - 1) / kRowsBlock;
    LUTB_REQUIRE(n_blocks <= 0x7FFFFFFF, LUTB_ERR_SHAPE, "too many table rows for one launch");
    dw_rows_count_kernel<<<(unsigned)n_blocks, kRowsBlock, 0, stream>>>(counts, n_seg, table_rows, nblk, batch, block_sums);
    LUTB_LAUNCH_CHECK();
    dw_rows_scan_kernel<<<1, 1024, 0, stream>>>(block_sums, n_blocks, count_out);
    LUTB_LAUNCH_CHECK();
    dw_rows_emit_kernel<<<(unsigned)n_blocks, kRowsBlock, 0, stream>>>(dY, counts, perm, block_sums, n_seg, batch, n_outputs,
                                                                    table_rows, nblk, lr, capacity, row_ids, values);
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
