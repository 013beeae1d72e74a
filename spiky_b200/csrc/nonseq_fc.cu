// Non-sequence, fully connected LUT layer: anchor comparison + bit packing, table-row gather and
// accumulate, surrogate input gradient and table-gradient scatter.  sm_100a, no tensor cores: the
// path is gather/scatter bound.
#include "lutb_common.cuh"
#include "nonseq_fc.cuh"
#include "fc_dw_sorted.cuh"

namespace lutb {

// --------------------------------------------------------------------------------------------
// Kernel 1: anchor-pair comparison and bit packing.
//
// A block stages `GROUPS * R` input rows in shared memory, transposed to [input][row] so that one
// 128-bit shared load returns the same input of four rows.  Each thread owns one detector, walks its
// anchor pairs once and evaluates all R rows of its group from registers.  Per (row, detector) it
// emits the packed table index and, for training, the first anchor pair of minimal |delta| with its
// signed delta (reference: check_detectors[_eval]_logic, lut_runtime_kernels_logic.proto:1050-1158).
// --------------------------------------------------------------------------------------------
// 16-byte slots of the transposed staging area are XOR-swizzled with the 8-slot row they lie in: neighbouring
// lanes stage inputs 4 apart (slots 4 * R / 4 apart), which without the swizzle all fall into the same banks.
__device__ __forceinline__ int swizzle_slot(int slot) { return slot ^ ((slot >> 3) & 7); }
// floats of one row group's staging area (whole 8-slot rows, so a swizzled slot never leaves the area)
template <int R>
__host__ __device__ constexpr size_t staged_floats(int n_inputs) {
    return R % 4 == 0 ? ((((size_t)n_inputs * (R / 4)) + 7) & ~(size_t)7) * 4 : (size_t)R * n_inputs;
}

// Stages the R rows [row0, row0 + nrows) of one row group: coalesced global reads, transposed shared writes.
template <int R>
__device__ __forceinline__ void stage_rows(float *xs, const float *__restrict__ x, int64_t row0, int nrows, int n_inputs,
                                           int lt, int threads_per_group, bool vec_ok) {
    if (vec_ok) {
        const int n4 = n_inputs >> 2;
        for (int i4 = lt; i4 < n4; i4 += threads_per_group) {
            float v[R][4];
#pragma unroll
            for (int r = 0; r < R; r++) {
                float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r < nrows) q = __ldcs(reinterpret_cast<const float4 *>(x + (row0 + r) * n_inputs) + i4);
                v[r][0] = q.x; v[r][1] = q.y; v[r][2] = q.z; v[r][3] = q.w;
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float *dst = xs + (size_t)(4 * i4 + j) * R;
                if constexpr (R % 4 == 0) {
#pragma unroll
                    for (int r4 = 0; r4 < R / 4; r4++)
                        reinterpret_cast<float4 *>(xs)[swizzle_slot((4 * i4 + j) * (R / 4) + r4)] =
                            make_float4(v[4 * r4][j], v[4 * r4 + 1][j], v[4 * r4 + 2][j], v[4 * r4 + 3][j]);
                } else {
#pragma unroll
                    for (int r = 0; r < R; r++) dst[r] = v[r][j];
                }
            }
        }
    } else {
        for (int i = lt; i < n_inputs; i += threads_per_group) {
#pragma unroll
            for (int r = 0; r < R; r++) {
                const float v = (r < nrows) ? __ldcs(x + (row0 + r) * n_inputs + i) : 0.f;
                if constexpr (R % 4 == 0) xs[swizzle_slot(i * (R / 4) + (r >> 2)) * 4 + (r & 3)] = v;
                else xs[(size_t)i * R + r] = v;
            }
        }
    }
}

// Work items: (row tile of GROUPS * R rows, chunk of threads_per_group detectors), row tile major.  Block b takes the
// items [n * b / grid, n * (b + 1) / grid): with a grid of one block per row tile that is the tile's own chunks; small
// batches launch a multiple of the SM count instead and a block's range may cross into the next tile, which it then
// stages as well.  (Splitting the detectors into a fixed number of slices per tile left 320 blocks on 148 SMs: the SMs
// with three blocks set the kernel's time, max / avg active cycles 1.3.)
template <int R, bool TRAIN>
__global__ void __launch_bounds__(256) check_detectors_kernel(const float *__restrict__ x, int64_t rows, int n_inputs,
                                                             const int2 *__restrict__ anchors, int n_detectors,
                                                             int n_anchors, float cmp_eps, int threads_per_group,
                                                             int32_t *__restrict__ idx,
                                                             float *__restrict__ min_delta,
                                                             int32_t *__restrict__ min_k) {
    extern __shared__ __align__(16) float xs_all[];
    const int groups = blockDim.x / threads_per_group;
    const int g = threadIdx.x / threads_per_group;
    const int lt = threadIdx.x - g * threads_per_group;
    float *xs = xs_all + (size_t)g * staged_floats<R>(n_inputs);
    const bool vec_ok = (n_inputs % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const int chunks = (n_detectors + threads_per_group - 1) / threads_per_group;
    const int64_t rows_per_tile = (int64_t)groups * R;
    const int64_t n_items = ((rows + rows_per_tile - 1) / rows_per_tile) * chunks;
    const int64_t item0 = n_items * blockIdx.x / gridDim.x, item1 = n_items * (blockIdx.x + 1) / gridDim.x;
    int64_t staged = -1;
    for (int64_t item = item0; item < item1; ++item) {
        const int64_t tile = item / chunks;
        const int chunk = (int)(item - tile * chunks);
        const int64_t row0 = (tile * groups + g) * R;
        const int nrows = (int)min((int64_t)R, max((int64_t)0, rows - row0));
        if (tile != staged) {
            if (staged >= 0) __syncthreads();   // everyone is done reading the previous tile
            stage_rows<R>(xs, x, row0, nrows, n_inputs, lt, threads_per_group, vec_ok);
            __syncthreads();
            staged = tile;
        }
        const int t = chunk * threads_per_group + lt;
        if (nrows <= 0 || t >= n_detectors) continue;
        int32_t li[R];
        float md[R];
        int32_t mk[R];
#pragma unroll
        for (int r = 0; r < R; r++) { li[r] = 0; md[r] = 0.f; mk[r] = -1; }
        const int2 *ap = anchors + (size_t)t * n_anchors;
#pragma unroll 4
        for (int k = 0; k < n_anchors; k++) {
            const int2 p = __ldg(ap + k);
            if (p.x == kNoAnchor || p.y == kNoAnchor) continue;
            float a[R], b[R];
            if constexpr (R % 4 == 0) {
#pragma unroll
                for (int r4 = 0; r4 < R / 4; r4++) {
                    const float4 qa = reinterpret_cast<const float4 *>(xs)[swizzle_slot(p.x * (R / 4) + r4)];
                    const float4 qb = reinterpret_cast<const float4 *>(xs)[swizzle_slot(p.y * (R / 4) + r4)];
                    a[4 * r4] = qa.x; a[4 * r4 + 1] = qa.y; a[4 * r4 + 2] = qa.z; a[4 * r4 + 3] = qa.w;
                    b[4 * r4] = qb.x; b[4 * r4 + 1] = qb.y; b[4 * r4 + 2] = qb.z; b[4 * r4 + 3] = qb.w;
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; r++) { a[r] = xs[(size_t)p.x * R + r]; b[r] = xs[(size_t)p.y * R + r]; }
            }
#pragma unroll
            for (int r = 0; r < R; r++) {
                const float d = __fsub_rn(a[r], b[r]);
                if (greater_than_zero(d, cmp_eps)) li[r] |= (1 << k);
                if (TRAIN) {
                    if (mk[r] == -1 || fabsf(d) < fabsf(md[r])) { md[r] = d; mk[r] = k; }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            if (r < nrows) {
                const int64_t o = (row0 + r) * n_detectors + t;
                idx[o] = li[r];
                if (TRAIN) { min_delta[o] = md[r]; min_k[o] = mk[r]; }
            }
        }
    }
}

// Fallback for input rows that do not fit in shared memory: gathers straight from global memory.
template <bool TRAIN>
__global__ void check_detectors_global_kernel(const float *__restrict__ x, int64_t rows, int n_inputs,
                                              const int2 *__restrict__ anchors, int n_detectors, int n_anchors,
                                              float cmp_eps, int32_t *__restrict__ idx, float *__restrict__ min_delta,
                                              int32_t *__restrict__ min_k) {
    const int64_t total = rows * n_detectors;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / n_detectors;
        const int t = (int)(i - r * n_detectors);
        const float *xr = x + r * n_inputs;
        int32_t li = 0, mk = -1;
        float md = 0.f;
        for (int k = 0; k < n_anchors; k++) {
            const int2 p = __ldg(anchors + (size_t)t * n_anchors + k);
            if (p.x == kNoAnchor || p.y == kNoAnchor) continue;
            const float d = __fsub_rn(__ldg(xr + p.x), __ldg(xr + p.y));
            if (greater_than_zero(d, cmp_eps)) li |= (1 << k);
            if (TRAIN) {
                if (mk == -1 || fabsf(d) < fabsf(md)) { md = d; mk = k; }
            }
        }
        idx[i] = li;
        if (TRAIN) { min_delta[i] = md; min_k[i] = mk; }
    }
}

template <int R>
static int launch_check_detectors_r(const float *x, int64_t rows, int n_inputs, const int32_t *anchors,
                                    int n_detectors, int n_anchors, float cmp_eps, int32_t *idx, float *min_delta,
                                    int32_t *min_k, int tpg, int groups, int64_t blocks, cudaStream_t stream) {
    const size_t smem = (size_t)groups * staged_floats<R>(n_inputs) * sizeof(float);
    LUTB_REQUIRE(blocks <= 0x7FFFFFFF, LUTB_ERR_SHAPE, "batch too large for one launch");
    const bool train = min_delta != nullptr;
    auto kern = train ? check_detectors_kernel<R, true> : check_detectors_kernel<R, false>;
    if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    KernelScope scope(K_CHECK_DETECTORS, stream);
    kern<<<(unsigned)blocks, tpg * groups, smem, stream>>>(x, rows, n_inputs, reinterpret_cast<const int2 *>(anchors),
                                                          n_detectors, n_anchors, cmp_eps, tpg, idx, min_delta, min_k);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

int launch_check_detectors(const float *x, int64_t rows, int n_inputs, const int32_t *anchors, int n_detectors,
                           int n_anchors, float cmp_eps, int32_t *idx, float *min_delta, int32_t *min_k,
                           cudaStream_t stream) {
    const int sm = device_info().sm_count;
    // threads per row group: one per detector, rounded to warps, at most 256
    int tpg = ((min(n_detectors, 256) + 31) / 32) * 32;
    // rows per group: up to 8 (each anchor pair is fetched once per 8 rows), fewer when rows are long
    const size_t row_bytes = (size_t)n_inputs * sizeof(float);
    const size_t budget = 100 * 1024;  // two resident blocks per SM
    int R = 8;
    while (R > 1 && ((size_t)R * row_bytes > budget || rows < R)) R >>= 1;
    if ((size_t)R * row_bytes > (size_t)kMaxSmemPerBlock - 1024) {
        const bool train = min_delta != nullptr;
        const int64_t total = rows * n_detectors;
        int64_t blocks = min((total + 255) / 256, (int64_t)sm * 32);
        KernelScope scope(K_CHECK_DETECTORS, stream);
        if (train)
            check_detectors_global_kernel<true><<<(unsigned)blocks, 256, 0, stream>>>(
                x, rows, n_inputs, reinterpret_cast<const int2 *>(anchors), n_detectors, n_anchors, cmp_eps, idx,
                min_delta, min_k);
        else
            check_detectors_global_kernel<false><<<(unsigned)blocks, 256, 0, stream>>>(
                x, rows, n_inputs, reinterpret_cast<const int2 *>(anchors), n_detectors, n_anchors, cmp_eps, idx,
                min_delta, min_k);
        LUTB_LAUNCH_CHECK();
        return LUTB_OK;
    }
    int groups = 256 / tpg;
    while (groups > 1 && ((size_t)groups * R * row_bytes > budget || rows < (int64_t)groups * R * 2 * sm)) groups >>= 1;
    // one block per row tile; small batches: two blocks per SM, each with an equal share of the (tile, detector chunk)
    // work items
    const int64_t row_tiles = (rows + (int64_t)groups * R - 1) / ((int64_t)groups * R);
    const int64_t items = row_tiles * ((n_detectors + tpg - 1) / tpg);
    const int64_t blocks = row_tiles >= (int64_t)2 * sm ? row_tiles : min(items, (int64_t)2 * sm);
    switch (R) {
        case 8: return launch_check_detectors_r<8>(x, rows, n_inputs, anchors, n_detectors, n_anchors, cmp_eps, idx, min_delta, min_k, tpg, groups, blocks, stream);
        case 4: return launch_check_detectors_r<4>(x, rows, n_inputs, anchors, n_detectors, n_anchors, cmp_eps, idx, min_delta, min_k, tpg, groups, blocks, stream);
        case 2: return launch_check_detectors_r<2>(x, rows, n_inputs, anchors, n_detectors, n_anchors, cmp_eps, idx, min_delta, min_k, tpg, groups, blocks, stream);
        default: return launch_check_detectors_r<1>(x, rows, n_inputs, anchors, n_detectors, n_anchors, cmp_eps, idx, min_delta, min_k, tpg, groups, blocks, stream);
    }
}

// --------------------------------------------------------------------------------------------
// Kernel 2: table-row gather and accumulate, y[b, :] += sum_t W[t, idx[b, t], :]
// (reference: fill_outputs_non_seq_fc_logic, proto:1214-1299).
//
// One warp per (sample, output chunk).  The warp is split into NG lane groups of LG lanes; a group
// owns every NG-th detector and its lanes cover the chunk's columns VEC floats at a time, so a row
// read is one coalesced 16*LG byte segment.  Table indices are fetched 32 at a time (coalesced)
// and broadcast with shuffles, so the row loads do not wait on a dependent index load.  Partial
// sums are fp32 inside a block of 32 detectors and double across blocks.
//
// Fixed-point mode reproduces the reference bit for bit: detectors are summed in double in order,
// in blocks of `det_block` (backward_group_size), each block sum is truncated to int32 and added.
// --------------------------------------------------------------------------------------------
constexpr int kFwdJ = 4;  // vectors per lane and chunk

template <int VEC>
struct Vec;
template <>
struct Vec<4> {
    using T = float4;
    static __device__ __forceinline__ void load(const float *p, float (&v)[4]) {
        const float4 q = __ldg(reinterpret_cast<const float4 *>(p));
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
};
template <>
struct Vec<1> {
    using T = float;
    static __device__ __forceinline__ void load(const float *p, float (&v)[1]) { v[0] = __ldg(p); }
};

template <int VEC, bool INT_MODE>
__global__ void __launch_bounds__(256) fc_gather_forward_kernel(const float *__restrict__ W, const int32_t *__restrict__ idx,
                                                               float *__restrict__ y, int64_t batch, int n_outputs,
                                                               int n_detectors, int table_rows, int t0, int t1,
                                                               int det_block, int lanes_per_row, int chunk,
                                                               double fixed_scale) {
    const int lane = threadIdx.x & 31;
    const int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= batch) return;
    const int c0 = blockIdx.y * chunk;
    const int clen = min(chunk, n_outputs - c0);
    const int LG = INT_MODE ? 32 : lanes_per_row;
    const int NG = 32 / LG;
    const int g = lane / LG;
    const int j = lane - g * LG;
    const int32_t *idx_b = idx + b * n_detectors;
    const size_t row_stride = (size_t)n_outputs;

    if constexpr (!INT_MODE) {
        double acc[kFwdJ][VEC];
#pragma unroll
        for (int q = 0; q < kFwdJ; q++)
#pragma unroll
            for (int e = 0; e < VEC; e++) acc[q][e] = 0.0;
        for (int tb = t0; tb < t1; tb += 32) {
            const int nvalid = min(32, t1 - tb);
            const int32_t mine = (lane < nvalid) ? __ldg(idx_b + tb + lane) : 0;
            float part[kFwdJ][VEC];
#pragma unroll
            for (int q = 0; q < kFwdJ; q++)
#pragma unroll
                for (int e = 0; e < VEC; e++) part[q][e] = 0.f;
#pragma unroll 4
            for (int sb = 0; sb < nvalid; sb += NG) {
                const int s = sb + g;
                const int32_t li = __shfl_sync(0xffffffffu, mine, s & 31);
                if (s < nvalid) {
                    const float *row = W + ((size_t)(tb + s) * table_rows + li) * row_stride + c0;
#pragma unroll
                    for (int q = 0; q < kFwdJ; q++) {
                        const int col = (j + q * LG) * VEC;
                        if (col < clen) {
                            float v[VEC];
                            Vec<VEC>::load(row + col, v);
#pragma unroll
                            for (int e = 0; e < VEC; e++) part[q][e] += v[e];
                        }
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < kFwdJ; q++)
#pragma unroll
                for (int e = 0; e < VEC; e++) acc[q][e] += (double)part[q][e];
        }
        for (int off = LG; off < 32; off <<= 1) {
#pragma unroll
            for (int q = 0; q < kFwdJ; q++)
#pragma unroll
                for (int e = 0; e < VEC; e++) acc[q][e] += __shfl_xor_sync(0xffffffffu, acc[q][e], off);
        }
        if (g == 0) {
            float *yb = y + b * n_outputs + c0;
#pragma unroll
            for (int q = 0; q < kFwdJ; q++) {
                const int col = (j + q * LG) * VEC;
                if (col < clen) {
                    if constexpr (VEC == 4) {
                        float4 cur = *reinterpret_cast<float4 *>(yb + col);
                        cur.x += (float)acc[q][0]; cur.y += (float)acc[q][1];
                        cur.z += (float)acc[q][2]; cur.w += (float)acc[q][3];
                        *reinterpret_cast<float4 *>(yb + col) = cur;
                    } else {
                        yb[col] += (float)acc[q][0];
                    }
                }
            }
        }
    } else {
        int32_t iacc[kFwdJ][VEC];
#pragma unroll
        for (int q = 0; q < kFwdJ; q++)
#pragma unroll
            for (int e = 0; e < VEC; e++) iacc[q][e] = 0;
        for (int tb = t0; tb < t1; tb += det_block) {
            const int tend = min(tb + det_block, t1);
            double s[kFwdJ][VEC];
#pragma unroll
            for (int q = 0; q < kFwdJ; q++)
#pragma unroll
                for (int e = 0; e < VEC; e++) s[q][e] = 0.0;
            for (int t = tb; t < tend; t++) {
                const int32_t li = __ldg(idx_b + t);
                const float *row = W + ((size_t)t * table_rows + li) * row_stride + c0;
#pragma unroll
                for (int q = 0; q < kFwdJ; q++) {
                    const int col = (j + q * LG) * VEC;
                    if (col < clen) {
                        float v[VEC];
                        Vec<VEC>::load(row + col, v);
#pragma unroll
                        for (int e = 0; e < VEC; e++) s[q][e] += (double)v[e];
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < kFwdJ; q++)
#pragma unroll
                for (int e = 0; e < VEC; e++) iacc[q][e] += to_fixed(s[q][e], fixed_scale);
        }
        int32_t *yb = reinterpret_cast<int32_t *>(y) + b * n_outputs + c0;
#pragma unroll
        for (int q = 0; q < kFwdJ; q++) {
            const int col = (j + q * LG) * VEC;
            if (col < clen) {
#pragma unroll
                for (int e = 0; e < VEC; e++) yb[col + e] += iacc[q][e];
            }
        }
    }
}

// Fast path of the forward gather for fp32 accumulators and 16-byte aligned rows: one warp per (sample,
// chunk of LG float4 columns); the row loads of up to 16 detectors per lane are all issued before the first
// one is consumed, which is what hides the latency of the (random) row reads.
template <int LG>
__global__ void __launch_bounds__(256) fc_gather_forward_vec_kernel(const float *__restrict__ W,
                                                                   const int32_t *__restrict__ idx,
                                                                   float *__restrict__ y, int64_t batch, int n_outputs,
                                                                   int n_detectors, int table_rows, int t0, int t1) {
    constexpr int NG = 32 / LG;
    constexpr int IT = 32 / NG;                  // row loads per lane and 32 detectors
    constexpr int BATCH = IT > 16 ? 16 : IT;     // loads in flight per lane
    const int lane = threadIdx.x & 31;
    const int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= batch) return;
    const int g = lane / LG, j = lane - g * LG;
    const int col = (blockIdx.y * LG + j) * 4;
    const bool active = col < n_outputs;
    const int32_t *idx_b = idx + b * n_detectors;
    const float *Wc = W + col;
    double acc[4] = {0.0, 0.0, 0.0, 0.0};
    for (int tb = t0; tb < t1; tb += 32) {
        const int nvalid = min(32, t1 - tb);
        const int32_t mine = (lane < nvalid) ? __ldg(idx_b + tb + lane) : 0;
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i0 = 0; i0 < IT; i0 += BATCH) {
            float4 w[BATCH];
#pragma unroll
            for (int i = 0; i < BATCH; i++) {
                const int d = (i0 + i) * NG + g;
                const int32_t li = __shfl_sync(0xffffffffu, mine, d);
                w[i] = (active && d < nvalid)
                           ? __ldg(reinterpret_cast<const float4 *>(Wc + ((size_t)(tb + d) * table_rows + li) * n_outputs))
                           : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < BATCH; i++) { part[0] += w[i].x; part[1] += w[i].y; part[2] += w[i].z; part[3] += w[i].w; }
        }
#pragma unroll
        for (int e = 0; e < 4; e++) acc[e] += (double)part[e];
    }
#pragma unroll
    for (int m = LG; m < 32; m <<= 1) {
#pragma unroll
        for (int e = 0; e < 4; e++) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], m);
    }
    if (active && g == 0) {
        float4 *out = reinterpret_cast<float4 *>(y + b * n_outputs + col);
        float4 cur = *out;
        cur.x += (float)acc[0]; cur.y += (float)acc[1]; cur.z += (float)acc[2]; cur.w += (float)acc[3];
        *out = cur;
    }
}

static int pow2_ceil(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

int launch_fc_gather_forward(const float *W, const int32_t *idx, float *y, int64_t batch, int n_outputs,
                             int n_detectors, int table_rows, int det_block, bool int_mode, double fixed_scale,
                             cudaStream_t stream) {
    const bool vec4 = (n_outputs % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
    const int vec = vec4 ? 4 : 1;
    const int vpr = (n_outputs + vec - 1) / vec;  // vectors per row
    const int lanes = int_mode ? 32 : min(32, pow2_ceil(vpr));
    const int chunk = min(n_outputs, lanes * kFwdJ * vec);
    const int n_chunks = (n_outputs + chunk - 1) / chunk;
    const int warps = 8;
    const int64_t blocks = (batch + warps - 1) / warps;
    LUTB_REQUIRE(blocks <= 0x7FFFFFFF && n_chunks <= 65535, LUTB_ERR_SHAPE, "grid too large");
    // Detector ranges are sized so that one range's tables stay resident in L2 while the whole batch
    // streams through them; fixed-point blocks must not straddle a range.
    const size_t table_bytes = (size_t)table_rows * n_outputs * sizeof(float);
    int64_t per_range = (int64_t)((size_t)(48u << 20) / (table_bytes ? table_bytes : 1));
    const int align = int_mode ? det_block : 32;
    per_range = max((int64_t)align, per_range / align * align);
    dim3 grid((unsigned)blocks, (unsigned)n_chunks);
    for (int64_t t0 = 0; t0 < n_detectors; t0 += per_range) {
        const int t1 = (int)min((int64_t)n_detectors, t0 + per_range);
        KernelScope scope(K_FC_GATHER_FORWARD, stream);
        if (vec4 && !int_mode) {
            const dim3 vgrid((unsigned)blocks, (unsigned)((vpr + lanes - 1) / lanes));
#define LUTB_FWD(LGV) fc_gather_forward_vec_kernel<LGV><<<vgrid, warps * 32, 0, stream>>>(W, idx, y, batch, n_outputs, n_detectors, table_rows, (int)t0, t1)
            switch (lanes) {
                case 32: LUTB_FWD(32); break;
                case 16: LUTB_FWD(16); break;
                case 8: LUTB_FWD(8); break;
                case 4: LUTB_FWD(4); break;
                case 2: LUTB_FWD(2); break;
                default: LUTB_FWD(1); break;
            }
#undef LUTB_FWD
        } else if (vec4) {
            if (int_mode)
                fc_gather_forward_kernel<4, true><<<grid, warps * 32, 0, stream>>>(W, idx, y, batch, n_outputs, n_detectors, table_rows, (int)t0, t1, det_block, lanes, chunk, fixed_scale);
            else
                fc_gather_forward_kernel<4, false><<<grid, warps * 32, 0, stream>>>(W, idx, y, batch, n_outputs, n_detectors, table_rows, (int)t0, t1, det_block, lanes, chunk, fixed_scale);
        } else {
            if (int_mode)
                fc_gather_forward_kernel<1, true><<<grid, warps * 32, 0, stream>>>(W, idx, y, batch, n_outputs, n_detectors, table_rows, (int)t0, t1, det_block, lanes, chunk, fixed_scale);
            else
                fc_gather_forward_kernel<1, false><<<grid, warps * 32, 0, stream>>>(W, idx, y, batch, n_outputs, n_detectors, table_rows, (int)t0, t1, det_block, lanes, chunk, fixed_scale);
        }
        LUTB_LAUNCH_CHECK();
    }
    return LUTB_OK;
}

// --------------------------------------------------------------------------------------------
// Kernel 3: surrogate input gradient (reference: propagate_through_detectors_non_seq_fc_logic,
// proto:1421-1499).  Per (sample, detector): g = sum_o dY[o] * (W[t, j, o] - W[t, j ^ 2^k, o]),
// du = up(min_delta) * g, then +du / -du on the two inputs of the flipped anchor pair.
// Same warp layout as the forward gather; both rows are read with coalesced vector loads.  The products of one
// vector are summed in fp32 and added to a double per lane (converting every operand to double kept the
// conversion unit busy: three conversions per element), the lane groups are reduced in double, and the dot
// products of 32 detectors are parked in shared memory so that the surrogate derivative (a double division) and
// the two reductions into dX run once per detector on 32 lanes instead of once per lane group on one lane in LG.
// --------------------------------------------------------------------------------------------
template <int VEC>
__global__ void __launch_bounds__(256) fc_input_grad_kernel(const float *__restrict__ W, const float *__restrict__ dY,
                                                           const int2 *__restrict__ anchors,
                                                           const int32_t *__restrict__ idx,
                                                           const float *__restrict__ min_delta,
                                                           const int32_t *__restrict__ min_k, float *__restrict__ dX,
                                                           int64_t batch, int n_inputs, int n_outputs, int n_detectors,
                                                           int n_anchors, int table_rows, int lanes_per_row) {
    __shared__ double dots[8][32];
    const int lane = threadIdx.x & 31;
    const int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= batch) return;
    double *my_dots = dots[(threadIdx.x >> 5) & 7];
    const int LG = lanes_per_row;
    const int NG = 32 / LG;
    const int g = lane / LG;
    const int j = lane - g * LG;
    const float *dy = dY + b * n_outputs;
    float *dx = dX + b * n_inputs;
    const int64_t base = b * n_detectors;
    const int step = LG * VEC;

    for (int tb = 0; tb < n_detectors; tb += 32) {
        const int nvalid = min(32, n_detectors - tb);
        int32_t my_idx = 0, my_k = -1;
        float my_m = 0.f;
        if (lane < nvalid) {
            my_idx = __ldg(idx + base + tb + lane);
            my_k = __ldg(min_k + base + tb + lane);
            my_m = __ldg(min_delta + base + tb + lane);
        }
        for (int sb = 0; sb < nvalid; sb += NG) {   // uniform trip count: every lane runs every shuffle
            const int s = sb + g;
            const int32_t li = __shfl_sync(0xffffffffu, my_idx, s & 31);
            const int32_t k = __shfl_sync(0xffffffffu, my_k, s & 31);
            double acc = 0.0;
            const bool valid = s < nvalid && k >= 0;
            if (valid) {
                const int t = tb + s;
                const float *row = W + ((size_t)t * table_rows + li) * n_outputs;
                const float *alt = W + ((size_t)t * table_rows + (li ^ (1 << k))) * n_outputs;
                for (int col = j * VEC; col < n_outputs; col += step) {
                    float a[VEC], c[VEC], d[VEC];
                    Vec<VEC>::load(row + col, a);
                    Vec<VEC>::load(alt + col, c);
                    Vec<VEC>::load(dy + col, d);
                    float part = 0.f;
#pragma unroll
                    for (int e = 0; e < VEC; e++) part = fmaf(d[e], a[e] - c[e], part);
                    acc += (double)part;
                }
            }
            for (int off = 1; off < LG; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (s < nvalid && j == 0) my_dots[s] = acc;
        }
        __syncwarp();
        if (lane < nvalid && my_k >= 0) {
            const double du = surrogate_up(my_m) * my_dots[lane];
            if (fabs(du) > kEps) {
                const int2 p = __ldg(anchors + (size_t)(tb + lane) * n_anchors + my_k);
                atomicAdd(dx + p.x, (float)du);
                atomicAdd(dx + p.y, -(float)du);
            }
        }
        __syncwarp();
    }
}

// Fixed-point variant: one thread per (sample, detector), outputs walked in order in blocks of
// `out_block` (forward_group_size); each block's du is truncated to int32 on its own, exactly as
// the reference does, and added with integer atomics (order independent).
__global__ void fc_input_grad_fixed_kernel(const float *__restrict__ W, const float *__restrict__ dY,
                                           const int2 *__restrict__ anchors, const int32_t *__restrict__ idx,
                                           const float *__restrict__ min_delta, const int32_t *__restrict__ min_k,
                                           float *__restrict__ dX, int64_t batch, int n_inputs, int n_outputs,
                                           int n_detectors, int n_anchors, int table_rows, int out_block,
                                           double fixed_scale) {
    const int64_t total = batch * n_detectors;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / n_detectors;
        const int t = (int)(i - b * n_detectors);
        const int32_t li = idx[i];
        const int32_t k = min_k[i];
        const double up = surrogate_up(min_delta[i]);
        const float *row = W + ((size_t)t * table_rows + li) * n_outputs;
        const float *alt = W + ((size_t)t * table_rows + (li ^ (1 << k))) * n_outputs;
        const float *dy = dY + b * n_outputs;
        const int2 p = __ldg(anchors + (size_t)t * n_anchors + k);
        int32_t *dx = reinterpret_cast<int32_t *>(dX) + b * n_inputs;
        for (int o0 = 0; o0 < n_outputs; o0 += out_block) {
            const int o1 = min(o0 + out_block, n_outputs);
            double ms = 0.0, as = 0.0;
            for (int o = o0; o < o1; o++) {
                const double gdy = (double)__ldg(dy + o);
                ms += (double)__ldg(row + o) * gdy;
                as += (double)__ldg(alt + o) * gdy;
            }
            const double du = up * (ms - as);
            if (fabs(du) > kEps) {
                const int32_t d = to_fixed(du, fixed_scale);
                atomicAdd(dx + p.x, d);
                atomicAdd(dx + p.y, -d);
            }
        }
    }
}

// --------------------------------------------------------------------------------------------
// Kernel 4a: table-gradient scatter with row-coalesced global reductions
// (reference: gather_w_gradients_non_seq_fc_logic, proto:1547-1585, helper :716-819):
// target[t, idx[b, t], :] += lr * dY[b, :] for |dY| > EPS.  `target` is dW, or W itself for the
// internal (in-place SGD) policy with lr = -external_lr * lr_meta.
// --------------------------------------------------------------------------------------------
__device__ __forceinline__ void red_add_v4(float *addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int VEC, bool INT_MODE>
__global__ void __launch_bounds__(256) fc_weight_grad_atomic_kernel(const float *__restrict__ dY, const int32_t *__restrict__ idx,
                                                                   float *__restrict__ target, int64_t batch,
                                                                   int n_outputs, int n_detectors, int table_rows,
                                                                   int lanes_per_row, int chunk, double lr,
                                                                   double fixed_scale) {
    const int lane = threadIdx.x & 31;
    const int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= batch) return;
    const int c0 = blockIdx.y * chunk;
    const int clen = min(chunk, n_outputs - c0);
    const int LG = lanes_per_row;
    const int NG = 32 / LG;
    const int g = lane / LG;
    const int j = lane - g * LG;
    const float *dy = dY + b * n_outputs + c0;
    const int32_t *idx_b = idx + b * n_detectors;

    float val[kFwdJ][VEC];
    int32_t ival[kFwdJ][VEC];
#pragma unroll
    for (int q = 0; q < kFwdJ; q++) {
        const int col = (j + q * LG) * VEC;
#pragma unroll
        for (int e = 0; e < VEC; e++) { val[q][e] = 0.f; ival[q][e] = 0; }
        if (col < clen) {
            float d[VEC];
            Vec<VEC>::load(dy + col, d);
#pragma unroll
            for (int e = 0; e < VEC; e++) {
                const double gd = (double)d[e];
                if (fabs(gd) > kEps) {
                    if (INT_MODE) ival[q][e] = to_fixed(gd * lr, fixed_scale);
                    else val[q][e] = (float)(gd * lr);
                }
            }
        }
    }
    for (int tb = 0; tb < n_detectors; tb += 32) {
        const int nvalid = min(32, n_detectors - tb);
        const int32_t mine = (lane < nvalid) ? __ldg(idx_b + tb + lane) : 0;
        for (int sb = 0; sb < nvalid; sb += NG) {
            const int s = sb + g;
            const int32_t li = __shfl_sync(0xffffffffu, mine, s & 31);
            if (s < nvalid) {
                float *row = target + ((size_t)(tb + s) * table_rows + li) * n_outputs + c0;
#pragma unroll
                for (int q = 0; q < kFwdJ; q++) {
                    const int col = (j + q * LG) * VEC;
                    if (col < clen) {
                        if constexpr (INT_MODE) {
#pragma unroll
                            for (int e = 0; e < VEC; e++)
                                if (ival[q][e] != 0) atomicAdd(reinterpret_cast<int32_t *>(row + col + e), ival[q][e]);
                        } else if constexpr (VEC == 4) {
                            red_add_v4(row + col, val[q][0], val[q][1], val[q][2], val[q][3]);
                        } else {
                            if (val[q][0] != 0.f) atomicAdd(row + col, val[q][0]);
                        }
                    }
                }
            }
        }
    }
}

int launch_fc_backward(const lutb_layer_cfg *cfg, int64_t batch, float *W, const float *dY, const int32_t *anchors,
                       const int32_t *idx, const float *min_delta, const int32_t *min_k, float *dX, float *target,
                       double lr, cudaStream_t stream, bool skip_table_gradient = false) {
    const int O = cfg->n_outputs, Nt = cfg->n_detectors, T = 1 << cfg->n_anchors;
    const bool int_mode = cfg->int_mode != 0;
    const bool vec4 = (O % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(dY) & 15) == 0) && ((reinterpret_cast<uintptr_t>(target) & 15) == 0);
    const int vec = vec4 ? 4 : 1;
    const int vpr = (O + vec - 1) / vec;
    const int lanes = min(32, pow2_ceil(vpr));
    const int warps = 8;
    const int64_t blocks = (batch + warps - 1) / warps;
    LUTB_REQUIRE(blocks <= 0x7FFFFFFF, LUTB_ERR_SHAPE, "batch too large for one launch");
    const int sm = device_info().sm_count;

    // input gradient (dX == nullptr: the caller does not want it)
    if (dX != nullptr) {
    KernelScope scope(K_FC_INPUT_GRAD, stream);
    if (int_mode) {
        const int64_t total = batch * Nt;
        const int64_t gblocks = min((total + 127) / 128, (int64_t)sm * 64);
        fc_input_grad_fixed_kernel<<<(unsigned)gblocks, 128, 0, stream>>>(
            W, dY, reinterpret_cast<const int2 *>(anchors), idx, min_delta, min_k, dX, batch, cfg->n_inputs, O, Nt,
            cfg->n_anchors, T, cfg->forward_group, cfg->int_rescaler);
    } else if (vec4) {
        fc_input_grad_kernel<4><<<(unsigned)blocks, warps * 32, 0, stream>>>(
            W, dY, reinterpret_cast<const int2 *>(anchors), idx, min_delta, min_k, dX, batch, cfg->n_inputs, O, Nt,
            cfg->n_anchors, T, lanes);
    } else {
        fc_input_grad_kernel<1><<<(unsigned)blocks, warps * 32, 0, stream>>>(
            W, dY, reinterpret_cast<const int2 *>(anchors), idx, min_delta, min_k, dX, batch, cfg->n_inputs, O, Nt,
            cfg->n_anchors, T, lanes);
    }
    }
    LUTB_LAUNCH_CHECK();

    if (skip_table_gradient) return LUTB_OK;
    // table gradient (or in-place update)
    const int chunk = min(O, lanes * kFwdJ * vec);
    const int n_chunks = (O + chunk - 1) / chunk;
    LUTB_REQUIRE(n_chunks <= 65535, LUTB_ERR_SHAPE, "too many output chunks");
    dim3 grid((unsigned)blocks, (unsigned)n_chunks);
    KernelScope scope(K_FC_WEIGHT_GRAD, stream);
    if (vec4) {
        if (int_mode)
            fc_weight_grad_atomic_kernel<4, true><<<grid, warps * 32, 0, stream>>>(dY, idx, target, batch, O, Nt, T, lanes, chunk, lr, cfg->int_rescaler);
        else
            fc_weight_grad_atomic_kernel<4, false><<<grid, warps * 32, 0, stream>>>(dY, idx, target, batch, O, Nt, T, lanes, chunk, lr, cfg->int_rescaler);
    } else {
        if (int_mode)
            fc_weight_grad_atomic_kernel<1, true><<<grid, warps * 32, 0, stream>>>(dY, idx, target, batch, O, Nt, T, lanes, chunk, lr, cfg->int_rescaler);
        else
            fc_weight_grad_atomic_kernel<1, false><<<grid, warps * 32, 0, stream>>>(dY, idx, target, batch, O, Nt, T, lanes, chunk, lr, cfg->int_rescaler);
    }
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

}  // namespace lutb

// ------------------------------------------------------------------------------------------ C ABI
using namespace lutb;

extern "C" int lutb_nonseq_fc_forward(const lutb_layer_cfg *cfg, int64_t batch, const float *weights, const float *x,
                                      const int32_t *anchors, float *y, int32_t *idx, float *min_delta,
                                      int32_t *min_k, void *stream) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->seq_len == 1, LUTB_ERR_MODE, "forward_step should only be called when sequence_length == 1");
    LUTB_REQUIRE(batch > 0, LUTB_ERR_SHAPE, "batch_size == 0");
    LUTB_REQUIRE(weights && x && anchors && y && idx, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE((min_delta == nullptr) == (min_k == nullptr), LUTB_ERR_MODE,
                 "min_anchor_deltas and min_anchor_delta_indices must be given together");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = launch_check_detectors(x, batch, cfg->n_inputs, anchors, cfg->n_detectors, cfg->n_anchors, cfg->cmp_eps, idx,
                                min_delta, min_k, st);
    if (rc) return rc;
    rc = launch_fc_gather_forward(weights, idx, y, batch, cfg->n_outputs, cfg->n_detectors, 1 << cfg->n_anchors,
                                  cfg->backward_group, cfg->int_mode != 0, cfg->int_rescaler, st);
    if (rc) return rc;
    if (cfg->int_mode) return launch_fixed_to_float(y, batch * (int64_t)cfg->n_outputs, cfg->int_rescaler, st);
    return LUTB_OK;
}

extern "C" size_t lutb_nonseq_fc_backward_workspace(const lutb_layer_cfg *cfg, int64_t batch, int dw_variant) {
    if (cfg == nullptr || batch <= 0 || dw_variant != LUTB_DW_SORTED || cfg->int_mode) return 0;
    return fc_dw_sorted_workspace(batch, cfg->n_detectors, 1 << cfg->n_anchors);
}

extern "C" int lutb_nonseq_fc_backward(const lutb_layer_cfg *cfg, int64_t batch, float *weights, const float *dY,
                                       const int32_t *anchors, const int32_t *idx, const float *min_delta,
                                       const int32_t *min_k, float *dX, float *dW, double external_lr, int dw_variant,
                                       void *workspace, size_t workspace_bytes, void *stream) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->seq_len == 1, LUTB_ERR_MODE, "backward_backprop should only be called when sequence_length == 1");
    LUTB_REQUIRE(dw_variant == LUTB_DW_AUTO || dw_variant == LUTB_DW_ATOMIC || dw_variant == LUTB_DW_SORTED, LUTB_ERR_MODE,
                 "unknown dw_variant %d", dw_variant);
    // fixed-point sums are order independent already: the sorted variant only applies to fp32 accumulators
    const bool sorted = dw_variant == LUTB_DW_SORTED && !cfg->int_mode;
    if (sorted) {
        const size_t need = fc_dw_sorted_workspace(batch, cfg->n_detectors, 1 << cfg->n_anchors);
        LUTB_REQUIRE(workspace != nullptr && workspace_bytes >= need, LUTB_ERR_WORKSPACE,
                     "the sorted table-gradient variant needs %zu bytes of workspace", need);
        LUTB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, LUTB_ERR_ALIGN, "workspace must be 256-byte aligned");
    }
    LUTB_REQUIRE(batch > 0, LUTB_ERR_SHAPE, "batch_size == 0");
    LUTB_REQUIRE(weights && dY && anchors && idx && min_delta && min_k, LUTB_ERR_NULL,
                 "a required tensor pointer is NULL");
    LUTB_REQUIRE(!(external_lr >= 0.0 && dW != nullptr), LUTB_ERR_MODE,
                 "in internal weight gradients mode w_weights_gradients should be nullptr");
    const bool skip_table = external_lr == LUTB_SKIP_TABLE_GRADIENT;
    LUTB_REQUIRE(!(skip_table && dW != nullptr), LUTB_ERR_MODE, "no table gradient asked for, w_weights_gradients should be nullptr");
    LUTB_REQUIRE(!(external_lr < 0.0 && dW == nullptr && !skip_table), LUTB_ERR_NULL, "w_weights_gradients is NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    double lr = cfg->lr_meta;
    // the reference narrows external_lr to fp32 before use (lut.cu:1076)
    if (external_lr >= 0.0) lr *= -(double)(float)external_lr;
    float *target = external_lr >= 0.0 ? weights : dW;
    rc = launch_fc_backward(cfg, batch, weights, dY, anchors, idx, min_delta, min_k, dX, target, lr, st, sorted || skip_table);
    if (rc) return rc;
    if (sorted && !skip_table) {
        rc = launch_fc_dw_sorted(dY, idx, target, batch, cfg->n_outputs, cfg->n_detectors, 1 << cfg->n_anchors, lr,
                                 workspace, st);
        if (rc) return rc;
    }
    if (cfg->int_mode) {
        if (dX) rc = launch_fixed_to_float(dX, batch * (int64_t)cfg->n_inputs, cfg->int_rescaler, st);
        if (rc) return rc;
        if (dW) rc = launch_fixed_to_float(dW, (int64_t)cfg->n_detectors * (1 << cfg->n_anchors) * cfg->n_outputs, cfg->int_rescaler, st);
    }
    return rc;
}

extern "C" size_t lutb_nonseq_fc_table_grad_rows_workspace(const lutb_layer_cfg *cfg, int64_t batch) {
    if (cfg == nullptr || batch <= 0 || cfg->int_mode) return 0;
    return fc_dw_rows_workspace(batch, cfg->n_detectors, 1 << cfg->n_anchors);
}

extern "C" int lutb_nonseq_fc_table_grad_rows(const lutb_layer_cfg *cfg, int64_t batch, const float *dY,
                                              const int32_t *idx, int64_t *row_ids, float *values, int64_t capacity,
                                              int64_t *count_out, void *workspace, size_t workspace_bytes, void *stream) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->seq_len == 1, LUTB_ERR_MODE, "the row-list table gradient is for sequence_length == 1");
    LUTB_REQUIRE(cfg->int_mode == 0, LUTB_ERR_MODE, "the row-list table gradient needs fp32 accumulators");
    LUTB_REQUIRE(batch > 0, LUTB_ERR_SHAPE, "batch_size == 0");
    LUTB_REQUIRE(dY && idx && row_ids && values && count_out, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE(capacity > 0, LUTB_ERR_SHAPE, "capacity == 0");
    const size_t need = fc_dw_rows_workspace(batch, cfg->n_detectors, 1 << cfg->n_anchors);
    LUTB_REQUIRE(workspace != nullptr && workspace_bytes >= need, LUTB_ERR_WORKSPACE,
                 "the row-list table gradient needs %zu bytes of workspace", need);
    LUTB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, LUTB_ERR_ALIGN, "workspace must be 256-byte aligned");
    return launch_fc_dw_rows(dY, idx, batch, cfg->n_outputs, cfg->n_detectors, 1 << cfg->n_anchors, cfg->lr_meta, row_ids,
                             values, capacity, count_out, workspace, static_cast<cudaStream_t>(stream));
}

extern "C" int lutb_nonseq_fc_backward_noalloc(const lutb_layer_cfg *cfg, int64_t batch, float *weights,
                                               const float *dY, const int32_t *anchors, const int32_t *idx,
                                               const float *min_delta, const int32_t *min_k, float *dX, float *dW,
                                               double external_lr, void *stream) {
    NoEventsGuard no_events;  // event creation allocates
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->int_mode == 0, LUTB_ERR_MODE,
                 "the no-allocation backward supports fp32 accumulators only (int_mode must be 0)");
    LUTB_REQUIRE(batch > 0, LUTB_ERR_SHAPE, "batch_size == 0");
    const size_t need = fc_dw_sorted_workspace(batch, cfg->n_detectors, 1 << cfg->n_anchors);
    LUTB_REQUIRE(need <= (size_t)LUTB_STATIC_SCRATCH_BYTES, LUTB_ERR_WORKSPACE,
                 "problem needs %zu bytes of scratch, the built-in array holds %u: reduce the batch or use "
                 "lutb_nonseq_fc_backward with a caller workspace", need, (unsigned)LUTB_STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    rc = static_scratch(&scratch);
    if (rc) return rc;
    return lutb_nonseq_fc_backward(cfg, batch, weights, dY, anchors, idx, min_delta, min_k, dX, dW, external_lr,
                                   LUTB_DW_SORTED, scratch, (size_t)LUTB_STATIC_SCRATCH_BYTES, stream);
}
