// Histogram formulation of the product-mode sequence layer (see product_hist.cuh).
//
// Reference semantics: fill_outputs_product_cpu_logic (lut_runtime_kernels_logic.proto:2148-2264),
// propagate_backward_product_cpu_logic (:2396-2628), gather_w_gradients_internal_product_cpu_logic (:2630-2744).
#include "product_hist.cuh"
#include "fp32_gemm_sm100.cuh"
#include "product_pairs.cuh"

namespace lutb {

// --------------------------------------------------------------------------------------------
// Row-selection histogram.  Block = (detector, sequence of the chunk); a warp owns a query j, counts the
// rows its j keys select in a per-warp shared-memory histogram and writes it out as T uint16 counters.
// H layout: [detector][row of the chunk = local sequence * S + j][T].
// --------------------------------------------------------------------------------------------
// F32_ROWS: the counters are written as fp32 in the layout [row of the chunk][detector][T], the operand layout of the
// tensor-core contractions (one plain GEMM over all detectors per pass).
template <bool F32_ROWS>
__global__ void __launch_bounds__(512) product_hist_kernel(const float *__restrict__ x1, const float *__restrict__ x2,
                                                          const float *__restrict__ pe,
                                                          const int32_t *__restrict__ anchors, void *__restrict__ Hout,
                                                          int64_t b0, int64_t chunk_rows, int S, int e1, int e2, int npe,
                                                          int n_detectors, int n_anchors, int sliced, float cmp_eps) {
    extern __shared__ __align__(16) float smem[];
    const int t = blockIdx.x;
    const int64_t bl = blockIdx.y, b = b0 + bl;
    PairStage st;
    stage_pairs(st, smem, x1 + b * S * e1, x2 + b * S * e2, pe, anchors + (size_t)t * n_anchors * 2, S, e1, e2, npe,
                n_anchors, n_detectors, t, sliced != 0, cmp_eps);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int T = 1 << n_anchors;
    uint32_t *hist = reinterpret_cast<uint32_t *>(st.scratch) + warp * T;
    for (int r = lane; r < T; r += 32) hist[r] = 0u;
    __syncwarp();
    for (int j = warp; j < S; j += nwarps) {
        for (int i0 = 0; i0 < j; i0 += 32) {
            const int i = i0 + lane;
            int km; float dm;
            if (i < j) atomicAdd(hist + eval_pair<false>(st, n_anchors, i, j, cmp_eps, km, dm), 1u);
        }
        __syncwarp();
        if (F32_ROWS) {
            float *out = static_cast<float *>(Hout) + ((size_t)(bl * S + j) * n_detectors + t) * T;
            for (int r = lane * 4; r < T; r += 128) {
                const uint4 c = *reinterpret_cast<const uint4 *>(hist + r);
                *reinterpret_cast<float4 *>(out + r) = make_float4((float)c.x, (float)c.y, (float)c.z, (float)c.w);
                *reinterpret_cast<uint4 *>(hist + r) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
            continue;
        }
        uint16_t *out = static_cast<uint16_t *>(Hout) + ((size_t)t * chunk_rows + bl * S + j) * T;
        for (int r = lane * 8; r < T; r += 256) {
            const uint4 lo = *reinterpret_cast<const uint4 *>(hist + r);
            const uint4 hi = *reinterpret_cast<const uint4 *>(hist + r + 4);
            uint4 packed;
            packed.x = lo.x | (lo.y << 16);
            packed.y = lo.z | (lo.w << 16);
            packed.z = hi.x | (hi.y << 16);
            packed.w = hi.z | (hi.w << 16);
            *reinterpret_cast<uint4 *>(out + r) = packed;
            *reinterpret_cast<uint4 *>(hist + r) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4 *>(hist + r + 4) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
    }
}

// --------------------------------------------------------------------------------------------
// Input-gradient routing.  Same block / warp layout; the warp stages Q_t[(b,j), :] (the dot product of
// dY[b,j,:] with every row of table t) and each pair reads its two entries: g = Q[idx] - Q[idx ^ 2^kmin],
// du = up(min_delta) * g, +du / -du to the sources of the flipped anchor's two ends.
// SMEM_ACC: the block first sums its contributions per (token, anchor end) and per (distance, element) in shared
// memory and issues one global atomic per touched cell at the end (the global atomics of a block drop from one
// or two per pair to at most S * 2 * Nc + (S-1) * Npe); without it only the query token's cells are pre-reduced
// per warp.
// --------------------------------------------------------------------------------------------
// MAXM > 0: the pair loop keeps the address plan of the detector's mixed anchors (at most MAXM) in registers
// (product_pairs.cuh, MixedPlan); 0: plain eval_pair.  The plan costs about 5 registers per anchor: it pays where the
// block's shared memory already limits an SM to one block (tables of 1024 rows and more: 257 against 286 ms per step on
// the 1024-token, 1024-row configuration) and loses where it takes the second block away (256-row tables: 5.1 against 3.5 ms).
// HIST: the kernel evaluates every pair anyway, so it can count the selected rows on the way and write the histogram
// the table-gradient contraction needs (1: uint16 [detector][row of the chunk][T], 2: fp32 [row of the chunk][detector][T],
// the layouts of product_hist_kernel); the backward pass then launches no histogram kernel of its own.  Used where the
// extra T counters per warp do not cost the block its occupancy.
// QG: the two entries of Q a pair needs are read from global memory (through L1) instead of from a staged copy of the
// query's row: T floats less scratch per warp, on long sequences the difference between 8 and 16 warps per block.
template <bool SMEM_ACC, int MAXM, int HIST, bool QG>
__global__ void __launch_bounds__(512) product_route_kernel(const float *__restrict__ x1, const float *__restrict__ x2,
                                                           const float *__restrict__ pe,
                                                           const int32_t *__restrict__ anchors,
                                                           const float *__restrict__ Q, float *__restrict__ dX1,
                                                           float *__restrict__ dX2, float *__restrict__ dPE, int64_t b0,
                                                           int64_t q_row_stride, int64_t q_det_stride, int S, int e1,
                                                           int e2, int npe, int n_detectors, int n_anchors, int sliced,
                                                           float cmp_eps, void *__restrict__ Hout, int64_t chunk_rows) {
    extern __shared__ __align__(16) float smem[];
    const int t = blockIdx.x;
    const int64_t bl = blockIdx.y, b = b0 + bl;
    PairStage st;
    stage_pairs(st, smem, x1 + b * S * e1, x2 + b * S * e2, pe, anchors + (size_t)t * n_anchors * 2, S, e1, e2, npe,
                n_anchors, n_detectors, t, sliced != 0, cmp_eps);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int T = 1 << n_anchors;
    const int ends = 2 * n_anchors;
    const int q_floats = QG ? 0 : T;
    const int per_warp = q_floats + 32 * ends + (HIST ? T : 0);
    float *q_s = st.scratch + warp * per_warp;
    uint32_t *hist = reinterpret_cast<uint32_t *>(q_s + q_floats + 32 * ends);
    if (HIST) {
        for (int r = lane; r < T; r += 32) hist[r] = 0u;
        __syncwarp();
    }
    // contributions to the query token j: a private column per lane ([end][lane], plain read-modify-write; every
    // lane of a pair batch would otherwise hit the same few cells), summed over the lanes once per query
    float *jacc = q_s + q_floats;
    float *tacc = st.scratch + nwarps * per_warp;  // [S][ends]
    float *pacc = tacc + S * ends;                            // [S-1][npe]
    if (SMEM_ACC) {
        for (int w = threadIdx.x; w < S * ends + (S - 1) * npe; w += blockDim.x) tacc[w] = 0.f;
        __syncthreads();
    }
    MixedPlan<MAXM == 0 ? 1 : MAXM> mp;
    if (MAXM > 0) mp.load(st);
    for (int j = (HIST ? 0 : 1) + warp; j < S; j += nwarps) {   // (query 0 has no pair: only its empty histogram row)
        QueryPart qp{0u, 0.f};
        if (MAXM > 0) {
            mp.set_query(st, j);
            qp = query_part(st, j);
        }
        const float *qrow = Q + (size_t)t * q_det_stride + (size_t)(bl * S + j) * q_row_stride;
        if (!QG)
            for (int r = lane * 4; r < T; r += 128)
                *reinterpret_cast<float4 *>(q_s + r) = __ldcs(reinterpret_cast<const float4 *>(qrow + r));
        for (int q = 0; q < ends; q++) jacc[q * 32 + lane] = 0.f;
        __syncwarp();
        for (int i0 = 0; i0 < j; i0 += 32) {
            const int i = i0 + lane;
            if (i >= j) continue;
            int k; float d;
            const int32_t li = MAXM > 0 ? eval_pair_planned<true, (MAXM == 0 ? 1 : MAXM)>(st, mp, qp, i, j, cmp_eps, k, d)
                                        : eval_pair<true>(st, n_anchors, i, j, cmp_eps, k, d);
            if (HIST) atomicAdd(hist + li, 1u);
            if (k < 0) continue;
            // up(d) * (Q[row] - Q[flipped row]) in fp32: Q is an fp32 contraction already, and the double-precision
            // reciprocal of the reference's formula was the most expensive part of a pair (the direct kernels and the
            // fixed-point mode keep it)
            const float rcp = __frcp_rn(1.0f + fabsf(d));
            const float q_sel = QG ? __ldg(qrow + li) : q_s[li];
            const float q_alt = QG ? __ldg(qrow + (li ^ (1 << k))) : q_s[li ^ (1 << k)];
            const float du = (d > 0.f ? 0.5f : -0.5f) * rcp * rcp * (q_sel - q_alt);
            if (!(fabsf(du) > kEpsF)) continue;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int comp = st.comp[2 * k + e], elem = st.elem[2 * k + e];
                const float val = e == 0 ? du : -du;
                if (comp == 0) {
                    if (SMEM_ACC) atomicAdd(tacc + i * ends + 2 * k + e, val);
                    else atomicAdd(dX1 + ((size_t)b * S + i) * e1 + elem, val);
                } else if (comp == 1) {
                    jacc[(2 * k + e) * 32 + lane] += val;
                } else if (comp == 2) {
                    if (SMEM_ACC) atomicAdd(pacc + (j - i - 1) * npe + elem, val);
                    else atomicAdd(dPE + ((size_t)(j - i - 1) * n_detectors + t) * npe + elem, val);
                }
            }
        }
        __syncwarp();
        if (lane < ends && st.comp[lane] == 1) {
            float sum = 0.f;
#pragma unroll 8
            for (int m = 0; m < 32; m++) sum += jacc[lane * 32 + ((m + lane) & 31)];
            if (sum != 0.f) {
                if (SMEM_ACC) atomicAdd(tacc + j * ends + lane, sum);
                else atomicAdd(dX2 + ((size_t)b * S + j) * e2 + st.elem[lane], sum);
            }
        }
        __syncwarp();
        if (HIST == 2) {
            float *out = static_cast<float *>(Hout) + ((size_t)(bl * S + j) * n_detectors + t) * T;
            for (int r = lane * 4; r < T; r += 128) {
                const uint4 c = *reinterpret_cast<const uint4 *>(hist + r);
                *reinterpret_cast<float4 *>(out + r) = make_float4((float)c.x, (float)c.y, (float)c.z, (float)c.w);
                *reinterpret_cast<uint4 *>(hist + r) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
        } else if (HIST == 1) {
            uint16_t *out = static_cast<uint16_t *>(Hout) + ((size_t)t * chunk_rows + bl * S + j) * T;
            for (int r = lane * 8; r < T; r += 256) {
                const uint4 lo = *reinterpret_cast<const uint4 *>(hist + r);
                const uint4 hi = *reinterpret_cast<const uint4 *>(hist + r + 4);
                uint4 packed;
                packed.x = lo.x | (lo.y << 16);
                packed.y = lo.z | (lo.w << 16);
                packed.z = hi.x | (hi.y << 16);
                packed.w = hi.z | (hi.w << 16);
                *reinterpret_cast<uint4 *>(out + r) = packed;
                *reinterpret_cast<uint4 *>(hist + r) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4 *>(hist + r + 4) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
        }
    }
    if (SMEM_ACC) {
        __syncthreads();
        for (int w = threadIdx.x; w < S * ends; w += blockDim.x) {
            const float v = tacc[w];
            if (v == 0.f) continue;
            const int s = w / ends, q = w - s * ends;
            if (st.comp[q] == 0) atomicAdd(dX1 + ((size_t)b * S + s) * e1 + st.elem[q], v);
            else if (st.comp[q] == 1) atomicAdd(dX2 + ((size_t)b * S + s) * e2 + st.elem[q], v);
        }
        for (int w = threadIdx.x; w < (S - 1) * npe; w += blockDim.x) {
            const float v = pacc[w];
            if (v == 0.f) continue;
            const int d = w / npe, c = w - d * npe;
            atomicAdd(dPE + ((size_t)d * n_detectors + t) * npe + c, v);
        }
    }
}

// --------------------------------------------------------------------------------------------
// Register-tiled fp32 contraction  C[z] (+)= alpha * A[z] . B[z]  on 128 x 128 x 16 tiles: 256 threads, an
// 8 x 8 accumulator block per thread (updated with packed two-wide fp32 FMAs), operands staged k-major in shared
// memory ([k][m] and [k][n]) so the inner loop reads them with 16-byte loads, the next tile prefetched into registers while the current one is
// consumed.  Operand sources come in two layouts: "k contiguous" (element (m, k) at m * ld + k) and "row of k"
// (element (m, k) at k * ld + m); A may hold uint16 counters.
// --------------------------------------------------------------------------------------------
constexpr int GM = 128, GK = 16, GLD = GM + 4;

enum OperandKind { KC_F32, KC_U16, RK_F32, RK_U16 };

struct Frag { uint4 r[2]; };

// Loads this thread's part of the tile rows [m0, m0+128) x k [k0, k0+16); out-of-range parts read as zero.
template <int KIND>
__device__ __forceinline__ void fetch_tile(Frag &f, const void *base, int64_t ld, int m0, int M, int k0, int K) {
    const int tid = threadIdx.x;
    f.r[0] = make_uint4(0u, 0u, 0u, 0u);
    f.r[1] = make_uint4(0u, 0u, 0u, 0u);
    if (KIND == KC_F32) {
        const float *p = static_cast<const float *>(base);
        const int k = k0 + (tid & 3) * 4;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int m = m0 + (tid >> 2) + h * 64;
            if (m < M && k < K) f.r[h] = __ldg(reinterpret_cast<const uint4 *>(p + (int64_t)m * ld + k));
        }
    } else if (KIND == KC_U16) {
        const uint16_t *p = static_cast<const uint16_t *>(base);
        // a warp takes 32 consecutive rows of one k-half: its transposed stores then fall into 32 different banks
        const int m = m0 + (tid & 127), k = k0 + (tid >> 7) * 8;
        if (m < M && k < K) f.r[0] = __ldg(reinterpret_cast<const uint4 *>(p + (int64_t)m * ld + k));
    } else if (KIND == RK_F32) {
        const float *p = static_cast<const float *>(base);
        const int m = m0 + (tid & 31) * 4;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int k = k0 + (tid >> 5) + h * 8;
            if (m < M && k < K) f.r[h] = __ldg(reinterpret_cast<const uint4 *>(p + (int64_t)k * ld + m));
        }
    } else {
        const uint16_t *p = static_cast<const uint16_t *>(base);
        const int m = m0 + (tid & 15) * 8, k = k0 + (tid >> 4);
        if (m < M && k < K) f.r[0] = __ldg(reinterpret_cast<const uint4 *>(p + (int64_t)k * ld + m));
    }
}

__device__ __forceinline__ float lo16(uint32_t v) { return (float)(v & 0xffffu); }
__device__ __forceinline__ float hi16(uint32_t v) { return (float)(v >> 16); }

template <int KIND>
__device__ __forceinline__ void stash_tile(const Frag &f, float (*tile)[GLD]) {
    const int tid = threadIdx.x;
    if (KIND == KC_F32) {
        const int k = (tid & 3) * 4;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int m = (tid >> 2) + h * 64;
            tile[k + 0][m] = __uint_as_float(f.r[h].x);
            tile[k + 1][m] = __uint_as_float(f.r[h].y);
            tile[k + 2][m] = __uint_as_float(f.r[h].z);
            tile[k + 3][m] = __uint_as_float(f.r[h].w);
        }
    } else if (KIND == KC_U16) {
        const int m = tid & 127, k = (tid >> 7) * 8;
        tile[k + 0][m] = lo16(f.r[0].x); tile[k + 1][m] = hi16(f.r[0].x);
        tile[k + 2][m] = lo16(f.r[0].y); tile[k + 3][m] = hi16(f.r[0].y);
        tile[k + 4][m] = lo16(f.r[0].z); tile[k + 5][m] = hi16(f.r[0].z);
        tile[k + 6][m] = lo16(f.r[0].w); tile[k + 7][m] = hi16(f.r[0].w);
    } else if (KIND == RK_F32) {
        const int m = (tid & 31) * 4;
#pragma unroll
        for (int h = 0; h < 2; h++) *reinterpret_cast<uint4 *>(&tile[(tid >> 5) + h * 8][m]) = f.r[h];
    } else {
        const int m = (tid & 15) * 8, k = tid >> 4;
        *reinterpret_cast<float4 *>(&tile[k][m]) = make_float4(lo16(f.r[0].x), hi16(f.r[0].x), lo16(f.r[0].y), hi16(f.r[0].y));
        *reinterpret_cast<float4 *>(&tile[k][m + 4]) = make_float4(lo16(f.r[0].z), hi16(f.r[0].z), lo16(f.r[0].w), hi16(f.r[0].w));
    }
}

struct GemmArgs {
    const void *A;
    const float *B;
    float *C;
    int M, N, K;
    int64_t lda, ldb, ldc;
    int64_t za, zb, zc;  // per blockIdx.z strides, in elements
    int kblock;          // A only: k = q * kblock + r is found at k-offset q * kblock_stride + r (k contiguous kinds)
    int64_t kblock_stride;
    float alpha;
    int accumulate;      // 0: C = alpha * acc, 1: C += alpha * acc
    int ksplit;          // > 1: blockIdx.z also splits K; partial sums are added atomically (accumulate only)
};

template <int KIND_A, int KIND_B>
__global__ void __launch_bounds__(256, 2) tile_contract_kernel(const GemmArgs g) {
    __shared__ __align__(16) float As[2][GK][GLD];
    __shared__ __align__(16) float Bs[2][GK][GLD];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GM, n0 = blockIdx.x * GM;
    const int64_t z = blockIdx.z / g.ksplit;
    const int split = blockIdx.z - (int)z * g.ksplit;
    const size_t a_elem = (KIND_A == KC_U16 || KIND_A == RK_U16) ? 2 : 4;
    const char *A = static_cast<const char *>(g.A) + (size_t)(z * g.za) * a_elem;
    const float *B = g.B + z * g.zb;
    float *C = g.C + z * g.zc;

    float2 acc[8][4];   // acc[i][j] = columns 2j, 2j+1 of accumulator row i (register pairs for the packed FMA)
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = make_float2(0.f, 0.f);

    const int all_tiles = (g.K + GK - 1) / GK, per_split = (all_tiles + g.ksplit - 1) / g.ksplit;
    const int kt0 = split * per_split, nkt = min(all_tiles, kt0 + per_split);
    Frag fa, fb;
    auto fetch = [&](int kt) {
        const int k0 = kt * GK;
        if (KIND_A == KC_F32 || KIND_A == KC_U16) {
            const int q = k0 / g.kblock, r = k0 - q * g.kblock;
            fetch_tile<KIND_A>(fa, A + (size_t)(q * g.kblock_stride) * a_elem, g.lda, m0, g.M, r, g.kblock < g.K ? g.kblock : g.K);
        } else {
            fetch_tile<KIND_A>(fa, A, g.lda, m0, g.M, k0, g.K);
        }
        fetch_tile<KIND_B>(fb, B, g.ldb, n0, g.N, k0, g.K);
    };
    if (kt0 >= nkt) return;
    fetch(kt0);
    stash_tile<KIND_A>(fa, As[kt0 & 1]);
    stash_tile<KIND_B>(fb, Bs[kt0 & 1]);
    __syncthreads();
    for (int kt = kt0; kt < nkt; kt++) {
        const int buf = kt & 1;
        if (kt + 1 < nkt) fetch(kt + 1);
#pragma unroll 2
        for (int k = 0; k < GK; k++) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&As[buf][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4 *>(&As[buf][k][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[buf][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[buf][k][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float2 b[4] = {make_float2(b0.x, b0.y), make_float2(b0.z, b0.w), make_float2(b1.x, b1.y),
                                 make_float2(b1.z, b1.w)};
            // packed fp32 FMA (two independent round-to-nearest FMAs per instruction on sm_100): the loop is bound by
            // instruction issue, and halving the FMA instructions measured +15-18 %
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float2 aa = make_float2(a[i], a[i]);
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = __ffma2_rn(aa, b[j], acc[i][j]);
            }
        }
        if (kt + 1 < nkt) {
            stash_tile<KIND_A>(fa, As[buf ^ 1]);
            stash_tile<KIND_B>(fb, Bs[buf ^ 1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (m >= g.M) continue;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int n = n0 + h * 64 + tx * 4;
            if (n >= g.N) continue;
            float4 *dst = reinterpret_cast<float4 *>(C + (int64_t)m * g.ldc + n);
            float4 v = make_float4(g.alpha * acc[i][h * 2].x, g.alpha * acc[i][h * 2].y, g.alpha * acc[i][h * 2 + 1].x,
                                   g.alpha * acc[i][h * 2 + 1].y);
            if (g.ksplit > 1) {
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                             : "memory");
                continue;
            }
            if (g.accumulate) {
                const float4 old = *dst;
                v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
            }
            *dst = v;
        }
    }
}

template <int KIND_A, int KIND_B>
static int launch_contract(KernelId id, GemmArgs g, int batches, cudaStream_t stream) {
    if (g.ksplit < 1) g.ksplit = 1;
    dim3 grid((unsigned)((g.N + GM - 1) / GM), (unsigned)((g.M + GM - 1) / GM), (unsigned)(batches * g.ksplit));
    LUTB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, LUTB_ERR_SHAPE, "product histogram path: chunk too large");
    KernelScope scope(id, stream);
    tile_contract_kernel<KIND_A, KIND_B><<<grid, 256, 0, stream>>>(g);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

static size_t stage_bytes(const ProductCall &c, size_t per_warp_floats, int warps = 8) {
    return (pair_stage_floats(c.S, c.cfg->n_anchors, c.cfg->pos_dim) + (size_t)warps * per_warp_floats) * 4;
}

// Long sequences leave room for only one block per SM (the staged tokens alone are 130 KB at 1024 tokens): give that
// block 16 warps when its per-warp scratch still fits.
static int pair_block_warps(const ProductCall &c, size_t per_warp_floats) {
    return (c.S >= 512 && stage_bytes(c, per_warp_floats, 16) <= (size_t)kMaxSmemPerBlock - 1024) ? 16 : 8;
}

bool product_hist_supported(const ProductCall &c, const void *weights, const void *io_rows, const void *dW) {
    const lutb_layer_cfg *cfg = c.cfg;
    if (cfg->int_mode || c.S < 2 || c.S > 65535) return false;
    if (cfg->n_anchors < 4 || cfg->n_anchors > 12 || cfg->n_outputs % 4 != 0) return false;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(weights) | reinterpret_cast<uintptr_t>(io_rows) |
                           reinterpret_cast<uintptr_t>(dW);
    if (bits & 15) return false;
    const size_t T = (size_t)1 << cfg->n_anchors;
    return stage_bytes(c, T + 64 * cfg->n_anchors) <= (size_t)kMaxSmemPerBlock - 1024;
}

static size_t bytes_per_sequence(const lutb_layer_cfg *cfg, int S, bool backward, bool tc) {
    const size_t cells = (size_t)cfg->n_detectors * S * ((size_t)1 << cfg->n_anchors);
    return align256(cells * (tc ? 4 : 2)) + (backward ? align256(cells * 4) : 0) + 512;
}

// Scratch of the tensor-core GEMMs of one pass over `rows` query rows: their own workspace plus the hi / lo copies of
// the operands (the tables, and the output gradients in the backward pass); the largest of the calls the pass makes.
static size_t tc_scratch_bytes(const lutb_layer_cfg *cfg, int64_t rows, bool backward) {
    const int KT = cfg->n_detectors << cfg->n_anchors, O = cfg->n_outputs;
    const size_t fwd = tc_gemm_workspace(TC_A_ROWS_B_ROWS_OF_K, (int)rows, O, KT, true);
    if (!backward) return align256(fwd);
    // (the forward contraction's scratch counts here too: a forward pass that leaves its histogram for the backward
    // pass lays the workspace out as the backward pass does)
    const size_t dw = tc_gemm_workspace(TC_A_COLS_B_ROWS_OF_K, KT, O, (int)rows, true),
                 q = tc_gemm_workspace(TC_A_ROWS_B_ROWS_OF_N, (int)rows, KT, O, false);
    const size_t m = dw > q ? dw : q;
    return align256(m > fwd ? m : fwd);
}

size_t product_hist_workspace_bytes(const lutb_layer_cfg *cfg, int64_t batch, int S, bool backward) {
    // what lets `batch` sequences through in one pass with either contraction: fp32 counters and operand copies for the
    // tensor cores, uint16 counters for the FMA kernel
    const bool tc = tc_gemm_available();
    return (tc ? tc_scratch_bytes(cfg, batch * S, backward) : 0) + (size_t)batch * bytes_per_sequence(cfg, S, backward, tc) + 256;
}

struct HistPlan {
    int64_t chunk;  // sequences per pass
    bool tc;        // tensor-core contractions: H is fp32 [row][detector][T], Q fp32 [row][detector][T]
    void *H;
    float *Q;
    void *gemm_ws;
    size_t gemm_ws_bytes;
};

static int plan(const ProductCall &c, bool backward, bool allow_tc, void *workspace, size_t bytes, HistPlan &p) {
    LUTB_REQUIRE(workspace != nullptr, LUTB_ERR_WORKSPACE, "product histogram path needs a workspace");
    const uintptr_t base0 = (reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t)255;
    const size_t slack = base0 - reinterpret_cast<uintptr_t>(workspace);
    const size_t T = (size_t)1 << c.cfg->n_anchors;
    // tensor cores when the library has them, the workspace holds at least one sequence in their layout, the GEMM
    // extents fit 32-bit sizes and the row counts (at most S - 1) are exact in TF32
    p.tc = allow_tc && tc_gemm_available() && c.S <= 2048 && (size_t)c.cfg->n_detectors * T < ((size_t)1 << 30) &&
           bytes >= slack + tc_scratch_bytes(c.cfg, c.S, backward) + bytes_per_sequence(c.cfg, c.S, backward, true);
    const size_t per_seq = bytes_per_sequence(c.cfg, c.S, backward, p.tc);
    LUTB_REQUIRE(bytes >= slack + per_seq, LUTB_ERR_WORKSPACE,
                 "product histogram path: workspace of %zu bytes is smaller than the %zu bytes one sequence needs", bytes,
                 per_seq + 256);
    p.chunk = (int64_t)((bytes - slack) / per_seq);
    if (p.chunk > c.batch) p.chunk = c.batch;
    // grid.y of the FMA contraction covers chunk * S / 128 row tiles; the GEMM extents are 32-bit
    const int64_t max_rows = p.tc ? (int64_t)1 << 30 : (int64_t)65535 * GM;
    if (p.chunk * c.S > max_rows) p.chunk = max_rows / c.S;
    size_t head = 0;
    if (p.tc) {
        // the GEMM scratch grows with the rows of a pass: shrink the pass until both fit
        while (p.chunk > 1 && slack + tc_scratch_bytes(c.cfg, p.chunk * c.S, backward) + (size_t)p.chunk * per_seq > bytes) p.chunk--;
        head = tc_scratch_bytes(c.cfg, p.chunk * c.S, backward);
    }
    LUTB_REQUIRE(p.chunk >= 1, LUTB_ERR_SHAPE, "product histogram path: sequence too long");
    const size_t cells = (size_t)c.cfg->n_detectors * (size_t)p.chunk * c.S * T;
    uintptr_t base = base0;
    p.gemm_ws = p.tc ? reinterpret_cast<void *>(base) : nullptr;
    p.gemm_ws_bytes = head;
    base += head;
    p.H = reinterpret_cast<void *>(base);
    p.Q = backward ? reinterpret_cast<float *>(base + align256(cells * (p.tc ? 4 : 2))) : nullptr;
    return LUTB_OK;
}

static int launch_hist(const ProductCall &c, const HistPlan &p, int64_t b0, int64_t n, cudaStream_t stream) {
    const lutb_layer_cfg *cfg = c.cfg;
    const size_t T = (size_t)1 << cfg->n_anchors;
    const int warps = pair_block_warps(c, T);
    const size_t smem = stage_bytes(c, T, warps);
    dim3 grid((unsigned)cfg->n_detectors, (unsigned)n);
    KernelScope scope(K_PRODUCT_HIST, stream);
    auto launch = [&](auto kern) -> int {
        if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, warps * 32, smem, stream>>>(c.x1, c.x2, c.pe, c.anchors, p.H, b0, n * c.S, c.S, c.e1, c.e2, cfg->pos_dim,
                                                 cfg->n_detectors, cfg->n_anchors, cfg->sliced_product, cfg->cmp_eps);
        return LUTB_OK;
    };
    const int rc = p.tc ? launch(product_hist_kernel<true>) : launch(product_hist_kernel<false>);
    if (rc) return rc;
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

bool product_hist_keeps(const ProductCall &c, bool allow_tc, void *workspace, size_t workspace_bytes) {
    HistPlan p;
    if (workspace == nullptr || workspace_bytes < product_hist_workspace_bytes(c.cfg, 1, c.S, true)) return false;
    if (plan(c, true, allow_tc, workspace, workspace_bytes, p) != LUTB_OK) return false;
    return p.chunk == c.batch;
}

int launch_product_hist_forward(const ProductCall &c, const float *weights, float *y, bool allow_tc, void *workspace,
                                size_t workspace_bytes, cudaStream_t stream, bool keep) {
    HistPlan p;
    // keep: the workspace is laid out as the backward pass lays it out, so that the histogram stays where that pass
    // looks for it (only when the whole batch goes through in one pass; otherwise the forward pass's own layout)
    const bool as_backward = keep && product_hist_keeps(c, allow_tc, workspace, workspace_bytes);
    int rc = plan(c, as_backward, allow_tc, workspace, workspace_bytes, p);
    if (rc) return rc;
    const lutb_layer_cfg *cfg = c.cfg;
    const int T = 1 << cfg->n_anchors, O = cfg->n_outputs, Nt = cfg->n_detectors;
    for (int64_t b0 = 0; b0 < c.batch; b0 += p.chunk) {
        const int64_t n = (c.batch - b0 < p.chunk) ? c.batch - b0 : p.chunk;
        const int64_t rows = n * c.S;
        rc = launch_hist(c, p, b0, n, stream);
        if (rc) return rc;
        if (p.tc) {
            // y[rows, O] += H[rows, Nt*T] . W[Nt*T, O]
            KernelScope scope(K_PRODUCT_HIST_FORWARD, stream);
            rc = tc_gemm(TC_A_ROWS_B_ROWS_OF_K, (int)rows, O, Nt * T, static_cast<const float *>(p.H), (int64_t)Nt * T, weights, O,
                         y + b0 * c.S * O, O, 1.f, 1.f, /*a_exact=*/true, p.gemm_ws, p.gemm_ws_bytes, stream);
            if (rc) return rc;
            continue;
        }
        GemmArgs g{};
        g.A = p.H; g.B = weights; g.C = y + b0 * c.S * O;
        g.M = (int)rows; g.N = O; g.K = Nt * T;
        g.lda = T; g.ldb = O; g.ldc = O;
        g.kblock = T; g.kblock_stride = rows * T;
        g.alpha = 1.f; g.accumulate = 1;
        rc = launch_contract<KC_U16, RK_F32>(K_PRODUCT_HIST_FORWARD, g, 1, stream);
        if (rc) return rc;
    }
    return LUTB_OK;
}

int launch_product_hist_backward(const ProductCall &c, const float *weights, const float *dY, float *dX1, float *dX2,
                                 float *dPE, float *target, double lr, bool in_place, bool allow_tc, void *workspace,
                                 size_t workspace_bytes, cudaStream_t stream, bool reuse) {
    HistPlan p;
    int rc = plan(c, true, allow_tc, workspace, workspace_bytes, p);
    if (rc) return rc;
    // reuse: the caller vouches that the workspace still holds the histogram a forward pass over the same inputs left
    // there; it is complete only when the whole batch is one pass
    const bool have_hist = reuse && p.chunk == c.batch;
    const lutb_layer_cfg *cfg = c.cfg;
    const int T = 1 << cfg->n_anchors, O = cfg->n_outputs, Nt = cfg->n_detectors;
    int route_warps = pair_block_warps(c, (size_t)T + 64 * cfg->n_anchors);
    // long sequences: Q read from global memory when that is what gives the block 16 warps
    const bool q_global = route_warps < 16 && pair_block_warps(c, (size_t)64 * cfg->n_anchors) == 16;
    if (q_global) route_warps = 16;
    size_t route_smem = stage_bytes(c, (q_global ? 0 : (size_t)T) + 64 * cfg->n_anchors, route_warps);
    const size_t acc_bytes = ((size_t)c.S * 2 * cfg->n_anchors + (size_t)(c.S - 1) * cfg->pos_dim) * 4;
    // block-level accumulators only while two blocks still fit an SM
    const bool smem_acc = !q_global && route_smem + acc_bytes <= 100 * 1024;
    if (smem_acc) route_smem += acc_bytes;
    // In-place SGD reads unmodified tables for every input gradient: with more than one chunk the table update
    // runs as a second sweep over the chunks.
    const bool second_sweep = in_place && p.chunk < c.batch;
    // the routing kernel counts the rows itself where T more counters per warp still leave room for two blocks per SM
    const bool fuse_hist = !have_hist && !second_sweep && smem_acc && !q_global && cfg->n_anchors <= 8 &&
                           route_smem + (size_t)route_warps * T * 4 <= 100 * 1024;
    if (fuse_hist) route_smem += (size_t)route_warps * T * 4;
    auto table_gradient = [&](int64_t b0, int64_t rows) -> int {
        if (p.tc) {
            // target[Nt*T, O] += lr * H^T . dY  (H stored [rows, Nt*T])
            KernelScope scope(K_PRODUCT_HIST_WEIGHT_GRAD, stream);
            return tc_gemm(TC_A_COLS_B_ROWS_OF_K, Nt * T, O, (int)rows, static_cast<const float *>(p.H), (int64_t)Nt * T,
                           dY + b0 * c.S * O, O, target, O, (float)lr, 1.f, /*a_exact=*/true, p.gemm_ws, p.gemm_ws_bytes, stream);
        }
        GemmArgs g{};
        g.A = p.H; g.B = dY + b0 * c.S * O; g.C = target;
        g.M = T; g.N = O; g.K = (int)rows;
        g.lda = T; g.ldb = O; g.ldc = O;
        g.za = rows * T; g.zb = 0; g.zc = (int64_t)T * O;
        g.kblock = g.K; g.kblock_stride = 0;
        g.alpha = (float)lr; g.accumulate = 1;
        // few output tiles and a long reduction: split K so that every SM gets several blocks
        const int64_t tiles = (int64_t)((T + GM - 1) / GM) * ((O + GM - 1) / GM) * Nt;
        const int64_t want = (8 * (int64_t)device_info().sm_count + tiles - 1) / tiles;
        const int64_t most = (rows / GK + 31) / 32;  // at least 32 k-tiles per block
        g.ksplit = (int)(want < 1 ? 1 : (want > most ? (most < 1 ? 1 : most) : want));
        return launch_contract<RK_U16, RK_F32>(K_PRODUCT_HIST_WEIGHT_GRAD, g, Nt, stream);
    };
    for (int64_t b0 = 0; b0 < c.batch; b0 += p.chunk) {
        const int64_t n = (c.batch - b0 < p.chunk) ? c.batch - b0 : p.chunk;
        const int64_t rows = n * c.S;
        if (!fuse_hist && !have_hist) {
            rc = launch_hist(c, p, b0, n, stream);
            if (rc) return rc;
        }
        if (p.tc) {
            // Q[rows, Nt*T] = dY[rows, O] . W^T  (W stored [Nt*T, O])
            KernelScope scope(K_PRODUCT_ROW_DOTS, stream);
            rc = tc_gemm(TC_A_ROWS_B_ROWS_OF_N, (int)rows, Nt * T, O, dY + b0 * c.S * O, O, weights, O, p.Q, (int64_t)Nt * T, 1.f,
                         0.f, /*a_exact=*/false, p.gemm_ws, p.gemm_ws_bytes, stream);
            if (rc) return rc;
        } else {
            GemmArgs g{};
            g.A = dY + b0 * c.S * O; g.B = weights; g.C = p.Q;
            g.M = (int)rows; g.N = T; g.K = O;
            g.lda = O; g.ldb = O; g.ldc = T;
            g.za = 0; g.zb = (int64_t)T * O; g.zc = rows * T;
            g.kblock = O; g.kblock_stride = 0;
            g.alpha = 1.f; g.accumulate = 0;
            rc = launch_contract<KC_F32, KC_F32>(K_PRODUCT_ROW_DOTS, g, Nt, stream);
            if (rc) return rc;
        }
        {
            const int64_t q_row_stride = p.tc ? (int64_t)Nt * T : T, q_det_stride = p.tc ? T : rows * T;
            dim3 grid((unsigned)Nt, (unsigned)n);
            KernelScope scope(K_PRODUCT_ROUTE, stream);
            auto launch = [&](auto kern) -> int {
                if (route_smem > 48 * 1024)
                    LUTB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)route_smem));
                kern<<<grid, route_warps * 32, route_smem, stream>>>(c.x1, c.x2, c.pe, c.anchors, p.Q, dX1, dX2, dPE, b0, q_row_stride,
                                                                     q_det_stride, c.S, c.e1, c.e2, cfg->pos_dim, Nt, cfg->n_anchors,
                                                                     cfg->sliced_product, cfg->cmp_eps, p.H, n * c.S);
                return LUTB_OK;
            };
            const int na = cfg->n_anchors;
            if (fuse_hist) rc = p.tc ? launch(product_route_kernel<true, 0, 2, false>) : launch(product_route_kernel<true, 0, 1, false>);
            else if (q_global)
                rc = na <= 8 ? launch(product_route_kernel<false, 0, 0, true>) : na <= 12 ? launch(product_route_kernel<false, 12, 0, true>)
                                                                                          : launch(product_route_kernel<false, 16, 0, true>);
            else if (smem_acc) rc = na <= 8 ? launch(product_route_kernel<true, 0, 0, false>) : na <= 12 ? launch(product_route_kernel<true, 12, 0, false>)
                                                                                                         : launch(product_route_kernel<true, 16, 0, false>);
            else rc = na <= 8 ? launch(product_route_kernel<false, 0, 0, false>) : na <= 12 ? launch(product_route_kernel<false, 12, 0, false>)
                                                                                             : launch(product_route_kernel<false, 16, 0, false>);
            if (rc) return rc;
            LUTB_LAUNCH_CHECK();
        }
        if (!second_sweep) {
            rc = table_gradient(b0, rows);
            if (rc) return rc;
        }
    }
    if (second_sweep) {
        for (int64_t b0 = 0; b0 < c.batch; b0 += p.chunk) {
            const int64_t n = (c.batch - b0 < p.chunk) ? c.batch - b0 : p.chunk;
            rc = launch_hist(c, p, b0, n, stream);
            if (rc) return rc;
            rc = table_gradient(b0, n * c.S);
            if (rc) return rc;
        }
    }
    return LUTB_OK;
}

}  // namespace lutb
