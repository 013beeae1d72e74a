// Non-sequence LUT layer with sparse lookup -> output connectivity (projection / convolution layers).
// Each table row holds one weight per target of its detector; all rows of a detector share the target
// list, so the layer is a set of small fully connected tables whose outputs are scattered to shared
// output cells.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "lutb_common.cuh"
#include "nonseq_fc.cuh"
#include "sparse_staged.cuh"
#include "sparse_view.cuh"

namespace lutb {

// The training kernels give one warp to a (chunk, run of kSampleRun samples) pair.  A chunk is a run of
// up to 32 consecutive detectors that share one target list (the detectors of one group) and whose
// tables lie back to back.  Work is ordered chunk-major: warps that run at the same time work on the
// same few chunks for different samples, so a chunk's tables (a few hundred KB) are fetched from HBM
// once and then served by L2 for the rest of the batch.
// Per sample, lane L loads the table index of detector L of the chunk (one coalesced read, issued one
// sample ahead so that it overlaps the row reads of the current sample) and turns it into the offset
// of the selected row from the chunk's first table; offsets are broadcast with shuffles while the lanes
// cover the synapses of a row, so every row access is one contiguous segment and all row reads of a
// sample are in flight together.  Rows of up to LG synapses use LG-lane groups (NG = 32 / LG groups
// take detectors round-robin).
constexpr int kSampleRun = 4;

// With 512 samples over 256-row tables every row is touched about twice per step, so half of the row gathers are
// compulsory DRAM misses at random addresses.  Each warp therefore asks L2 for its share of the tables of the
// chunk that will be processed kPrefetchAhead chunks later (about the chunks in flight on the whole GPU), turning
// those misses into a sequential stream that is resident when the gathers arrive.  Forward only: it runs 4 % faster
// for 20 % more DRAM reads (rows no sample selects are fetched too); the fused backward gained nothing from prefetching
// the table rows and lost time when its gradient rows were prefetched as well.
constexpr int kPrefetchAhead = 40;

__device__ __forceinline__ void prefetch_chunk(const SparseView &sp, const float *base, int64_t c, int64_t r, int64_t runs,
                                               int lane) {
    if (c >= sp.n_chunks) return;
    const ChunkStatic cs = load_chunk(sp, c);
    const int64_t lines = ((int64_t)cs.ndet * cs.table * 4 + 127) >> 7;
    const int64_t per = (lines + runs - 1) / runs;
    const int64_t end = min(lines, (r + 1) * per);
    const char *p = reinterpret_cast<const char *>(base + cs.wbase0);
    for (int64_t l = r * per + lane; l < end; l += 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + (l << 7)));
}

// --------------------------------------------------------------------------------------------
// Forward: y[b, target(p)] += sum over the chunk's detectors of W[row(t, idx[b, t]) + p]
// (reference: fill_outputs_non_seq_sparse_logic + fire_single_synapse_group, proto:1160-1212, 215-313).
// The chunk's detectors are summed in registers, so the shared output cells see one reduction per
// (sample, chunk, target) instead of one per synapse.
// --------------------------------------------------------------------------------------------
template <int LG, bool INT_MODE>
__device__ __forceinline__ void chunk_forward(const SparseView &sp, const ChunkStatic &cs, const float *__restrict__ W,
                                              const int32_t *__restrict__ idx, float *__restrict__ y, int64_t b0,
                                              int64_t b1, int n_outputs, int n_detectors, int lane,
                                              double fixed_scale) {
    constexpr int NG = 32 / LG;
    const int g = lane / LG, j = lane - g * LG;
    const bool valid = j < cs.P;
    const bool has_det = lane < cs.ndet;
    const float *Wb = W + cs.wbase0 + j + hole_offset(j, sp);
    const int target = (valid && g == 0) ? __ldg(sp.syn_target + cs.toff + j) : 0;
    const int32_t *idx_l = idx + cs.det0 + lane;
    int32_t li_next = has_det ? __ldg(idx_l + b0 * n_detectors) : 0;
    for (int64_t b = b0; b < b1; b++) {
        const int32_t row_off = has_det ? lane * cs.table + li_next * cs.stride : 0;
        if (b + 1 < b1 && has_det) li_next = __ldg(idx_l + (b + 1) * n_detectors);
        float w[LG];
#pragma unroll
        for (int i = 0; i < LG; i++) {
            const int d = i * NG + g;
            const int32_t off = __shfl_sync(0xffffffffu, row_off, d);
            w[i] = (valid && d < cs.ndet) ? __ldg(Wb + off) : 0.f;
        }
        float acc = 0.f;
        int32_t iacc = 0;
#pragma unroll
        for (int i = 0; i < LG; i++) {
            // beyond the chunk w is exactly 0 and truncates to 0
            if (INT_MODE) iacc += to_fixed((double)w[i], fixed_scale);
            else acc += w[i];
        }
#pragma unroll
        for (int m = LG; m < 32; m <<= 1) {
            if (INT_MODE) iacc += __shfl_xor_sync(0xffffffffu, iacc, m);
            else acc += __shfl_xor_sync(0xffffffffu, acc, m);
        }
        if (valid && g == 0) {
            if (INT_MODE) atomicAdd(reinterpret_cast<int32_t *>(y) + b * n_outputs + target, iacc);
            else atomicAdd(y + b * n_outputs + target, acc);
        }
    }
}

template <bool INT_MODE>
__global__ void __launch_bounds__(256, 4) sparse_forward_kernel(SparseView sp, const float *__restrict__ W,
                                                            const int32_t *__restrict__ idx, float *__restrict__ y,
                                                            int64_t batch, int n_outputs, int n_detectors,
                                                            double fixed_scale) {
    const int lane = threadIdx.x & 31;
    const int64_t runs = (batch + kSampleRun - 1) / kSampleRun;
    const int64_t work = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (work >= runs * sp.n_chunks) return;
    const int64_t c = work / runs;
    const int64_t b0 = (work - c * runs) * kSampleRun;
    const int64_t b1 = min(batch, b0 + kSampleRun);
    prefetch_chunk(sp, W, c + kPrefetchAhead, work - c * runs, runs, lane);
    const ChunkStatic cs = load_chunk(sp, c);
    if (cs.P <= 8) chunk_forward<8, INT_MODE>(sp, cs, W, idx, y, b0, b1, n_outputs, n_detectors, lane, fixed_scale);
    else if (cs.P <= 16) chunk_forward<16, INT_MODE>(sp, cs, W, idx, y, b0, b1, n_outputs, n_detectors, lane, fixed_scale);
    else if (cs.P <= 32) chunk_forward<32, INT_MODE>(sp, cs, W, idx, y, b0, b1, n_outputs, n_detectors, lane, fixed_scale);
    else {
        // rows longer than a warp: plain loop, one detector at a time
        const float *Wb = W + cs.wbase0;
        for (int64_t b = b0; b < b1; b++) {
            const int32_t li = lane < cs.ndet ? __ldg(idx + b * n_detectors + cs.det0 + lane) : 0;
            const int32_t row_off = lane * cs.table + li * cs.stride;
            // uniform trip count: every lane takes part in the offset broadcasts, lanes beyond the row only skip the loads
            for (int p0 = 0; p0 < cs.P; p0 += 32) {
                const int p = p0 + lane;
                const bool in_row = p < cs.P;
                const int q = p + hole_offset(p, sp);
                float acc = 0.f;
                int32_t iacc = 0;
                for (int d = 0; d < cs.ndet; d++) {
                    const int32_t ro = __shfl_sync(0xffffffffu, row_off, d);
                    if (!in_row) continue;
                    const float w = __ldg(Wb + (int64_t)ro + q);
                    if (INT_MODE) iacc += to_fixed((double)w, fixed_scale);
                    else acc += w;
                }
                if (!in_row) continue;
                const int target = __ldg(sp.syn_target + cs.toff + p);
                if (INT_MODE) atomicAdd(reinterpret_cast<int32_t *>(y) + b * n_outputs + target, iacc);
                else atomicAdd(y + b * n_outputs + target, acc);
            }
        }
    }
}

// --------------------------------------------------------------------------------------------
// Backward over a chunk (rows of at most 32 synapses):
//   input gradient (reference: propagate_through_detectors_non_seq_sparse_logic, proto:1303-1419):
//     per detector g = sum_p dY[target(p)] * (W[row + p] - W[alt + p]), du = up(min_delta) * g,
//     +du / -du on the two inputs of the minimum-margin anchor pair;
//   table gradient (reference: gather_w_gradients_non_seq_sparse_logic, proto:1501-1545, helper :584-714):
//     target[row + p] += lr * dY[target(p)] for |dY| > EPS.
// Each lane keeps one partial product sum per detector it sees (LG of them); a butterfly of LG - 1
// shuffles transposes and reduces them so that every lane ends with the full sum of exactly one
// detector and performs that detector's two updates itself.  Partial sums are fp32 (<= 32 terms), the
// scaling by up() is done in double.  The launcher runs the two parts as two passes (DO_DX, then DO_DW):
// measured faster than one fused pass, and required by the internal (in-place SGD) policy, where the
// table gradient modifies the very weights other samples still have to read.
// --------------------------------------------------------------------------------------------
template <int LG, bool DO_DX, bool DO_DW, bool INT_DW>
__device__ __forceinline__ void chunk_backward(const SparseView &sp, const ChunkStatic &cs, const float *__restrict__ W,
                                               const float *__restrict__ dY, const int2 *__restrict__ anchors,
                                               const int32_t *__restrict__ idx, const float *__restrict__ min_delta,
                                               const int32_t *__restrict__ min_k, float *__restrict__ dX,
                                               float *__restrict__ target_arr, int64_t b0, int64_t b1, int n_inputs,
                                               int n_outputs, int n_detectors, int n_anchors, int lane, double lr,
                                               double fixed_scale) {
    constexpr int NG = 32 / LG;
    const int g = lane / LG, j = lane - g * LG;
    const bool valid = j < cs.P;
    const bool has_det = lane < cs.ndet;
    const int q = j + hole_offset(j, sp);
    const int my_target = valid ? __ldg(sp.syn_target + cs.toff + j) : 0;
    const float *Wb = W + cs.wbase0 + q;
    float *Tb = DO_DW ? target_arr + cs.wbase0 + q : nullptr;
    // lane (g, j) ends up owning detector j * NG + g of the chunk
    const int own = j * NG + g;
    const int64_t det_l = cs.det0 + lane;
    // per-sample inputs are fetched one sample ahead
    int32_t li_n = 0, k_n = 0;
    float m_n = 0.f, gp_n = 0.f;
    if (has_det) {
        li_n = __ldg(idx + b0 * n_detectors + det_l);
        if (DO_DX) { k_n = __ldg(min_k + b0 * n_detectors + det_l); m_n = __ldg(min_delta + b0 * n_detectors + det_l); }
    }
    if (valid) gp_n = __ldg(dY + b0 * n_outputs + my_target);
    for (int64_t b = b0; b < b1; b++) {
        const int32_t li = li_n, my_k = k_n;
        const float my_m = m_n, gp = gp_n;
        if (b + 1 < b1) {
            if (has_det) {
                li_n = __ldg(idx + (b + 1) * n_detectors + det_l);
                if (DO_DX) { k_n = __ldg(min_k + (b + 1) * n_detectors + det_l); m_n = __ldg(min_delta + (b + 1) * n_detectors + det_l); }
            }
            if (valid) gp_n = __ldg(dY + (b + 1) * n_outputs + my_target);
        }
        const int32_t row_off = has_det ? lane * cs.table + li * cs.stride : 0;
        // alternative row: minimum-margin bit flipped
        const int32_t alt_off = (DO_DX && has_det) ? row_off + ((li ^ (1 << my_k)) - li) * cs.stride : 0;
        float val = 0.f;
        int32_t ival = 0;
        bool active = false;
        if (DO_DW && valid && fabsf(gp) > kEpsF) {
            active = true;
            if (INT_DW) ival = to_fixed((double)gp * lr, fixed_scale);
            else val = lr == 1.0 ? gp : (float)((double)gp * lr);   // the product with 1.0 is gp itself
        }
        float v[LG];
#pragma unroll
        for (int i = 0; i < LG; i++) {
            const int d = i * NG + g;
            const int32_t ro = __shfl_sync(0xffffffffu, row_off, d);
            if (DO_DX) {
                const int32_t ao = __shfl_sync(0xffffffffu, alt_off, d);
                // detectors beyond the chunk have ro == ao == 0: the difference is exactly zero
                v[i] = valid ? gp * (__ldg(Wb + ro) - __ldg(Wb + ao)) : 0.f;
            }
            if (DO_DW && active && d < cs.ndet) {
                if (INT_DW) atomicAdd(reinterpret_cast<int32_t *>(Tb) + ro, ival);
                else atomicAdd(Tb + ro, val);
            }
        }
        if (!DO_DX) continue;
        // transpose-reduce: after the stage with offset o a lane keeps the half of the values whose
        // index bit matches its own lane bit, summed with the partner lane's copy
#pragma unroll
        for (int o = LG / 2; o >= 1; o >>= 1) {
            const bool upper = (j & o) != 0;
#pragma unroll
            for (int i = 0; i < o; i++) {
                const float send = upper ? v[i] : v[i + o];
                const float keep = upper ? v[i + o] : v[i];
                v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
            }
        }
        const int32_t k = __shfl_sync(0xffffffffu, my_k, own);
        const float m = __shfl_sync(0xffffffffu, my_m, own);
        if (own < cs.ndet) {
            const double du = surrogate_up(m) * (double)v[0];
            if (fabs(du) > kEps) {
                const int2 a = __ldg(anchors + (size_t)(cs.det0 + own) * n_anchors + k);
                float *dxb = dX + b * n_inputs;
                atomicAdd(dxb + a.x, (float)du);
                atomicAdd(dxb + a.y, -(float)du);
            }
        }
    }
}

template <bool DO_DX, bool DO_DW, bool INT_DW>
__global__ void __launch_bounds__(256, DO_DX ? 3 : 4) sparse_backward_kernel(SparseView sp, const float *__restrict__ W,
                                                             const float *__restrict__ dY,
                                                             const int2 *__restrict__ anchors,
                                                             const int32_t *__restrict__ idx,
                                                             const float *__restrict__ min_delta,
                                                             const int32_t *__restrict__ min_k,
                                                             float *__restrict__ dX, float *__restrict__ target_arr,
                                                             int64_t batch, int n_inputs, int n_outputs,
                                                             int n_detectors, int n_anchors, double lr,
                                                             double fixed_scale) {
    const int lane = threadIdx.x & 31;
    const int64_t runs = (batch + kSampleRun - 1) / kSampleRun;
    const int64_t work = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (work >= runs * sp.n_chunks) return;
    const int64_t c = work / runs;
    const int64_t b0 = (work - c * runs) * kSampleRun;
    const int64_t b1 = min(batch, b0 + kSampleRun);
    const ChunkStatic cs = load_chunk(sp, c);
    if (cs.P <= 8)
        chunk_backward<8, DO_DX, DO_DW, INT_DW>(sp, cs, W, dY, anchors, idx, min_delta, min_k, dX, target_arr, b0, b1, n_inputs, n_outputs, n_detectors, n_anchors, lane, lr, fixed_scale);
    else if (cs.P <= 16)
        chunk_backward<16, DO_DX, DO_DW, INT_DW>(sp, cs, W, dY, anchors, idx, min_delta, min_k, dX, target_arr, b0, b1, n_inputs, n_outputs, n_detectors, n_anchors, lane, lr, fixed_scale);
    else
        chunk_backward<32, DO_DX, DO_DW, INT_DW>(sp, cs, W, dY, anchors, idx, min_delta, min_k, dX, target_arr, b0, b1, n_inputs, n_outputs, n_detectors, n_anchors, lane, lr, fixed_scale);
}

// --------------------------------------------------------------------------------------------
// Table gradient alone over a range of chunks, table indices of 1, 2 or 4 bytes.  For data-parallel ranks
// that own a share of the detectors: every rank gathers the (index, output gradient) pairs of the whole
// batch - one byte per (sample, detector) for 256-row tables, against a dense gradient as large as the
// tables - and applies the update of all samples to its own share.  Same reductions as the DO_DW pass of
// chunk_backward.
// --------------------------------------------------------------------------------------------
template <int LG, typename IdxT>
__device__ __forceinline__ void chunk_table_grad(const SparseView &sp, const ChunkStatic &cs,
                                                 const float *__restrict__ dY, const IdxT *__restrict__ idx,
                                                 float *__restrict__ target_arr, int64_t b0, int64_t b1,
                                                 int n_outputs, int n_detectors, int lane, double lr) {
    constexpr int NG = 32 / LG;
    const int g = lane / LG, j = lane - g * LG;
    const bool valid = j < cs.P;
    const bool has_det = lane < cs.ndet;
    const int my_target = valid ? __ldg(sp.syn_target + cs.toff + j) : 0;
    float *Tb = target_arr + cs.wbase0 + j + hole_offset(j, sp);
    const int64_t det_l = cs.det0 + lane;
    int32_t li_n = has_det ? (int32_t)__ldg(idx + b0 * n_detectors + det_l) : 0;
    float gp_n = valid ? __ldg(dY + b0 * n_outputs + my_target) : 0.f;
    for (int64_t b = b0; b < b1; b++) {
        const int32_t li = li_n;
        const float gp = gp_n;
        if (b + 1 < b1) {
            if (has_det) li_n = (int32_t)__ldg(idx + (b + 1) * n_detectors + det_l);
            if (valid) gp_n = __ldg(dY + (b + 1) * n_outputs + my_target);
        }
        const int32_t row_off = has_det ? lane * cs.table + li * cs.stride : 0;
        const bool active = valid && fabsf(gp) > kEpsF;
        const float val = lr == 1.0 ? gp : (float)((double)gp * lr);
        // every lane takes part in the offset broadcasts; only the reductions are predicated
#pragma unroll
        for (int i = 0; i < LG; i++) {
            const int d = i * NG + g;
            const int32_t ro = __shfl_sync(0xffffffffu, row_off, d);
            if (active && d < cs.ndet) atomicAdd(Tb + ro, val);
        }
    }
}

template <typename IdxT>
__global__ void __launch_bounds__(256, 4) sparse_table_grad_range_kernel(SparseView sp, const float *__restrict__ dY,
                                                                     const IdxT *__restrict__ idx,
                                                                     float *__restrict__ target_arr, int64_t batch,
                                                                     int n_outputs, int n_detectors, double lr,
                                                                     int64_t chunk_begin, int64_t n_range) {
    const int lane = threadIdx.x & 31;
    const int64_t runs = (batch + kSampleRun - 1) / kSampleRun;
    const int64_t work = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (work >= runs * n_range) return;
    const int64_t c = work / runs;
    const int64_t b0 = (work - c * runs) * kSampleRun;
    const int64_t b1 = min(batch, b0 + kSampleRun);
    const ChunkStatic cs = load_chunk(sp, chunk_begin + c);
    if (cs.P <= 8) chunk_table_grad<8, IdxT>(sp, cs, dY, idx, target_arr, b0, b1, n_outputs, n_detectors, lane, lr);
    else if (cs.P <= 16) chunk_table_grad<16, IdxT>(sp, cs, dY, idx, target_arr, b0, b1, n_outputs, n_detectors, lane, lr);
    else chunk_table_grad<32, IdxT>(sp, cs, dY, idx, target_arr, b0, b1, n_outputs, n_detectors, lane, lr);
}

// Generic fp32 backward for rows longer than 32 synapses: one warp per (sample, detector).
template <bool DO_DX, bool DO_DW, bool INT_DW>
__global__ void __launch_bounds__(256) sparse_backward_long_kernel(SparseView sp, const float *__restrict__ W,
                                                                  const float *__restrict__ dY,
                                                                  const int2 *__restrict__ anchors,
                                                                  const int32_t *__restrict__ idx,
                                                                  const float *__restrict__ min_delta,
                                                                  const int32_t *__restrict__ min_k,
                                                                  float *__restrict__ dX,
                                                                  float *__restrict__ target_arr, int64_t batch,
                                                                  int n_inputs, int n_outputs, int n_detectors,
                                                                  int n_anchors, double lr, double fixed_scale) {
    const int lane = threadIdx.x & 31;
    const int64_t work = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (work >= batch * n_detectors) return;
    const int t = (int)(work / batch);
    const int64_t b = work - (int64_t)t * batch;
    const int64_t bt = b * n_detectors + t;
    const int32_t li = __ldg(idx + bt);
    const int32_t k = DO_DX ? __ldg(min_k + bt) : 0;
    const int P = __ldg(sp.det_count + t);
    const int64_t wbase = __ldg(sp.det_wbase + t);
    const int stride = __ldg(sp.det_stride + t);
    const int32_t *tg = sp.syn_target + __ldg(sp.det_sstart + t);
    const int64_t row = wbase + (int64_t)li * stride;
    const int64_t alt = wbase + (int64_t)(li ^ (1 << k)) * stride;
    const float *dy = dY + b * n_outputs;
    double acc = 0.0;
    for (int p = lane; p < P; p += 32) {
        const int q = p + hole_offset(p, sp);
        const double gd = (double)__ldg(dy + __ldg(tg + p));
        if (DO_DX) acc += gd * ((double)__ldg(W + row + q) - (double)__ldg(W + alt + q));
        if (DO_DW && fabs(gd) > kEps) {
            if (INT_DW) atomicAdd(reinterpret_cast<int32_t *>(target_arr) + row + q, to_fixed(gd * lr, fixed_scale));
            else atomicAdd(target_arr + row + q, (float)(gd * lr));
        }
    }
    if (!DO_DX) return;
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) {
        const double du = surrogate_up(__ldg(min_delta + bt)) * acc;
        if (fabs(du) > kEps) {
            const int2 a = __ldg(anchors + (size_t)t * n_anchors + k);
            atomicAdd(dX + b * n_inputs + a.x, (float)du);
            atomicAdd(dX + b * n_inputs + a.y, -(float)du);
        }
    }
}

// Fixed-point variant: one thread per (sample, detector) walks the synapse groups in order; each group's
// du is truncated on its own (bit-exact with the reference), integer atomics make the order irrelevant.
__global__ void sparse_input_grad_fixed_kernel(SparseView sp, const float *__restrict__ W, const float *__restrict__ dY,
                                               const int2 *__restrict__ anchors, const int32_t *__restrict__ idx,
                                               const float *__restrict__ min_delta, const int32_t *__restrict__ min_k,
                                               float *__restrict__ dX, int64_t batch, int n_inputs, int n_outputs,
                                               int n_detectors, int n_anchors, double fixed_scale) {
    const int64_t total = batch * n_detectors;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / n_detectors;
        const int t = (int)(i - b * n_detectors);
        const int32_t li = idx[i];
        const int32_t k = min_k[i];
        const double up = surrogate_up(min_delta[i]);
        const int P = sp.det_count[t];
        const int64_t wbase = sp.det_wbase[t];
        const int stride = sp.det_stride[t];
        const int32_t *tg = sp.syn_target + sp.det_sstart[t];
        const float *row = W + wbase + (int64_t)li * stride;
        const float *alt = W + wbase + (int64_t)(li ^ (1 << k)) * stride;
        const float *dy = dY + b * n_outputs;
        const int2 a = __ldg(anchors + (size_t)t * n_anchors + k);
        int32_t *dx = reinterpret_cast<int32_t *>(dX) + b * n_inputs;
        for (int p0 = 0; p0 < P; p0 += sp.group) {
            const int p1 = min(p0 + sp.group, P);
            double ms = 0.0, as = 0.0;
            for (int p = p0; p < p1; p++) ms += (double)__ldg(row + p + hole_offset(p, sp)) * (double)__ldg(dy + tg[p]);
            for (int p = p0; p < p1; p++) as += (double)__ldg(alt + p + hole_offset(p, sp)) * (double)__ldg(dy + tg[p]);
            const double du = up * (ms - as);
            if (fabs(du) > kEps) {
                const int32_t d = to_fixed(du, fixed_scale);
                atomicAdd(dx + a.x, d);
                atomicAdd(dx + a.y, -d);
            }
        }
    }
}

// Kernel family of the forward pass and of the input-gradient pass, chosen independently: the library's choice, or
// forced by lutb_sparse_kernel_select / the LUTB_SPARSE_KERNELS environment variable
// ("<forward>,<input gradient>" or one word for both; auto, gather, staged).
static std::atomic<int> g_sparse_kernels[2] = {{-1}, {-1}};

static int parse_kernels(const char *word, size_t len) {
    if (len == 6 && !strncmp(word, "gather", 6)) return LUTB_SPARSE_GATHER;
    if (len == 6 && !strncmp(word, "staged", 6)) return LUTB_SPARSE_STAGED;
    return LUTB_SPARSE_AUTO;
}

static int sparse_kernels(int pass) {
    int v = g_sparse_kernels[pass].load(std::memory_order_relaxed);
    if (v >= 0) return v;
    int both[2] = {LUTB_SPARSE_AUTO, LUTB_SPARSE_AUTO};
    if (const char *e = getenv("LUTB_SPARSE_KERNELS")) {
        const char *comma = strchr(e, ',');
        both[0] = parse_kernels(e, comma ? (size_t)(comma - e) : strlen(e));
        both[1] = comma ? parse_kernels(comma + 1, strlen(comma + 1)) : both[0];
    }
    for (int i = 0; i < 2; i++) {
        int expected = -1;
        g_sparse_kernels[i].compare_exchange_strong(expected, both[i]);
    }
    return g_sparse_kernels[pass].load(std::memory_order_relaxed);
}

// 1: run the staged kernel, 0: the gather kernel, < 0: staged was forced but cannot run this layer.
// pass 0 = forward, 1 = input gradient.
static int use_staged(int pass, const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch, const float *weights) {
    const int v = sparse_kernels(pass);
    if (v == LUTB_SPARSE_GATHER) return 0;
    const bool possible = sparse_staged_possible(cfg, sp, weights);
    if (v == LUTB_SPARSE_STAGED) {
        LUTB_REQUIRE(possible, LUTB_ERR_MODE,
                     "the staged sparse kernels need fp32 accumulators, rows of at most 32 synapses and 16-byte aligned "
                     "detector tables of which three fit shared memory");
        return 1;
    }
    return possible && sparse_staged_preferred(pass, cfg, sp, batch) ? 1 : 0;
}

static int validate_sparse(const lutb_sparse_index *sp) {
    LUTB_REQUIRE(sp != nullptr, LUTB_ERR_NULL, "sparse index is NULL");
    LUTB_REQUIRE(sp->det_wbase && sp->det_stride && sp->det_count && sp->det_sstart && sp->syn_det && sp->syn_target &&
                     sp->chunk_info,
                 LUTB_ERR_NULL, "a sparse index array is NULL");
    LUTB_REQUIRE(sp->group_size > 0 && sp->n_syn_per_sample > 0 && sp->n_weights > 0 && sp->max_count > 0 &&
                     sp->n_chunks > 0,
                 LUTB_ERR_SHAPE, "empty sparse index");
    LUTB_REQUIRE((reinterpret_cast<uintptr_t>(sp->chunk_info) & 31) == 0, LUTB_ERR_ALIGN,
                 "chunk_info must be 32-byte aligned");
    return LUTB_OK;
}

static int chunk_grid(int64_t items, unsigned *blocks) {
    const int64_t n = (items + 7) / 8;  // 8 warps per block
    LUTB_REQUIRE(n <= 0x7FFFFFFF, LUTB_ERR_SHAPE, "batch too large for one launch");
    *blocks = (unsigned)n;
    return LUTB_OK;
}

}  // namespace lutb

using namespace lutb;

extern "C" int lutb_sparse_kernel_select(int forward_kernels, int input_grad_kernels) {
    for (int k : {forward_kernels, input_grad_kernels})
        LUTB_REQUIRE(k == LUTB_SPARSE_AUTO || k == LUTB_SPARSE_GATHER || k == LUTB_SPARSE_STAGED, LUTB_ERR_MODE,
                     "kernels must be LUTB_SPARSE_AUTO, LUTB_SPARSE_GATHER or LUTB_SPARSE_STAGED");
    g_sparse_kernels[0].store(forward_kernels);
    g_sparse_kernels[1].store(input_grad_kernels);
    return LUTB_OK;
}

extern "C" int lutb_nonseq_sparse_forward(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                                          const float *weights, const float *x, const int32_t *anchors, float *y,
                                          int32_t *idx, float *min_delta, int32_t *min_k, void *stream) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    rc = validate_sparse(sp);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->seq_len == 1, LUTB_ERR_MODE, "forward_step should only be called when sequence_length == 1");
    LUTB_REQUIRE(batch > 0 && batch <= 0x7FFFFFFF, LUTB_ERR_SHAPE, "batch_size == 0 or too large");
    LUTB_REQUIRE(weights && x && anchors && y && idx, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE((min_delta == nullptr) == (min_k == nullptr), LUTB_ERR_MODE,
                 "min_anchor_deltas and min_anchor_delta_indices must be given together");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = launch_check_detectors(x, batch, cfg->n_inputs, anchors, cfg->n_detectors, cfg->n_anchors, cfg->cmp_eps, idx,
                                min_delta, min_k, st);
    if (rc) return rc;
    const int staged = use_staged(0, cfg, sp, batch, weights);
    if (staged < 0) return staged;
    if (staged) return launch_sparse_forward_staged(cfg, sp, batch, weights, idx, y, st);
    SparseView v = make_view(sp);
    unsigned blocks;
    rc = chunk_grid(((batch + kSampleRun - 1) / kSampleRun) * sp->n_chunks, &blocks);
    if (rc) return rc;
    {
        KernelScope scope(K_SPARSE_FORWARD, st);
        if (cfg->int_mode)
            sparse_forward_kernel<true><<<blocks, 256, 0, st>>>(v, weights, idx, y, batch, cfg->n_outputs, cfg->n_detectors, cfg->int_rescaler);
        else
            sparse_forward_kernel<false><<<blocks, 256, 0, st>>>(v, weights, idx, y, batch, cfg->n_outputs, cfg->n_detectors, cfg->int_rescaler);
    }
    LUTB_LAUNCH_CHECK();
    if (cfg->int_mode) return launch_fixed_to_float(y, batch * (int64_t)cfg->n_outputs, cfg->int_rescaler, st);
    return LUTB_OK;
}

extern "C" int lutb_nonseq_sparse_backward(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                                           float *weights, const float *dY, const int32_t *anchors,
                                           const int32_t *idx, const float *min_delta, const int32_t *min_k,
                                           float *dX, float *dW, double external_lr, void *stream) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    rc = validate_sparse(sp);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->seq_len == 1, LUTB_ERR_MODE, "backward_backprop should only be called when sequence_length == 1");
    LUTB_REQUIRE(batch > 0 && batch <= 0x7FFFFFFF, LUTB_ERR_SHAPE, "batch_size == 0 or too large");
    LUTB_REQUIRE(weights && dY && anchors && idx && min_delta && min_k, LUTB_ERR_NULL,
                 "a required tensor pointer is NULL");
    LUTB_REQUIRE(!(external_lr >= 0.0 && dW != nullptr), LUTB_ERR_MODE,
                 "in internal weight gradients mode w_weights_gradients should be nullptr");
    const bool skip_table = external_lr == LUTB_SKIP_TABLE_GRADIENT;
    LUTB_REQUIRE(!(skip_table && dW != nullptr), LUTB_ERR_MODE, "no table gradient asked for, w_weights_gradients should be nullptr");
    LUTB_REQUIRE(!(external_lr < 0.0 && dW == nullptr && !skip_table), LUTB_ERR_NULL, "w_weights_gradients is NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int sm = device_info().sm_count;
    SparseView v = make_view(sp);
    const int O = cfg->n_outputs, Nt = cfg->n_detectors;
    const int2 *an = reinterpret_cast<const int2 *>(anchors);
    double lr = cfg->lr_meta;
    if (external_lr >= 0.0) lr *= -(double)(float)external_lr;
    float *target = external_lr >= 0.0 ? weights : dW;
    const bool long_rows = sp->max_count > 32;
    unsigned blocks;
    rc = chunk_grid(long_rows ? batch * (int64_t)Nt : ((batch + kSampleRun - 1) / kSampleRun) * sp->n_chunks, &blocks);
    if (rc) return rc;
#define LUTB_SPARSE_BWD(DX, DWF, INTF)                                                                              \
    do {                                                                                                            \
        if (long_rows)                                                                                              \
            sparse_backward_long_kernel<DX, DWF, INTF><<<blocks, 256, 0, st>>>(v, weights, dY, an, idx, min_delta, min_k, dX, target, batch, cfg->n_inputs, O, Nt, cfg->n_anchors, lr, cfg->int_rescaler); \
        else                                                                                                        \
            sparse_backward_kernel<DX, DWF, INTF><<<blocks, 256, 0, st>>>(v, weights, dY, an, idx, min_delta, min_k, dX, target, batch, cfg->n_inputs, O, Nt, cfg->n_anchors, lr, cfg->int_rescaler); \
    } while (0)
    // Two passes.  The input gradient (row gathers, dX updates) and the table gradient (fire-and-forget reductions into
    // the selected rows) run faster one after the other than fused into one kernel (0.33 + 0.19 ms against 0.70 ms for the
    // three layers of the conv-net step): the reductions of the fused kernel queue in front of its own row gathers.  With
    // in-place SGD the order is also required: every sample must read the weights before any of them is modified.
    // dX == nullptr: the caller does not want the input gradient (first layer of a network).
    const int staged = dX != nullptr ? use_staged(1, cfg, sp, batch, weights) : 0;
    if (staged < 0) return staged;
    if (staged) {
        rc = launch_sparse_input_grad_staged(cfg, sp, batch, weights, dY, anchors, idx, min_delta, min_k, dX, st);
        if (rc) return rc;
    } else if (dX != nullptr) {
        KernelScope scope(K_SPARSE_INPUT_GRAD, st);
        if (cfg->int_mode) {
            const int64_t total = batch * Nt;
            const int64_t gblocks = min((total + 127) / 128, (int64_t)sm * 64);
            sparse_input_grad_fixed_kernel<<<(unsigned)gblocks, 128, 0, st>>>(v, weights, dY, an, idx, min_delta, min_k, dX, batch,
                                                                            cfg->n_inputs, O, Nt, cfg->n_anchors, cfg->int_rescaler);
        } else {
            LUTB_SPARSE_BWD(true, false, false);
        }
        LUTB_LAUNCH_CHECK();
    }
    if (!skip_table) {
        KernelScope scope(K_SPARSE_WEIGHT_GRAD, st);
        if (cfg->int_mode) LUTB_SPARSE_BWD(false, true, true);
        else LUTB_SPARSE_BWD(false, true, false);
    }
#undef LUTB_SPARSE_BWD
    LUTB_LAUNCH_CHECK();
    if (cfg->int_mode) {
        if (dX) rc = launch_fixed_to_float(dX, batch * (int64_t)cfg->n_inputs, cfg->int_rescaler, st);
        if (rc) return rc;
        if (dW) rc = launch_fixed_to_float(dW, sp->n_weights, cfg->int_rescaler, st);
    }
    return rc;
}

extern "C" int lutb_nonseq_sparse_table_grad(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                                             const float *dY, const void *idx, int idx_bytes, float *target,
                                             double scale, int64_t chunk_begin, int64_t chunk_end, void *stream) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    rc = validate_sparse(sp);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->seq_len == 1, LUTB_ERR_MODE, "the table-gradient pass is for sequence_length == 1");
    LUTB_REQUIRE(cfg->int_mode == 0, LUTB_ERR_MODE, "the ranged table-gradient pass needs fp32 accumulators");
    LUTB_REQUIRE(sp->max_count <= 32, LUTB_ERR_MODE, "the ranged table-gradient pass supports rows of at most 32 synapses");
    LUTB_REQUIRE(batch > 0 && batch <= 0x7FFFFFFF, LUTB_ERR_SHAPE, "batch_size == 0 or too large");
    LUTB_REQUIRE(dY && idx && target, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE(idx_bytes == 1 || idx_bytes == 2 || idx_bytes == 4, LUTB_ERR_MODE, "idx_bytes must be 1, 2 or 4");
    LUTB_REQUIRE(idx_bytes == 4 || cfg->n_anchors <= 8 * idx_bytes, LUTB_ERR_MODE,
                 "table indices of 2^%d rows do not fit %d byte(s)", cfg->n_anchors, idx_bytes);
    LUTB_REQUIRE(chunk_begin >= 0 && chunk_begin <= chunk_end && chunk_end <= sp->n_chunks, LUTB_ERR_SHAPE,
                 "chunk range [%lld, %lld) outside [0, %lld)", (long long)chunk_begin, (long long)chunk_end,
                 (long long)sp->n_chunks);
    if (chunk_begin == chunk_end) return LUTB_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SparseView v = make_view(sp);
    const int64_t n_range = chunk_end - chunk_begin;
    unsigned blocks;
    rc = chunk_grid(((batch + kSampleRun - 1) / kSampleRun) * n_range, &blocks);
    if (rc) return rc;
    const double lr = cfg->lr_meta * scale;
    const int O = cfg->n_outputs, Nt = cfg->n_detectors;
    KernelScope scope(K_SPARSE_WEIGHT_GRAD, st);
    if (idx_bytes == 1)
        sparse_table_grad_range_kernel<uint8_t><<<blocks, 256, 0, st>>>(v, dY, static_cast<const uint8_t *>(idx), target, batch, O, Nt, lr, chunk_begin, n_range);
    else if (idx_bytes == 2)
        sparse_table_grad_range_kernel<uint16_t><<<blocks, 256, 0, st>>>(v, dY, static_cast<const uint16_t *>(idx), target, batch, O, Nt, lr, chunk_begin, n_range);
    else
        sparse_table_grad_range_kernel<int32_t><<<blocks, 256, 0, st>>>(v, dY, static_cast<const int32_t *>(idx), target, batch, O, Nt, lr, chunk_begin, n_range);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}
