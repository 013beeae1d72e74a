// Concatenation-mode sequence (attention) layer.  Every token has its own table index (anchor
// comparison over the B*S token rows, the non-sequence kernel), every (distance, detector) a positional
// index; a causal pair (i < j) selects row (Q_j << (Nc + Npe)) | (K_i << Npe) | PE_{j-i-1} of a table
// with 2^(2Nc+Npe) rows.
//
// Reference: check_positional_embeddings[_eval]_logic (lut_runtime_kernels_logic.proto:1709-1805),
// fill_outputs_fully_connected_seq_logic (:1807-1904), propagate_through_detectors_seq_fc_logic
// (:3629-3835), gather_w_gradients_seq_fc_cpu_logic (:3944-4044).
#include "lutb_common.cuh"
#include "nonseq_fc.cuh"

namespace lutb {

// sign bits of pe[d][t][:], first minimal |value| and its dimension
template <bool TRAIN>
__global__ void check_positional_kernel(const float *__restrict__ pe, int64_t n_items, int npe, float cmp_eps,
                                        int32_t *__restrict__ pidx, float *__restrict__ pmin,
                                        int32_t *__restrict__ pmin_k) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_items) return;
    const float *p = pe + i * npe;
    int32_t li = 0, mk = -1;
    float md = 0.f;
    for (int d = 0; d < npe; d++) {
        const float v = __ldg(p + d);
        if (greater_than_zero(v, cmp_eps)) li |= (1 << d);
        if (TRAIN && (mk == -1 || fabsf(v) < fabsf(md))) { md = v; mk = d; }
    }
    pidx[i] = li;
    if (TRAIN) { pmin[i] = md; pmin_k[i] = mk; }
}

__device__ __forceinline__ size_t concat_row(int32_t Q, int32_t K, int32_t PE, int nc, int npe) {
    return (size_t)(((uint32_t)Q << (nc + npe)) | ((uint32_t)K << npe) | (uint32_t)PE);
}

// --------------------------------------------------------------------------------------------
// Forward.  Block = (detector, sample): the sample's token indices of this detector and the detector's
// positional indices are staged in shared memory; each warp takes queries j round-robin and, with the
// lanes over the outputs, adds the rows of all keys i < j (coalesced 16-byte loads).  fp32 mode sums in
// fp32; fixed-point mode sums each (query, detector, output) in double in key order and truncates once,
// exactly as the reference does.
// --------------------------------------------------------------------------------------------
template <bool INT_MODE>
__global__ void __launch_bounds__(256) concat_forward_kernel(const float *__restrict__ W, const int32_t *__restrict__ idx,
                                                            const int32_t *__restrict__ pidx, float *__restrict__ y,
                                                            int S, int n_outputs, int n_detectors, int nc, int npe,
                                                            double fixed_scale, int j_begin, int j_end) {
    extern __shared__ __align__(16) int32_t ismem[];
    const int t = blockIdx.x;
    const int64_t b = blockIdx.y;
    int32_t *Ks = ismem;          // [S]
    int32_t *Ps = ismem + S;      // [S-1]
    for (int s = threadIdx.x; s < S; s += blockDim.x) Ks[s] = __ldg(idx + ((size_t)b * S + s) * n_detectors + t);
    for (int d = threadIdx.x; d < S - 1; d += blockDim.x) Ps[d] = npe > 0 ? __ldg(pidx + (size_t)d * n_detectors + t) : 0;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const size_t rows = (size_t)1 << (2 * nc + npe);
    const float *Wt = W + (size_t)t * rows * n_outputs;
    const bool vec4 = (n_outputs % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
    // queries [j_begin, j_end): the whole sequence, or one rank's share when the queries are sharded
    for (int j = max(1, j_begin) + warp; j < j_end; j += nwarps) {
        const int32_t Q = Ks[j];
        float *yj = y + ((size_t)b * S + j) * n_outputs;
        if (vec4) {
            for (int col = lane * 4; col < n_outputs; col += 128) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                double dacc[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll 4
                for (int i = 0; i < j; i++) {
                    const float4 w = __ldg(reinterpret_cast<const float4 *>(Wt + concat_row(Q, Ks[i], Ps[j - i - 1], nc, npe) * n_outputs + col));
                    if (INT_MODE) { dacc[0] += (double)w.x; dacc[1] += (double)w.y; dacc[2] += (double)w.z; dacc[3] += (double)w.w; }
                    else { acc[0] += w.x; acc[1] += w.y; acc[2] += w.z; acc[3] += w.w; }
                }
                if (INT_MODE) {
#pragma unroll
                    for (int e = 0; e < 4; e++) atomicAdd(reinterpret_cast<int32_t *>(yj) + col + e, to_fixed(dacc[e], fixed_scale));
                } else {
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(yj + col), "f"(acc[0]), "f"(acc[1]),
                                 "f"(acc[2]), "f"(acc[3]) : "memory");
                }
            }
        } else {
            for (int o = lane; o < n_outputs; o += 32) {
                float acc = 0.f;
                double dacc = 0.0;
                for (int i = 0; i < j; i++) {
                    const float w = __ldg(Wt + concat_row(Q, Ks[i], Ps[j - i - 1], nc, npe) * n_outputs + o);
                    if (INT_MODE) dacc += (double)w;
                    else acc += w;
                }
                if (INT_MODE) atomicAdd(reinterpret_cast<int32_t *>(yj) + o, to_fixed(dacc, fixed_scale));
                else atomicAdd(yj + o, acc);
            }
        }
    }
}

// --------------------------------------------------------------------------------------------
// Backward, fp32 accumulators.  Block = (detector, sample), a warp per query j, lanes over 32 keys at a
// time.  Per pair the side (query or key) with the smaller |min delta| is flipped; g = sum_o dY[b,j,o] *
// (W[row,o] - W[alt,o]) with the lanes over the outputs, transpose-reduced so that lane l ends with pair
// i0 + l, and du = up(delta) * g goes to the flipped token's two anchor inputs.  When the positional
// margin is the strictly smallest of the three, the positional embedding receives its own gradient from a
// second pass with the positional bit flipped.  The table gradient adds lr * dY[b,j,:] to the pair's row.
// --------------------------------------------------------------------------------------------
template <bool DO_DX, bool DO_DW>
__global__ void __launch_bounds__(256) concat_backward_kernel(const float *__restrict__ W, const float *__restrict__ dY,
                                                             const int2 *__restrict__ anchors,
                                                             const int32_t *__restrict__ idx,
                                                             const float *__restrict__ min_delta,
                                                             const int32_t *__restrict__ min_k,
                                                             const int32_t *__restrict__ pidx,
                                                             const float *__restrict__ pmin,
                                                             const int32_t *__restrict__ pmin_k, float *__restrict__ dX,
                                                             float *__restrict__ dPE, float *__restrict__ target, int S,
                                                             int n_inputs, int n_outputs, int n_detectors, int nc, int npe,
                                                             double lr, int j_begin, int j_end) {
    extern __shared__ __align__(16) int32_t ismem[];
    const int t = blockIdx.x;
    const int64_t b = blockIdx.y;
    int32_t *Ks = ismem;                                         // [S] token index
    int32_t *Kk = Ks + S;                                        // [S] token min-margin pair
    float *Km = reinterpret_cast<float *>(Kk + S);               // [S] token min margin
    int32_t *Ps = reinterpret_cast<int32_t *>(Km + S);           // [S] positional index (S-1 used)
    int32_t *Pk = Ps + S;                                        // [S]
    float *Pm = reinterpret_cast<float *>(Pk + S);               // [S]
    const int o_pad = (n_outputs + 3) & ~3;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    float *dy_s = reinterpret_cast<float *>(ismem) + ((6 * S + 3) & ~3) + warp * o_pad;
    for (int s = threadIdx.x; s < S; s += blockDim.x) {
        const size_t o = ((size_t)b * S + s) * n_detectors + t;
        Ks[s] = __ldg(idx + o); Kk[s] = __ldg(min_k + o); Km[s] = __ldg(min_delta + o);
    }
    for (int d = threadIdx.x; d < S - 1; d += blockDim.x) {
        const size_t o = (size_t)d * n_detectors + t;
        Ps[d] = npe > 0 ? __ldg(pidx + o) : 0;
        Pk[d] = npe > 0 ? __ldg(pmin_k + o) : -1;
        Pm[d] = npe > 0 ? __ldg(pmin + o) : 0.f;
    }
    __syncthreads();
    const size_t rows = (size_t)1 << (2 * nc + npe);
    const float *Wt = W + (size_t)t * rows * n_outputs;
    float *Tt = DO_DW ? target + (size_t)t * rows * n_outputs : nullptr;
    const bool vec4 = (n_outputs % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(target) & 15) == 0);
    for (int j = max(1, j_begin) + warp; j < j_end; j += nwarps) {
        const float *dyj = dY + ((size_t)b * S + j) * n_outputs;
        for (int o = lane; o < o_pad; o += 32) dy_s[o] = o < n_outputs ? __ldg(dyj + o) : 0.f;
        __syncwarp();
        const int32_t Q = Ks[j], qk = Kk[j];
        const float qm = Km[j];
        for (int i0 = 0; i0 < j; i0 += 32) {
            const int i = i0 + lane;
            // this lane's pair
            size_t my_row = 0, my_alt = 0, my_palt = 0;
            float my_m = 0.f;
            int my_flip = 0, my_pos = 0;
            bool my_pe = false;
            if (i < j) {
                const int32_t K = Ks[i], PEi = Ps[j - i - 1];
                const float km = Km[i], pm = Pm[j - i - 1];
                my_row = concat_row(Q, K, PEi, nc, npe);
                if (fabsf(qm) < fabsf(km)) { my_alt = concat_row(Q ^ (1 << qk), K, PEi, nc, npe); my_m = qm; my_flip = qk; my_pos = j; }
                else { my_alt = concat_row(Q, K ^ (1 << Kk[i]), PEi, nc, npe); my_m = km; my_flip = Kk[i]; my_pos = i; }
                if (npe > 0 && fabsf(pm) < fabsf(qm) && fabsf(pm) < fabsf(km)) {
                    my_pe = true;
                    my_palt = concat_row(Q, K, PEi ^ (1 << Pk[j - i - 1]), nc, npe);
                }
            }
            const int npairs = min(32, j - i0);
            const unsigned pe_mask = __ballot_sync(0xffffffffu, my_pe);
            for (int pass = 0; pass < 2; pass++) {
                if (pass == 1 && (!DO_DX || pe_mask == 0)) break;
                float v[32];
#pragma unroll
                for (int p = 0; p < 32; p++) {
                    v[p] = 0.f;
                    if (p < npairs) {  // warp-uniform
                        const size_t r0 = __shfl_sync(0xffffffffu, (unsigned long long)my_row, p);
                        const size_t r1 = __shfl_sync(0xffffffffu, (unsigned long long)(pass == 0 ? my_alt : my_palt), p);
                        const bool need = pass == 0 ? true : ((pe_mask >> p) & 1u);
                        const float *row = Wt + r0 * n_outputs;
                        const float *alt = Wt + r1 * n_outputs;
                        float part = 0.f;
                        if (vec4) {
                            for (int col = lane * 4; col < n_outputs; col += 128) {
                                const float4 g = *reinterpret_cast<const float4 *>(dy_s + col);
                                if (DO_DX && need) {
                                    const float4 a = __ldg(reinterpret_cast<const float4 *>(row + col));
                                    const float4 c = __ldg(reinterpret_cast<const float4 *>(alt + col));
                                    part += g.x * (a.x - c.x) + g.y * (a.y - c.y) + g.z * (a.z - c.z) + g.w * (a.w - c.w);
                                }
                                if (DO_DW && pass == 0) {
                                    float4 u = g;   // lr == 1: the product is dY itself
                                    if (lr != 1.0) {
                                        u.x = (float)((double)g.x * lr); u.y = (float)((double)g.y * lr);
                                        u.z = (float)((double)g.z * lr); u.w = (float)((double)g.w * lr);
                                    }
                                    u.x = fabsf(g.x) > kEpsF ? u.x : 0.f;
                                    u.y = fabsf(g.y) > kEpsF ? u.y : 0.f;
                                    u.z = fabsf(g.z) > kEpsF ? u.z : 0.f;
                                    u.w = fabsf(g.w) > kEpsF ? u.w : 0.f;
                                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(Tt + r0 * n_outputs + col),
                                                 "f"(u.x), "f"(u.y), "f"(u.z), "f"(u.w) : "memory");
                                }
                            }
                        } else {
                            for (int o = lane; o < n_outputs; o += 32) {
                                const float g = dy_s[o];
                                if (DO_DX && need) part += g * (__ldg(row + o) - __ldg(alt + o));
                                if (DO_DW && pass == 0 && fabs((double)g) > kEps) atomicAdd(Tt + r0 * n_outputs + o, (float)((double)g * lr));
                            }
                        }
                        v[p] = part;
                    }
                }
                if (!DO_DX) break;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) {
                    const bool upper = (lane & o) != 0;
#pragma unroll
                    for (int p = 0; p < o; p++) {
                        const float send = upper ? v[p] : v[p + o];
                        const float keep = upper ? v[p + o] : v[p];
                        v[p] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                    }
                }
                if (i < j) {
                    if (pass == 0) {
                        const double du = surrogate_up(my_m) * (double)v[0];
                        if (fabs(du) > kEps) {
                            const int2 a = __ldg(anchors + (size_t)t * nc + my_flip);
                            float *dx = dX + ((size_t)b * S + my_pos) * n_inputs;
                            atomicAdd(dx + a.x, (float)du);
                            atomicAdd(dx + a.y, -(float)du);
                        }
                    } else if (my_pe) {
                        const int d = j - i - 1;
                        const double dp = surrogate_up(Pm[d]) * (double)v[0];
                        atomicAdd(dPE + ((size_t)d * n_detectors + t) * npe + Pk[d], (float)dp);
                    }
                }
            }
        }
        __syncwarp();
    }
}

// Fixed-point backward: one thread per (sample, query, detector, key, output block) walks the block's
// outputs in order in double like the reference's host loop; contributions are truncated to int32 and
// added with integer atomics (order independent).
__global__ void concat_backward_fixed_kernel(const float *__restrict__ W, const float *__restrict__ dY,
                                             const int2 *__restrict__ anchors, const int32_t *__restrict__ idx,
                                             const float *__restrict__ min_delta, const int32_t *__restrict__ min_k,
                                             const int32_t *__restrict__ pidx, const float *__restrict__ pmin,
                                             const int32_t *__restrict__ pmin_k, float *__restrict__ dX,
                                             float *__restrict__ dPE, float *__restrict__ dW, int64_t batch, int S,
                                             int n_inputs, int n_outputs, int n_detectors, int nc, int npe, int out_block,
                                             double lr, double fixed_scale) {
    const int n_ob = (n_outputs + out_block - 1) / out_block;
    const int64_t total = batch * S * (int64_t)n_detectors * S * n_ob;
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
        const int ob = (int)(w % n_ob);
        int64_t r = w / n_ob;
        const int i = (int)(r % S); r /= S;
        const int t = (int)(r % n_detectors); r /= n_detectors;
        const int j = (int)(r % S);
        const int64_t b = r / S;
        if (i >= j) continue;
        const int o0 = ob * out_block, o1 = min(n_outputs, o0 + out_block);
        const size_t ko = ((size_t)b * S + i) * n_detectors + t, qo = ((size_t)b * S + j) * n_detectors + t;
        const int32_t K = idx[ko], Q = idx[qo];
        const float km = min_delta[ko], qm = min_delta[qo];
        const size_t po = (size_t)(j - i - 1) * n_detectors + t;
        int32_t PE = 0, pk = -1;
        float pm = 0.f;
        if (npe > 0) { PE = pidx[po]; pk = pmin_k[po]; pm = pmin[po]; }
        const size_t rows = (size_t)1 << (2 * nc + npe);
        const float *Wt = W + (size_t)t * rows * n_outputs;
        const size_t row = concat_row(Q, K, PE, nc, npe);
        size_t alt;
        float m;
        int flip, pos;
        if (fabsf(qm) < fabsf(km)) { alt = concat_row(Q ^ (1 << min_k[qo]), K, PE, nc, npe); m = qm; flip = min_k[qo]; pos = j; }
        else { alt = concat_row(Q, K ^ (1 << min_k[ko]), PE, nc, npe); m = km; flip = min_k[ko]; pos = i; }
        const float *dy = dY + ((size_t)b * S + j) * n_outputs;
        double ms = 0.0, as = 0.0;
        for (int o = o0; o < o1; o++) {
            const double g = (double)__ldg(dy + o);
            ms += (double)__ldg(Wt + row * n_outputs + o) * g;
            as += (double)__ldg(Wt + alt * n_outputs + o) * g;
        }
        const double du = surrogate_up(m) * (ms - as);
        if (fabs(du) > kEps) {
            const int2 a = __ldg(anchors + (size_t)t * nc + flip);
            int32_t *dx = reinterpret_cast<int32_t *>(dX) + ((size_t)b * S + pos) * n_inputs;
            const int32_t d = to_fixed(du, fixed_scale);
            atomicAdd(dx + a.x, d);
            atomicAdd(dx + a.y, -d);
        }
        if (npe > 0 && fabsf(pm) < fabsf(qm) && fabsf(pm) < fabsf(km)) {
            const size_t palt = concat_row(Q, K, PE ^ (1 << pk), nc, npe);
            double ps = 0.0;
            for (int o = o0; o < o1; o++) ps += (double)__ldg(Wt + palt * n_outputs + o) * (double)__ldg(dy + o);
            const double dp = surrogate_up(pm) * (ms - ps);
            atomicAdd(reinterpret_cast<int32_t *>(dPE) + po * npe + pk, to_fixed(dp, fixed_scale));
        }
        if (dW) {
            int32_t *drow = reinterpret_cast<int32_t *>(dW) + ((size_t)t * rows + row) * n_outputs;
            for (int o = o0; o < o1; o++) {
                const double g = (double)__ldg(dy + o);
                if (fabs(g) > kEps) atomicAdd(drow + o, to_fixed(g * lr, fixed_scale));
            }
        }
    }
}

// --------------------------------------------------------------------------------------------
// Concatenation-mode layers with sparse lookup -> output connectivity (reference: fill_outputs_sparse_seq_logic,
// proto:1906-2013; propagate_through_detectors_seq_sparse_logic, :3371-3627; gather_w_gradients_seq_sparse_logic,
// :3837-3942).  A causal pair selects lookup neuron (t, row(i, j)) as in the fully connected case; that neuron's
// synapses (slot p + 2 * (p / G) behind the row base, targets shared by all rows of the detector) are walked as in
// the non-sequence sparse layer.  One thread per (sample, query, detector, key): sums in double per synapse group
// (every group issues its own contribution, as the reference does with one block per group), fp32 or int32
// fixed-point atomics.  No layer of the benchmark configurations takes this path; it is written for exactness.
// --------------------------------------------------------------------------------------------
struct SparseRows {
    const int64_t *wbase;
    const int32_t *stride, *count, *sstart, *target;
    int group;
};

__device__ __forceinline__ int64_t sparse_slot(int64_t row_base, int p, int G) { return row_base + p + 2 * (p / G); }

template <bool INT_MODE>
__global__ void concat_sparse_forward_kernel(const float *__restrict__ W, const int32_t *__restrict__ idx,
                                             const int32_t *__restrict__ pidx, float *__restrict__ y, SparseRows sp,
                                             int64_t batch, int S, int n_outputs, int n_detectors, int nc, int npe,
                                             double fixed_scale) {
    const int64_t total = batch * S * (int64_t)n_detectors * S;
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)(w % S);
        int64_t r = w / S;
        const int t = (int)(r % n_detectors);
        r /= n_detectors;
        const int j = (int)(r % S);
        const int64_t b = r / S;
        if (i >= j) continue;
        const int32_t K = idx[(b * S + i) * n_detectors + t], Q = idx[(b * S + j) * n_detectors + t];
        const int32_t PE = npe > 0 ? pidx[(int64_t)(j - i - 1) * n_detectors + t] : 0;
        const int64_t row = sp.wbase[t] + (int64_t)concat_row(Q, K, PE, nc, npe) * sp.stride[t];
        const int32_t *tg = sp.target + sp.sstart[t];
        float *yb = y + (b * S + j) * n_outputs;
        const int P = sp.count[t];
        for (int p = 0; p < P; p++) {
            const float wv = __ldg(W + sparse_slot(row, p, sp.group));
            if (INT_MODE) atomicAdd(reinterpret_cast<int32_t *>(yb) + tg[p], to_fixed((double)wv, fixed_scale));
            else atomicAdd(yb + tg[p], wv);
        }
    }
}

template <bool INT_MODE>
__global__ void concat_sparse_backward_kernel(const float *__restrict__ W, const float *__restrict__ dY,
                                              const int2 *__restrict__ anchors, const int32_t *__restrict__ idx,
                                              const float *__restrict__ min_delta, const int32_t *__restrict__ min_k,
                                              const int32_t *__restrict__ pidx, const float *__restrict__ pmin,
                                              const int32_t *__restrict__ pmin_k, float *__restrict__ dX,
                                              float *__restrict__ dPE, float *__restrict__ target, SparseRows sp,
                                              int64_t batch, int S, int n_inputs, int n_outputs, int n_detectors, int nc,
                                              int npe, int do_dx, double lr, double fixed_scale) {
    const int64_t total = batch * S * (int64_t)n_detectors * S;
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)(w % S);
        int64_t r = w / S;
        const int t = (int)(r % n_detectors);
        r /= n_detectors;
        const int j = (int)(r % S);
        const int64_t b = r / S;
        if (i >= j) continue;
        const int64_t ko = (b * S + i) * n_detectors + t, qo = (b * S + j) * n_detectors + t;
        const int32_t K = idx[ko], Q = idx[qo];
        const int64_t po = (int64_t)(j - i - 1) * n_detectors + t;
        int32_t PE = 0, pk = -1;
        float pm = 0.f;
        if (npe > 0) { PE = pidx[po]; pk = pmin_k[po]; pm = pmin[po]; }
        const int64_t base = sp.wbase[t];
        const int64_t stride = sp.stride[t];
        const int64_t row = base + (int64_t)concat_row(Q, K, PE, nc, npe) * stride;
        const int32_t *tg = sp.target + sp.sstart[t];
        const float *dy = dY + (b * S + j) * n_outputs;
        const int P = sp.count[t], G = sp.group;
        if (do_dx) {
            const float qm = min_delta[qo], km = min_delta[ko];
            int64_t alt;
            double up;
            int flip, pos;
            if (fabsf(qm) < fabsf(km)) {
                alt = base + (int64_t)concat_row(Q ^ (1 << min_k[qo]), K, PE, nc, npe) * stride;
                up = surrogate_up(qm); flip = min_k[qo]; pos = j;
            } else {
                alt = base + (int64_t)concat_row(Q, K ^ (1 << min_k[ko]), PE, nc, npe) * stride;
                up = surrogate_up(km); flip = min_k[ko]; pos = i;
            }
            const bool pe_flip = npe > 0 && fabsf(pm) < fabsf(qm) && fabsf(pm) < fabsf(km);
            const int64_t palt = pe_flip ? base + (int64_t)concat_row(Q, K, PE ^ (1 << pk), nc, npe) * stride : 0;
            const int2 a = __ldg(anchors + (size_t)t * nc + flip);
            float *dx = dX + (b * S + pos) * (int64_t)n_inputs;
            for (int p0 = 0; p0 < P; p0 += G) {
                const int p1 = min(P, p0 + G);
                double ms = 0.0, as = 0.0, ps = 0.0;
                for (int p = p0; p < p1; p++) ms += (double)__ldg(W + sparse_slot(row, p, G)) * (double)__ldg(dy + tg[p]);
                for (int p = p0; p < p1; p++) as += (double)__ldg(W + sparse_slot(alt, p, G)) * (double)__ldg(dy + tg[p]);
                const double du = up * (ms - as);
                if (fabs(du) > kEps) {
                    if (INT_MODE) {
                        const int32_t d = to_fixed(du, fixed_scale);
                        atomicAdd(reinterpret_cast<int32_t *>(dx) + a.x, d);
                        atomicAdd(reinterpret_cast<int32_t *>(dx) + a.y, -d);
                    } else {
                        atomicAdd(dx + a.x, (float)du);
                        atomicAdd(dx + a.y, -(float)du);
                    }
                }
                if (pe_flip) {
                    for (int p = p0; p < p1; p++) ps += (double)__ldg(W + sparse_slot(palt, p, G)) * (double)__ldg(dy + tg[p]);
                    const double dp = surrogate_up(pm) * (ms - ps);
                    if (INT_MODE) atomicAdd(reinterpret_cast<int32_t *>(dPE) + po * npe + pk, to_fixed(dp, fixed_scale));
                    else atomicAdd(dPE + po * npe + pk, (float)dp);
                }
            }
        }
        if (target) {
            for (int p = 0; p < P; p++) {
                const double g = (double)__ldg(dy + tg[p]);
                if (fabs(g) > kEps) {
                    const int64_t slot = sparse_slot(row, p, G);
                    if (INT_MODE) atomicAdd(reinterpret_cast<int32_t *>(target) + slot, to_fixed(g * lr, fixed_scale));
                    else atomicAdd(target + slot, (float)(g * lr));
                }
            }
        }
    }
}

static int validate_sparse_rows(const lutb_sparse_index *sp, SparseRows *out) {
    LUTB_REQUIRE(sp != nullptr, LUTB_ERR_NULL, "sparse index is NULL");
    LUTB_REQUIRE(sp->det_wbase && sp->det_stride && sp->det_count && sp->det_sstart && sp->syn_target, LUTB_ERR_NULL,
                 "a sparse index array is NULL");
    LUTB_REQUIRE(sp->group_size > 0 && sp->n_weights > 0, LUTB_ERR_SHAPE, "empty sparse index");
    out->wbase = sp->det_wbase; out->stride = sp->det_stride; out->count = sp->det_count;
    out->sstart = sp->det_sstart; out->target = sp->syn_target; out->group = sp->group_size;
    return LUTB_OK;
}

static int validate_concat(const lutb_layer_cfg *cfg, int64_t batch) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    LUTB_REQUIRE(batch > 0, LUTB_ERR_SHAPE, "batch_size == 0");
    LUTB_REQUIRE(batch <= 65535, LUTB_ERR_SHAPE, "batch_size > 65535 is not supported by the sequence kernels");
    LUTB_REQUIRE(cfg->seq_len > 1, LUTB_ERR_MODE, "forward_step_concat should only be called when sequence_length > 1");
    LUTB_REQUIRE(2 * cfg->n_anchors + cfg->pos_dim <= 30, LUTB_ERR_SHAPE, "more than 2^30 rows per detector");
    return LUTB_OK;
}

}  // namespace lutb

using namespace lutb;

static int launch_check_positional(const lutb_layer_cfg *cfg, const float *pos_embeddings, int32_t *pos_idx,
                                   float *pos_min_delta, int32_t *pos_min_k, cudaStream_t st) {
    const int64_t n = (int64_t)(cfg->seq_len - 1) * cfg->n_detectors;
    const bool train = pos_min_delta != nullptr;
    KernelScope scope(K_CHECK_POSITIONAL, st);
    if (train) check_positional_kernel<true><<<(unsigned)((n + 127) / 128), 128, 0, st>>>(pos_embeddings, n, cfg->pos_dim, cfg->cmp_eps, pos_idx, pos_min_delta, pos_min_k);
    else check_positional_kernel<false><<<(unsigned)((n + 127) / 128), 128, 0, st>>>(pos_embeddings, n, cfg->pos_dim, cfg->cmp_eps, pos_idx, nullptr, nullptr);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

static int launch_concat_pairs_forward(const lutb_layer_cfg *cfg, int64_t batch, const float *weights, const int32_t *idx,
                                       const int32_t *pos_idx, float *y, int j_begin, int j_end, cudaStream_t st) {
    const int S = cfg->seq_len, npe = cfg->pos_dim, Nt = cfg->n_detectors;
    const size_t smem = (size_t)(2 * S) * 4;
    LUTB_REQUIRE(smem <= (size_t)kMaxSmemPerBlock - 1024, LUTB_ERR_SHAPE, "sequence too long for the sequence kernels");
    dim3 grid((unsigned)Nt, (unsigned)batch);
    KernelScope scope(K_CONCAT_FORWARD, st);
    if (cfg->int_mode) {
        if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(concat_forward_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        concat_forward_kernel<true><<<grid, 256, smem, st>>>(weights, idx, pos_idx, y, S, cfg->n_outputs, Nt, cfg->n_anchors, npe, cfg->int_rescaler, j_begin, j_end);
    } else {
        if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(concat_forward_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        concat_forward_kernel<false><<<grid, 256, smem, st>>>(weights, idx, pos_idx, y, S, cfg->n_outputs, Nt, cfg->n_anchors, npe, cfg->int_rescaler, j_begin, j_end);
    }
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

// fp32 accumulators only
static int launch_concat_pairs_backward(const lutb_layer_cfg *cfg, int64_t batch, float *weights, const float *dY,
                                        const int32_t *anchors, const int32_t *idx, const float *min_delta,
                                        const int32_t *min_k, const int32_t *pos_idx, const float *pos_min_delta,
                                        const int32_t *pos_min_k, float *dX, float *dPE, float *dW, double external_lr,
                                        int j_begin, int j_end, cudaStream_t st) {
    const int S = cfg->seq_len, npe = cfg->pos_dim, Nt = cfg->n_detectors, O = cfg->n_outputs, Nc = cfg->n_anchors;
    double lr = cfg->lr_meta;
    if (external_lr >= 0.0) lr *= -(double)(float)external_lr;
    const int2 *an = reinterpret_cast<const int2 *>(anchors);
    const int warps = 8;
    const size_t smem = ((size_t)((6 * S + 3) & ~3) + (size_t)warps * ((O + 3) & ~3)) * 4;
    LUTB_REQUIRE(smem <= (size_t)kMaxSmemPerBlock - 1024, LUTB_ERR_SHAPE, "sequence too long for the sequence kernels");
    dim3 grid((unsigned)Nt, (unsigned)batch);
#define LUTB_CONCAT_BWD(DX, DWF, TARGET)                                                                                  \
    do {                                                                                                                  \
        if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(concat_backward_kernel<DX, DWF>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        concat_backward_kernel<DX, DWF><<<grid, warps * 32, smem, st>>>(weights, dY, an, idx, min_delta, min_k, pos_idx, pos_min_delta, pos_min_k, dX, dPE, TARGET, S, cfg->n_inputs, O, Nt, Nc, npe, lr, j_begin, j_end); \
    } while (0)
    if (external_lr >= 0.0) {
        {
            KernelScope scope(K_CONCAT_BACKWARD, st);
            LUTB_CONCAT_BWD(true, false, nullptr);
        }
        LUTB_LAUNCH_CHECK();
        KernelScope scope(K_CONCAT_WEIGHT_UPDATE, st);
        LUTB_CONCAT_BWD(false, true, weights);
    } else {
        KernelScope scope(K_CONCAT_BACKWARD, st);
        LUTB_CONCAT_BWD(true, true, dW);
    }
#undef LUTB_CONCAT_BWD
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

extern "C" int lutb_check_detectors(const lutb_layer_cfg *cfg, int64_t rows, const float *x, const int32_t *anchors,
                                    int32_t *idx, float *min_delta, int32_t *min_k, void *stream) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    LUTB_REQUIRE(rows > 0, LUTB_ERR_SHAPE, "no input rows");
    LUTB_REQUIRE(x && anchors && idx, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE((min_delta == nullptr) == (min_k == nullptr), LUTB_ERR_MODE,
                 "min_anchor_deltas and min_anchor_delta_indices must be given together");
    return launch_check_detectors(x, rows, cfg->n_inputs, anchors, cfg->n_detectors, cfg->n_anchors, cfg->cmp_eps, idx,
                                  min_delta, min_k, static_cast<cudaStream_t>(stream));
}

extern "C" int lutb_check_positional(const lutb_layer_cfg *cfg, const float *pos_embeddings, int32_t *pos_idx,
                                     float *pos_min_delta, int32_t *pos_min_k, void *stream) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->seq_len > 1 && cfg->pos_dim > 0, LUTB_ERR_MODE, "the layer has no positional embeddings");
    LUTB_REQUIRE(pos_embeddings && pos_idx, LUTB_ERR_NULL, "positional embeddings / indices are NULL");
    LUTB_REQUIRE((pos_min_delta == nullptr) == (pos_min_k == nullptr), LUTB_ERR_MODE,
                 "positional min deltas and their indices must be given together");
    return launch_check_positional(cfg, pos_embeddings, pos_idx, pos_min_delta, pos_min_k, static_cast<cudaStream_t>(stream));
}

static int validate_query_range(const lutb_layer_cfg *cfg, int j_begin, int j_end) {
    LUTB_REQUIRE(j_begin >= 0 && j_begin <= j_end && j_end <= cfg->seq_len, LUTB_ERR_SHAPE,
                 "query range [%d, %d) outside [0, %d)", j_begin, j_end, cfg->seq_len);
    return LUTB_OK;
}

extern "C" int lutb_concat_pairs_forward(const lutb_layer_cfg *cfg, int64_t batch, const float *weights,
                                         const int32_t *idx, const int32_t *pos_idx, float *y, int32_t j_begin,
                                         int32_t j_end, void *stream) {
    int rc = validate_concat(cfg, batch);
    if (rc) return rc;
    rc = validate_query_range(cfg, j_begin, j_end);
    if (rc) return rc;
    LUTB_REQUIRE(weights && idx && y, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE(cfg->pos_dim == 0 || pos_idx, LUTB_ERR_NULL, "positional indices are NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (j_begin == j_end) return LUTB_OK;
    rc = launch_concat_pairs_forward(cfg, batch, weights, idx, pos_idx, y, j_begin, j_end, st);
    if (rc) return rc;
    if (cfg->int_mode) {
        // only the rows of the range hold fixed-point accumulators
        for (int64_t b = 0; b < batch; b++) {
            rc = launch_fixed_to_float(y + (b * cfg->seq_len + j_begin) * (int64_t)cfg->n_outputs,
                                       (int64_t)(j_end - j_begin) * cfg->n_outputs, cfg->int_rescaler, st);
            if (rc) return rc;
        }
    }
    return LUTB_OK;
}

extern "C" int lutb_concat_pairs_backward(const lutb_layer_cfg *cfg, int64_t batch, float *weights, const float *dY,
                                          const int32_t *anchors, const int32_t *idx, const float *min_delta,
                                          const int32_t *min_k, const int32_t *pos_idx, const float *pos_min_delta,
                                          const int32_t *pos_min_k, float *dX, float *dPE, float *dW, double external_lr,
                                          int32_t j_begin, int32_t j_end, void *stream) {
    int rc = validate_concat(cfg, batch);
    if (rc) return rc;
    rc = validate_query_range(cfg, j_begin, j_end);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->int_mode == 0, LUTB_ERR_MODE, "the query-range backward needs fp32 accumulators");
    LUTB_REQUIRE(weights && dY && anchors && idx && min_delta && min_k && dX, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE(cfg->pos_dim == 0 || (pos_idx && pos_min_delta && pos_min_k && dPE), LUTB_ERR_NULL, "positional tensors are NULL");
    LUTB_REQUIRE(!(external_lr >= 0.0 && dW != nullptr), LUTB_ERR_MODE,
                 "in internal weight gradients mode w_weights_gradients should be nullptr");
    LUTB_REQUIRE(!(external_lr < 0.0 && dW == nullptr), LUTB_ERR_NULL, "w_weights_gradients is NULL");
    if (j_begin == j_end) return LUTB_OK;
    return launch_concat_pairs_backward(cfg, batch, weights, dY, anchors, idx, min_delta, min_k, pos_idx, pos_min_delta,
                                        pos_min_k, dX, dPE, dW, external_lr, j_begin, j_end, static_cast<cudaStream_t>(stream));
}

extern "C" int lutb_concat_forward(const lutb_layer_cfg *cfg, int64_t batch, const float *weights, const float *x,
                                   const int32_t *anchors, const float *pos_embeddings, float *y, int32_t *idx,
                                   float *min_delta, int32_t *min_k, int32_t *pos_idx, float *pos_min_delta,
                                   int32_t *pos_min_k, void *stream) {
    int rc = validate_concat(cfg, batch);
    if (rc) return rc;
    LUTB_REQUIRE(weights && x && anchors && y && idx, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE((min_delta == nullptr) == (min_k == nullptr), LUTB_ERR_MODE,
                 "min_anchor_deltas and min_anchor_delta_indices must be given together");
    const int S = cfg->seq_len, npe = cfg->pos_dim, Nt = cfg->n_detectors;
    const bool train = min_delta != nullptr;
    if (npe > 0) {
        LUTB_REQUIRE(pos_embeddings && pos_idx, LUTB_ERR_NULL, "positional embeddings / indices are NULL");
        LUTB_REQUIRE(!train || (pos_min_delta && pos_min_k), LUTB_ERR_NULL, "positional min-delta outputs are NULL");
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = launch_check_detectors(x, batch * S, cfg->n_inputs, anchors, Nt, cfg->n_anchors, cfg->cmp_eps, idx, min_delta,
                                min_k, st);
    if (rc) return rc;
    if (npe > 0) {
        rc = launch_check_positional(cfg, pos_embeddings, pos_idx, train ? pos_min_delta : nullptr,
                                     train ? pos_min_k : nullptr, st);
        if (rc) return rc;
    }
    rc = launch_concat_pairs_forward(cfg, batch, weights, idx, pos_idx, y, 0, S, st);
    if (rc) return rc;
    if (cfg->int_mode) return launch_fixed_to_float(y, batch * S * (int64_t)cfg->n_outputs, cfg->int_rescaler, st);
    return LUTB_OK;
}

extern "C" int lutb_concat_backward(const lutb_layer_cfg *cfg, int64_t batch, float *weights, const float *dY,
                                    const int32_t *anchors, const int32_t *idx, const float *min_delta,
                                    const int32_t *min_k, const int32_t *pos_idx, const float *pos_min_delta,
                                    const int32_t *pos_min_k, float *dX, float *dPE, float *dW, double external_lr,
                                    void *stream) {
    int rc = validate_concat(cfg, batch);
    if (rc) return rc;
    LUTB_REQUIRE(weights && dY && anchors && idx && min_delta && min_k && dX, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    const int S = cfg->seq_len, npe = cfg->pos_dim, Nt = cfg->n_detectors, O = cfg->n_outputs, Nc = cfg->n_anchors;
    LUTB_REQUIRE(npe == 0 || (pos_idx && pos_min_delta && pos_min_k && dPE), LUTB_ERR_NULL, "positional tensors are NULL");
    LUTB_REQUIRE(!(external_lr >= 0.0 && dW != nullptr), LUTB_ERR_MODE,
                 "in internal weight gradients mode w_weights_gradients should be nullptr");
    LUTB_REQUIRE(!(external_lr < 0.0 && dW == nullptr), LUTB_ERR_NULL, "w_weights_gradients is NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cfg->int_mode) {
        double lr = cfg->lr_meta;
        if (external_lr >= 0.0) lr *= -(double)(float)external_lr;
        const int2 *an = reinterpret_cast<const int2 *>(anchors);
        const int n_ob = (O + cfg->forward_group - 1) / cfg->forward_group;
        const int64_t total = batch * S * (int64_t)Nt * S * n_ob;
        const int64_t blocks = min((total + 127) / 128, (int64_t)device_info().sm_count * 64);
        KernelScope scope(K_CONCAT_BACKWARD, st);
        concat_backward_fixed_kernel<<<(unsigned)blocks, 128, 0, st>>>(weights, dY, an, idx, min_delta, min_k, pos_idx, pos_min_delta, pos_min_k, dX, dPE, dW, batch, S, cfg->n_inputs, O, Nt, Nc, npe, cfg->forward_group, lr, cfg->int_rescaler);
        LUTB_LAUNCH_CHECK();
    } else {
        rc = launch_concat_pairs_backward(cfg, batch, weights, dY, anchors, idx, min_delta, min_k, pos_idx, pos_min_delta,
                                          pos_min_k, dX, dPE, dW, external_lr, 0, S, st);
        if (rc) return rc;
    }
    if (cfg->int_mode) {
        rc = launch_fixed_to_float(dX, batch * S * (int64_t)cfg->n_inputs, cfg->int_rescaler, st);
        if (rc) return rc;
        if (dW) {
            rc = launch_fixed_to_float(dW, (int64_t)Nt * ((int64_t)1 << (2 * Nc + npe)) * O, cfg->int_rescaler, st);
            if (rc) return rc;
        }
        if (npe > 0) rc = launch_fixed_to_float(dPE, (int64_t)(S - 1) * Nt * npe, cfg->int_rescaler, st);
    }
    return rc;
}

extern "C" int lutb_concat_sparse_forward(const lutb_layer_cfg *cfg, const lutb_sparse_index *sparse, int64_t batch,
                                          const float *weights, const float *x, const int32_t *anchors,
                                          const float *pos_embeddings, float *y, int32_t *idx, float *min_delta,
                                          int32_t *min_k, int32_t *pos_idx, float *pos_min_delta, int32_t *pos_min_k,
                                          void *stream) {
    int rc = validate_concat(cfg, batch);
    if (rc) return rc;
    SparseRows rows;
    rc = validate_sparse_rows(sparse, &rows);
    if (rc) return rc;
    LUTB_REQUIRE(weights && x && anchors && y && idx, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE((min_delta == nullptr) == (min_k == nullptr), LUTB_ERR_MODE,
                 "min_anchor_deltas and min_anchor_delta_indices must be given together");
    const int S = cfg->seq_len, npe = cfg->pos_dim, Nt = cfg->n_detectors;
    const bool train = min_delta != nullptr;
    if (npe > 0) {
        LUTB_REQUIRE(pos_embeddings && pos_idx, LUTB_ERR_NULL, "positional embeddings / indices are NULL");
        LUTB_REQUIRE(!train || (pos_min_delta && pos_min_k), LUTB_ERR_NULL, "positional min-delta outputs are NULL");
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = launch_check_detectors(x, batch * S, cfg->n_inputs, anchors, Nt, cfg->n_anchors, cfg->cmp_eps, idx, min_delta,
                                min_k, st);
    if (rc) return rc;
    if (npe > 0) {
        const int64_t n = (int64_t)(S - 1) * Nt;
        KernelScope scope(K_CHECK_POSITIONAL, st);
        if (train) check_positional_kernel<true><<<(unsigned)((n + 127) / 128), 128, 0, st>>>(pos_embeddings, n, npe, cfg->cmp_eps, pos_idx, pos_min_delta, pos_min_k);
        else check_positional_kernel<false><<<(unsigned)((n + 127) / 128), 128, 0, st>>>(pos_embeddings, n, npe, cfg->cmp_eps, pos_idx, nullptr, nullptr);
        LUTB_LAUNCH_CHECK();
    }
    {
        const int64_t total = batch * S * (int64_t)Nt * S;
        const int64_t blocks = min((total + 127) / 128, (int64_t)device_info().sm_count * 64);
        KernelScope scope(K_CONCAT_FORWARD, st);
        if (cfg->int_mode)
            concat_sparse_forward_kernel<true><<<(unsigned)blocks, 128, 0, st>>>(weights, idx, pos_idx, y, rows, batch, S, cfg->n_outputs, Nt, cfg->n_anchors, npe, cfg->int_rescaler);
        else
            concat_sparse_forward_kernel<false><<<(unsigned)blocks, 128, 0, st>>>(weights, idx, pos_idx, y, rows, batch, S, cfg->n_outputs, Nt, cfg->n_anchors, npe, cfg->int_rescaler);
        LUTB_LAUNCH_CHECK();
    }
    if (cfg->int_mode) return launch_fixed_to_float(y, batch * S * (int64_t)cfg->n_outputs, cfg->int_rescaler, st);
    return LUTB_OK;
}

extern "C" int lutb_concat_sparse_backward(const lutb_layer_cfg *cfg, const lutb_sparse_index *sparse, int64_t batch,
                                           float *weights, const float *dY, const int32_t *anchors, const int32_t *idx,
                                           const float *min_delta, const int32_t *min_k, const int32_t *pos_idx,
                                           const float *pos_min_delta, const int32_t *pos_min_k, float *dX, float *dPE,
                                           float *dW, double external_lr, void *stream) {
    int rc = validate_concat(cfg, batch);
    if (rc) return rc;
    SparseRows rows;
    rc = validate_sparse_rows(sparse, &rows);
    if (rc) return rc;
    LUTB_REQUIRE(weights && dY && anchors && idx && min_delta && min_k && dX, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    const int S = cfg->seq_len, npe = cfg->pos_dim, Nt = cfg->n_detectors, O = cfg->n_outputs, Nc = cfg->n_anchors;
    LUTB_REQUIRE(npe == 0 || (pos_idx && pos_min_delta && pos_min_k && dPE), LUTB_ERR_NULL, "positional tensors are NULL");
    LUTB_REQUIRE(!(external_lr >= 0.0 && dW != nullptr), LUTB_ERR_MODE,
                 "in internal weight gradients mode w_weights_gradients should be nullptr");
    LUTB_REQUIRE(!(external_lr < 0.0 && dW == nullptr), LUTB_ERR_NULL, "w_weights_gradients is NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    double lr = cfg->lr_meta;
    if (external_lr >= 0.0) lr *= -(double)(float)external_lr;
    const int2 *an = reinterpret_cast<const int2 *>(anchors);
    const int64_t total = batch * S * (int64_t)Nt * S;
    const int64_t blocks = min((total + 127) / 128, (int64_t)device_info().sm_count * 64);
#define LUTB_CS_BWD(DO_DX, TARGET)                                                                                          \
    do {                                                                                                                    \
        if (cfg->int_mode)                                                                                                  \
            concat_sparse_backward_kernel<true><<<(unsigned)blocks, 128, 0, st>>>(weights, dY, an, idx, min_delta, min_k, pos_idx, pos_min_delta, pos_min_k, dX, dPE, TARGET, rows, batch, S, cfg->n_inputs, O, Nt, Nc, npe, DO_DX, lr, cfg->int_rescaler); \
        else                                                                                                                \
            concat_sparse_backward_kernel<false><<<(unsigned)blocks, 128, 0, st>>>(weights, dY, an, idx, min_delta, min_k, pos_idx, pos_min_delta, pos_min_k, dX, dPE, TARGET, rows, batch, S, cfg->n_inputs, O, Nt, Nc, npe, DO_DX, lr, cfg->int_rescaler); \
    } while (0)
    if (external_lr >= 0.0) {
        // in-place SGD: every input gradient is computed from the unmodified tables first
        {
            KernelScope scope(K_CONCAT_BACKWARD, st);
            LUTB_CS_BWD(1, nullptr);
        }
        LUTB_LAUNCH_CHECK();
        KernelScope scope(K_CONCAT_WEIGHT_UPDATE, st);
        LUTB_CS_BWD(0, weights);
    } else {
        KernelScope scope(K_CONCAT_BACKWARD, st);
        LUTB_CS_BWD(1, dW);
    }
#undef LUTB_CS_BWD
    LUTB_LAUNCH_CHECK();
    if (cfg->int_mode) {
        rc = launch_fixed_to_float(dX, batch * S * (int64_t)cfg->n_inputs, cfg->int_rescaler, st);
        if (rc) return rc;
        if (dW) {
            rc = launch_fixed_to_float(dW, sparse->n_weights, cfg->int_rescaler, st);
            if (rc) return rc;
        }
        if (npe > 0) rc = launch_fixed_to_float(dPE, (int64_t)(S - 1) * Nt * npe, cfg->int_rescaler, st);
    }
    return rc;
}
