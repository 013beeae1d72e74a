// Product-mode sequence (attention) layer: for every causal pair (i < j) of a sample and every
// detector the table index is computed from the virtual vector [x1[b,i,:] | x2[b,j,:] | pe[j-i-1,t,:]]
// and the selected row is accumulated into y[b, j, :]; the backward pass recomputes the indices
// (nothing is cached from the forward, as in the reference) and routes the surrogate gradient to the
// token or positional embedding the flipped anchor reads.
//
// Reference: calculate_product_lookup_index[_backprop] (lut_runtime_kernels_logic.proto:32-198),
// fill_outputs_product_cpu_logic (:2148-2264), propagate_backward_product_cpu_logic (:2396-2628),
// gather_w_gradients_internal_product_cpu_logic (:2630-2744).
#include "fp32_gemm_sm100.cuh"
#include "product_hist.cuh"
#include "product_pairs.cuh"

namespace lutb {


// --------------------------------------------------------------------------------------------
// Forward.  Block = (detector, sample); each warp takes queries j round-robin: lanes first evaluate 32
// pairs (i, j) at a time into a per-warp index list in shared memory, then walk the list and add the
// selected rows with coalesced 16-byte loads (lanes over outputs), and finally reduce into y[b, j, :].
// --------------------------------------------------------------------------------------------
constexpr int kProdJ = 2;  // float4 vectors per lane and output chunk (256 outputs per chunk)

template <bool INT_MODE>
__global__ void __launch_bounds__(256) product_forward_kernel(const float *__restrict__ W, const float *__restrict__ x1,
                                                             const float *__restrict__ x2, const float *__restrict__ pe,
                                                             const int32_t *__restrict__ anchors, float *__restrict__ y,
                                                             int S, int e1, int e2, int npe, int n_outputs,
                                                             int n_detectors, int n_anchors, int sliced, float cmp_eps,
                                                             double fixed_scale) {
    extern __shared__ __align__(16) float smem[];
    const int t = blockIdx.x;
    const int64_t b = blockIdx.y;
    PairStage st;
    stage_pairs(st, smem, x1 + b * S * e1, x2 + b * S * e2, pe, anchors + (size_t)t * n_anchors * 2, S, e1, e2, npe,
                n_anchors, n_detectors, t, sliced != 0, cmp_eps);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    int32_t *idx_list = reinterpret_cast<int32_t *>(st.scratch) + warp * S;
    const float *Wt = W + (size_t)t * ((size_t)1 << n_anchors) * n_outputs;
    const bool vec4 = (n_outputs % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
    for (int j = 1 + warp; j < S; j += nwarps) {
        for (int i0 = 0; i0 < j; i0 += 32) {
            const int i = i0 + lane;
            int km; float dm;
            if (i < j) idx_list[i] = eval_pair<false>(st, n_anchors, i, j, cmp_eps, km, dm);
        }
        __syncwarp();
        float *yj = y + ((size_t)b * S + j) * n_outputs;
        if (vec4) {
            for (int c0 = 0; c0 < n_outputs; c0 += 128 * kProdJ) {
                float acc[kProdJ][4];
                int32_t iacc[kProdJ][4];
#pragma unroll
                for (int q = 0; q < kProdJ; q++)
#pragma unroll
                    for (int e = 0; e < 4; e++) { acc[q][e] = 0.f; iacc[q][e] = 0; }
#pragma unroll 8
                for (int i = 0; i < j; i++) {
                    const float *row = Wt + (size_t)idx_list[i] * n_outputs + c0;
#pragma unroll
                    for (int q = 0; q < kProdJ; q++) {
                        const int col = (lane + q * 32) * 4;
                        if (c0 + col < n_outputs) {
                            const float4 w = __ldg(reinterpret_cast<const float4 *>(row + col));
                            if (INT_MODE) {
                                iacc[q][0] += to_fixed((double)w.x, fixed_scale); iacc[q][1] += to_fixed((double)w.y, fixed_scale);
                                iacc[q][2] += to_fixed((double)w.z, fixed_scale); iacc[q][3] += to_fixed((double)w.w, fixed_scale);
                            } else {
                                acc[q][0] += w.x; acc[q][1] += w.y; acc[q][2] += w.z; acc[q][3] += w.w;
                            }
                        }
                    }
                }
#pragma unroll
                for (int q = 0; q < kProdJ; q++) {
                    const int col = c0 + (lane + q * 32) * 4;
                    if (col < n_outputs) {
                        if (INT_MODE) {
#pragma unroll
                            for (int e = 0; e < 4; e++) atomicAdd(reinterpret_cast<int32_t *>(yj) + col + e, iacc[q][e]);
                        } else {
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(yj + col), "f"(acc[q][0]),
                                         "f"(acc[q][1]), "f"(acc[q][2]), "f"(acc[q][3]) : "memory");
                        }
                    }
                }
            }
        } else {
            for (int o = lane; o < n_outputs; o += 32) {
                float acc = 0.f;
                int32_t iacc = 0;
                for (int i = 0; i < j; i++) {
                    const float w = __ldg(Wt + (size_t)idx_list[i] * n_outputs + o);
                    if (INT_MODE) iacc += to_fixed((double)w, fixed_scale);
                    else acc += w;
                }
                if (INT_MODE) atomicAdd(reinterpret_cast<int32_t *>(yj) + o, iacc);
                else atomicAdd(yj + o, acc);
            }
        }
        __syncwarp();
    }
}

// --------------------------------------------------------------------------------------------
// Backward, fp32 accumulators.  Same block / warp layout.  Per pair: g = sum_o dY[b,j,o] * (W[t,idx,o] -
// W[t,alt,o]) (lanes over outputs, fp32 partials per lane, transpose-reduce over 32 pairs so that lane l
// ends with the sum of pair i0 + l), du = up(min_delta) * g routed with +du / -du to the sources of the
// flipped anchor's two ends, and target[t, idx, :] += lr * dY[b, j, :].
// WEIGHTS selects what the launch does with the table gradient: 0 nothing, 1 accumulate into target.
// --------------------------------------------------------------------------------------------
template <bool DO_DX, bool DO_DW>
__global__ void __launch_bounds__(256) product_backward_kernel(const float *__restrict__ W, const float *__restrict__ x1,
                                                              const float *__restrict__ x2, const float *__restrict__ pe,
                                                              const int32_t *__restrict__ anchors,
                                                              const float *__restrict__ dY, float *__restrict__ dX1,
                                                              float *__restrict__ dX2, float *__restrict__ dPE,
                                                              float *__restrict__ target, int S, int e1, int e2, int npe,
                                                              int n_outputs, int n_detectors, int n_anchors, int sliced,
                                                              float cmp_eps, double lr) {
    extern __shared__ __align__(16) float smem[];
    const int t = blockIdx.x;
    const int64_t b = blockIdx.y;
    PairStage st;
    stage_pairs(st, smem, x1 + b * S * e1, x2 + b * S * e2, pe, anchors + (size_t)t * n_anchors * 2, S, e1, e2, npe,
                n_anchors, n_detectors, t, sliced != 0, cmp_eps);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    // per-warp scratch: dY row of the current query (padded to a multiple of 4)
    const int o_pad = (n_outputs + 3) & ~3;
    float *dy_s = st.scratch + warp * o_pad;
    const size_t rows = (size_t)1 << n_anchors;
    const float *Wt = W + (size_t)t * rows * n_outputs;
    float *Tt = DO_DW ? target + (size_t)t * rows * n_outputs : nullptr;
    const bool vec4 = (n_outputs % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(target) & 15) == 0);
    for (int j = 1 + warp; j < S; j += nwarps) {
        const float *dyj = dY + ((size_t)b * S + j) * n_outputs;
        for (int o = lane; o < o_pad; o += 32) dy_s[o] = o < n_outputs ? __ldg(dyj + o) : 0.f;
        __syncwarp();
        for (int i0 = 0; i0 < j; i0 += 32) {
            const int i = i0 + lane;
            int my_k = 0; float my_d = 0.f;
            int32_t my_idx = 0;
            if (i < j) my_idx = eval_pair<true>(st, n_anchors, i, j, cmp_eps, my_k, my_d);
            const int npairs = min(32, j - i0);
            float v[32];
#pragma unroll
            for (int p = 0; p < 32; p++) {
                v[p] = 0.f;
                if (p < npairs) {  // warp-uniform
                    const int32_t li = __shfl_sync(0xffffffffu, my_idx, p);
                    const int k = __shfl_sync(0xffffffffu, my_k, p);
                    const float *row = Wt + (size_t)li * n_outputs;
                    const float *alt = Wt + (size_t)(li ^ (1 << (k & 31))) * n_outputs;
                    float part = 0.f;
                    if (vec4) {
                        for (int col = lane * 4; col < n_outputs; col += 128) {
                            const float4 g = *reinterpret_cast<const float4 *>(dy_s + col);
                            if (DO_DX && k >= 0) {
                                const float4 a = __ldg(reinterpret_cast<const float4 *>(row + col));
                                const float4 c = __ldg(reinterpret_cast<const float4 *>(alt + col));
                                part += g.x * (a.x - c.x) + g.y * (a.y - c.y) + g.z * (a.z - c.z) + g.w * (a.w - c.w);
                            }
                            if (DO_DW) {
                                float4 u = g;   // lr == 1: the product is dY itself
                                if (lr != 1.0) {
                                    u.x = (float)((double)g.x * lr); u.y = (float)((double)g.y * lr);
                                    u.z = (float)((double)g.z * lr); u.w = (float)((double)g.w * lr);
                                }
                                u.x = fabsf(g.x) > kEpsF ? u.x : 0.f;
                                u.y = fabsf(g.y) > kEpsF ? u.y : 0.f;
                                u.z = fabsf(g.z) > kEpsF ? u.z : 0.f;
                                u.w = fabsf(g.w) > kEpsF ? u.w : 0.f;
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(Tt + (size_t)li * n_outputs + col),
                                             "f"(u.x), "f"(u.y), "f"(u.z), "f"(u.w) : "memory");
                            }
                        }
                    } else {
                        for (int o = lane; o < n_outputs; o += 32) {
                            const float g = dy_s[o];
                            if (DO_DX && k >= 0) part += g * (__ldg(row + o) - __ldg(alt + o));
                            if (DO_DW && fabs((double)g) > kEps) atomicAdd(Tt + (size_t)li * n_outputs + o, (float)((double)g * lr));
                        }
                    }
                    v[p] = part;
                }
            }
            if (DO_DX) {
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
                if (i < j && my_k >= 0) {
                    const double du = surrogate_up(my_d) * (double)v[0];
                    if (fabs(du) > kEps) {
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const int comp = st.comp[2 * my_k + e], elem = st.elem[2 * my_k + e];
                            const float val = e == 0 ? (float)du : (float)(-du);
                            if (comp == 0) atomicAdd(dX1 + ((size_t)b * S + i) * e1 + elem, val);
                            else if (comp == 1) atomicAdd(dX2 + ((size_t)b * S + j) * e2 + elem, val);
                            else if (comp == 2) atomicAdd(dPE + ((size_t)(j - i - 1) * n_detectors + t) * npe + elem, val);
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
}

// Fixed-point backward: one thread per (sample, query, detector, key) pair walks the outputs in order in
// double, exactly as the reference's host loop does; all contributions are truncated to int32 and added
// with integer atomics, which makes the result independent of the execution order.
__global__ void product_backward_fixed_kernel(const float *__restrict__ W, const float *__restrict__ x1,
                                              const float *__restrict__ x2, const float *__restrict__ pe,
                                              const int32_t *__restrict__ anchors, const float *__restrict__ dY,
                                              float *__restrict__ dX1, float *__restrict__ dX2, float *__restrict__ dPE,
                                              float *__restrict__ dW, int64_t batch, int S, int e1, int e2, int npe,
                                              int n_outputs, int n_detectors, int n_anchors, int sliced, float cmp_eps,
                                              double lr, double fixed_scale) {
    const int64_t total = batch * S * (int64_t)n_detectors * S;
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)(w % S);
        int64_t r = w / S;
        const int t = (int)(r % n_detectors);
        r /= n_detectors;
        const int j = (int)(r % S);
        const int64_t b = r / S;
        if (i >= j) continue;
        const float *xi = x1 + ((size_t)b * S + i) * e1;
        const float *xj = x2 + ((size_t)b * S + j) * e2;
        const float *p = npe > 0 ? pe + ((size_t)(j - i - 1) * n_detectors + t) * npe : nullptr;
        const int32_t *ap = anchors + (size_t)t * n_anchors * 2;
        int32_t li = 0;
        float md = 3.402823466e+38F;
        int mk = -1, c1m = 3, c2m = 3, e1m = 0, e2m = 0;
        for (int k = 0; k < n_anchors; k++) {
            int c1, c2, l1, l2;
            decode_anchor(__ldg(ap + 2 * k), sliced != 0, e1, e2, c1, l1);
            decode_anchor(__ldg(ap + 2 * k + 1), sliced != 0, e1, e2, c2, l2);
            if (c1 == 3 || c2 == 3) continue;
            const float v1 = c1 == 0 ? xi[l1] : (c1 == 1 ? xj[l1] : p[l1]);
            const float v2 = c2 == 0 ? xi[l2] : (c2 == 1 ? xj[l2] : p[l2]);
            const float d = __fsub_rn(v1, v2);
            if (greater_than_zero(d, cmp_eps)) li |= (1 << k);
            if (fabsf(d) < fabsf(md)) { md = d; mk = k; c1m = c1; c2m = c2; e1m = l1; e2m = l2; }
        }
        if (mk < 0) continue;
        const size_t rows = (size_t)1 << n_anchors;
        const float *row = W + ((size_t)t * rows + li) * n_outputs;
        const float *alt = W + ((size_t)t * rows + (li ^ (1 << mk))) * n_outputs;
        const float *dy = dY + ((size_t)b * S + j) * n_outputs;
        double ms = 0.0, as = 0.0;
        for (int o = 0; o < n_outputs; o++) ms += (double)__ldg(row + o) * (double)__ldg(dy + o);
        for (int o = 0; o < n_outputs; o++) as += (double)__ldg(alt + o) * (double)__ldg(dy + o);
        const double du = surrogate_up(md) * (ms - as);
        if (fabs(du) > kEps) {
            const int32_t d1 = to_fixed(du, fixed_scale);
            const int32_t d2 = to_fixed(-du, fixed_scale);
            int32_t *g1 = reinterpret_cast<int32_t *>(dX1), *g2 = reinterpret_cast<int32_t *>(dX2);
            int32_t *gp = reinterpret_cast<int32_t *>(dPE);
            if (c1m == 0) atomicAdd(g1 + ((size_t)b * S + i) * e1 + e1m, d1);
            else if (c1m == 1) atomicAdd(g2 + ((size_t)b * S + j) * e2 + e1m, d1);
            else atomicAdd(gp + ((size_t)(j - i - 1) * n_detectors + t) * npe + e1m, d1);
            if (c2m == 0) atomicAdd(g1 + ((size_t)b * S + i) * e1 + e2m, d2);
            else if (c2m == 1) atomicAdd(g2 + ((size_t)b * S + j) * e2 + e2m, d2);
            else atomicAdd(gp + ((size_t)(j - i - 1) * n_detectors + t) * npe + e2m, d2);
        }
        if (dW) {
            int32_t *drow = reinterpret_cast<int32_t *>(dW) + ((size_t)t * rows + li) * n_outputs;
            for (int o = 0; o < n_outputs; o++) {
                const double g = (double)__ldg(dy + o);
                if (fabs(g) > kEps) atomicAdd(drow + o, to_fixed(g * lr, fixed_scale));
            }
        }
    }
}

static int validate_product(const lutb_layer_cfg *cfg, int64_t batch, int S, int e1, int e2) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    LUTB_REQUIRE(batch > 0, LUTB_ERR_SHAPE, "batch_size == 0");
    LUTB_REQUIRE(batch <= 65535, LUTB_ERR_SHAPE, "batch_size > 65535 is not supported by the product kernels");
    LUTB_REQUIRE(S > 0, LUTB_ERR_SHAPE, "sequence_length == 0");
    LUTB_REQUIRE(e1 > 0 && e2 > 0, LUTB_ERR_SHAPE, "n_inputs_1 / n_inputs_2 == 0");
    LUTB_REQUIRE(cfg->n_anchors <= kMaxPairs, LUTB_ERR_SHAPE, "more than 16 anchor pairs per detector");
    return LUTB_OK;
}

// Resolves LUTB_PRODUCT_* into "use the histogram path" and "its contractions may run on the tensor cores".
static int choose_variant(const ProductCall &c, int variant, bool backward, const void *weights, const void *io_rows,
                          const void *dW, const void *workspace, size_t workspace_bytes, bool &hist, bool &allow_tc) {
    hist = false;
    allow_tc = variant != LUTB_PRODUCT_HIST_FMA;
    LUTB_REQUIRE(variant == LUTB_PRODUCT_AUTO || variant == LUTB_PRODUCT_DIRECT || variant == LUTB_PRODUCT_HIST ||
                     variant == LUTB_PRODUCT_HIST_FMA,
                 LUTB_ERR_MODE, "unknown product kernel variant %d", variant);
    if (variant == LUTB_PRODUCT_DIRECT) return LUTB_OK;
    const bool possible = product_hist_supported(c, weights, io_rows, dW);
    if (variant == LUTB_PRODUCT_HIST || variant == LUTB_PRODUCT_HIST_FMA) {
        LUTB_REQUIRE(possible, LUTB_ERR_MODE,
                     "the histogram variant needs fp32 accumulators, 4 <= Nc <= 12, O %% 4 == 0, S >= 2 and 16-byte aligned tensors");
        hist = true;
        return LUTB_OK;
    }
    // The contractions cost rows-per-table multiply-adds per (query, detector, output), the direct kernels one table
    // row through L2 per key: with the FMA contraction the histogram path pays once a query has about a quarter
    // (backward) or all (forward) of the table's rows as keys; on the tensor cores the contraction is several times
    // cheaper and the forward threshold drops to a quarter as well.
    const int64_t rows = (int64_t)1 << c.cfg->n_anchors;
    const bool long_enough = (backward || tc_gemm_available()) ? 4 * (int64_t)c.S >= rows : (int64_t)c.S >= rows;
    hist = possible && long_enough && workspace != nullptr &&
           workspace_bytes >= product_hist_workspace_bytes(c.cfg, 1, c.S, backward);
    return LUTB_OK;
}

}  // namespace lutb

using namespace lutb;

extern "C" size_t lutb_product_workspace(const lutb_layer_cfg *cfg, int64_t batch, int32_t seq_len, int backward) {
    if (!cfg || batch <= 0 || seq_len <= 0 || cfg->n_anchors < 1 || cfg->n_anchors > 16) return 0;
    return product_hist_workspace_bytes(cfg, batch, seq_len, backward != 0);
}

extern "C" int lutb_product_keeps_histogram(const lutb_layer_cfg *cfg, int64_t batch, int32_t seq_len, int32_t n_inputs_1,
                                            int32_t n_inputs_2, int variant, void *workspace, size_t workspace_bytes) {
    if (validate_product(cfg, batch, seq_len, n_inputs_1, n_inputs_2) != LUTB_OK) return 0;
    variant &= ~(LUTB_PRODUCT_KEEP_HIST | LUTB_PRODUCT_REUSE_HIST);
    const ProductCall call{cfg, batch, seq_len, n_inputs_1, n_inputs_2, nullptr, nullptr, nullptr, nullptr};
    bool hist_f = false, hist_b = false, tc_f = true, tc_b = true;
    // both passes must take the histogram path with this workspace (tensor alignment is the caller's to keep)
    const void *aligned = reinterpret_cast<const void *>((uintptr_t)256);
    if (choose_variant(call, variant, false, aligned, aligned, nullptr, workspace, workspace_bytes, hist_f, tc_f) != LUTB_OK) return 0;
    if (choose_variant(call, variant, true, aligned, aligned, aligned, workspace, workspace_bytes, hist_b, tc_b) != LUTB_OK) return 0;
    if (!hist_f || !hist_b) return 0;
    return product_hist_keeps(call, tc_f, workspace, workspace_bytes) ? 1 : 0;
}

extern "C" int lutb_product_forward(const lutb_layer_cfg *cfg, int64_t batch, int32_t seq_len, const float *weights,
                                    const float *x1, const float *x2, int32_t n_inputs_1, int32_t n_inputs_2,
                                    const float *pos_embeddings, const int32_t *anchors, float *y, int variant,
                                    void *workspace, size_t workspace_bytes, void *stream) {
    int rc = validate_product(cfg, batch, seq_len, n_inputs_1, n_inputs_2);
    if (rc) return rc;
    LUTB_REQUIRE(weights && x1 && x2 && anchors && y, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE(cfg->pos_dim == 0 || pos_embeddings, LUTB_ERR_NULL, "positional embeddings are NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const ProductCall call{cfg, batch, seq_len, n_inputs_1, n_inputs_2, x1, x2, pos_embeddings, anchors};
    bool hist = false, allow_tc = true;
    const bool keep = (variant & LUTB_PRODUCT_KEEP_HIST) != 0;
    variant &= ~(LUTB_PRODUCT_KEEP_HIST | LUTB_PRODUCT_REUSE_HIST);
    rc = choose_variant(call, variant, false, weights, y, nullptr, workspace, workspace_bytes, hist, allow_tc);
    if (rc) return rc;
    if (hist) return launch_product_hist_forward(call, weights, y, allow_tc, workspace, workspace_bytes, st, keep);
    if (seq_len > 1) {
        const int warps = 8;
        const size_t smem = (pair_stage_floats(seq_len, cfg->n_anchors, cfg->pos_dim) + (size_t)warps * seq_len) * 4;
        LUTB_REQUIRE(smem <= (size_t)kMaxSmemPerBlock - 1024, LUTB_ERR_SHAPE, "sequence too long for the product kernels");
        dim3 grid((unsigned)cfg->n_detectors, (unsigned)batch);
        KernelScope scope(K_PRODUCT_FORWARD, st);
        if (cfg->int_mode) {
            if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(product_forward_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            product_forward_kernel<true><<<grid, warps * 32, smem, st>>>(weights, x1, x2, pos_embeddings, anchors, y, seq_len, n_inputs_1, n_inputs_2, cfg->pos_dim, cfg->n_outputs, cfg->n_detectors, cfg->n_anchors, cfg->sliced_product, cfg->cmp_eps, cfg->int_rescaler);
        } else {
            if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(product_forward_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            product_forward_kernel<false><<<grid, warps * 32, smem, st>>>(weights, x1, x2, pos_embeddings, anchors, y, seq_len, n_inputs_1, n_inputs_2, cfg->pos_dim, cfg->n_outputs, cfg->n_detectors, cfg->n_anchors, cfg->sliced_product, cfg->cmp_eps, cfg->int_rescaler);
        }
        LUTB_LAUNCH_CHECK();
    }
    if (cfg->int_mode) return launch_fixed_to_float(y, batch * seq_len * (int64_t)cfg->n_outputs, cfg->int_rescaler, st);
    return LUTB_OK;
}

extern "C" int lutb_product_backward(const lutb_layer_cfg *cfg, int64_t batch, int32_t seq_len, float *weights,
                                     const float *x1, const float *x2, int32_t n_inputs_1, int32_t n_inputs_2,
                                     const float *pos_embeddings, const int32_t *anchors, const float *dY, float *dX1,
                                     float *dX2, float *dPE, float *dW, double external_lr, int variant, void *workspace,
                                     size_t workspace_bytes, void *stream) {
    int rc = validate_product(cfg, batch, seq_len, n_inputs_1, n_inputs_2);
    if (rc) return rc;
    LUTB_REQUIRE(weights && x1 && x2 && anchors && dY && dX1 && dX2, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE(cfg->pos_dim == 0 || (pos_embeddings && dPE), LUTB_ERR_NULL, "positional embeddings or their gradient are NULL");
    LUTB_REQUIRE(!(external_lr >= 0.0 && dW != nullptr), LUTB_ERR_MODE,
                 "in internal weight gradients mode w_weights_gradients should be nullptr");
    LUTB_REQUIRE(!(external_lr < 0.0 && dW == nullptr), LUTB_ERR_NULL, "w_weights_gradients is NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int O = cfg->n_outputs, Nt = cfg->n_detectors, Nc = cfg->n_anchors, npe = cfg->pos_dim;
    double lr = cfg->lr_meta;
    if (external_lr >= 0.0) lr *= -(double)(float)external_lr;
    const ProductCall call{cfg, batch, seq_len, n_inputs_1, n_inputs_2, x1, x2, pos_embeddings, anchors};
    bool hist = false, allow_tc = true;
    const bool reuse = (variant & LUTB_PRODUCT_REUSE_HIST) != 0;
    variant &= ~(LUTB_PRODUCT_KEEP_HIST | LUTB_PRODUCT_REUSE_HIST);
    rc = choose_variant(call, variant, true, weights, dY, dW, workspace, workspace_bytes, hist, allow_tc);
    if (rc) return rc;
    if (hist)
        return launch_product_hist_backward(call, weights, dY, dX1, dX2, dPE, external_lr >= 0.0 ? weights : dW, lr,
                                            external_lr >= 0.0, allow_tc, workspace, workspace_bytes, st, reuse);
    if (seq_len > 1) {
        if (cfg->int_mode) {
            const int64_t total = batch * seq_len * (int64_t)Nt * seq_len;
            const int64_t blocks = min((total + 127) / 128, (int64_t)device_info().sm_count * 64);
            KernelScope scope(K_PRODUCT_BACKWARD, st);
            product_backward_fixed_kernel<<<(unsigned)blocks, 128, 0, st>>>(weights, x1, x2, pos_embeddings, anchors, dY, dX1, dX2, dPE, dW, batch, seq_len, n_inputs_1, n_inputs_2, npe, O, Nt, Nc, cfg->sliced_product, cfg->cmp_eps, lr, cfg->int_rescaler);
            LUTB_LAUNCH_CHECK();
        } else {
            const int warps = 8;
            const size_t smem = (pair_stage_floats(seq_len, Nc, npe) + (size_t)warps * ((O + 3) & ~3)) * 4;
            LUTB_REQUIRE(smem <= (size_t)kMaxSmemPerBlock - 1024, LUTB_ERR_SHAPE, "sequence too long for the product kernels");
            dim3 grid((unsigned)Nt, (unsigned)batch);
#define LUTB_PROD_BWD(DX, DWF, TARGET)                                                                                   \
    do {                                                                                                                 \
        if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(product_backward_kernel<DX, DWF>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        product_backward_kernel<DX, DWF><<<grid, warps * 32, smem, st>>>(weights, x1, x2, pos_embeddings, anchors, dY, dX1, dX2, dPE, TARGET, seq_len, n_inputs_1, n_inputs_2, npe, O, Nt, Nc, cfg->sliced_product, cfg->cmp_eps, lr); \
    } while (0)
            if (external_lr >= 0.0) {
                // in-place SGD: all input gradients are computed from the unmodified tables first
                {
                    KernelScope scope(K_PRODUCT_BACKWARD, st);
                    LUTB_PROD_BWD(true, false, nullptr);
                }
                LUTB_LAUNCH_CHECK();
                KernelScope scope(K_PRODUCT_WEIGHT_UPDATE, st);
                LUTB_PROD_BWD(false, true, weights);
            } else {
                KernelScope scope(K_PRODUCT_BACKWARD, st);
                LUTB_PROD_BWD(true, true, dW);
            }
#undef LUTB_PROD_BWD
            LUTB_LAUNCH_CHECK();
        }
    }
    if (cfg->int_mode) {
        rc = launch_fixed_to_float(dX1, batch * seq_len * (int64_t)n_inputs_1, cfg->int_rescaler, st);
        if (rc) return rc;
        if (dX2 != dX1) {
            rc = launch_fixed_to_float(dX2, batch * seq_len * (int64_t)n_inputs_2, cfg->int_rescaler, st);
            if (rc) return rc;
        }
        if (dW) {
            rc = launch_fixed_to_float(dW, (int64_t)Nt * ((int64_t)1 << Nc) * O, cfg->int_rescaler, st);
            if (rc) return rc;
        }
        if (npe > 0 && seq_len > 1) rc = launch_fixed_to_float(dPE, (int64_t)(seq_len - 1) * Nt * npe, cfg->int_rescaler, st);
    }
    return rc;
}
