/*
 * CPU oracle for the LUT-layer hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the arithmetic the reference performs on its
 * CPU path (the reference executes its kernel source as nested host loops, batch outermost,
 * see spiky_cuda/misc/misc.h:119-129).  It is used as the checker in tests/, in the smoke
 * test and as the timed CPU baseline of the benchmark; nothing in the product path may
 * call it.  Loop nests follow the reference's host loop order so that fp32 results agree
 * with the reference CPU build to the last bit where the reference itself is
 * deterministic; the golden fixtures under tests/golden/ (produced by the real reference)
 * pin that.
 *
 * Conventions shared by every function:
 *   anchors  int32 [Nt][Nc][2]; a pair with either end == -1 (0xFFFFFFFF) is skipped
 *   W        fp32 [Nt][T][O] flat, element (t*T + row)*O + o   (fully connected layers)
 *   int_mode 0: fp32 accumulators; 1: int32 fixed-point accumulators (scale 0xFFFFF * rescaler,
 *            spiky_cuda/misc/misc.h:92-103), converted to fp32 at the end of each call
 *            (spiky_cuda/lut/lut_runtime_kernels_logic.proto:200-213)
 *
 * Compile with:  gcc -O2 -ffp-contract=off -fno-fast-math  (no FMA contraction, IEEE semantics)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_DENOM 1048575.0                 /* DENOMINATOR32, misc.h:101 */
#define ORC_DENOM_RECIP 9.536752259018191e-07 /* DENOMINATOR32_RECIPROC, misc.h:102 */
#define ORC_EPS 0.00000000000000001         /* EPS, misc.h:90 */
#define ORC_NO_ANCHOR (-1)

/*
 * Thread count of the batch-parallel loops.  1 reproduces the reference, whose CPU path is
 * single-threaded by construction (misc.h:119-129).  Larger values only split loops whose
 * iterations touch disjoint cells (samples for outputs / input gradients, detectors for weight
 * gradients), so every result stays bit-identical; they exist for the "all host cores" baseline.
 */
static int orc_threads = 1;
void orc_set_threads(int n) { orc_threads = n > 0 ? n : 1; }
#define ORC_PARALLEL_FOR _Pragma("omp parallel for schedule(static) num_threads(orc_threads)")

/* ROUNDED_COMPARISON_GREATER(delta, 0, eps), misc.h:16 */
static inline int orc_greater(float delta, float cmp_eps) {
    if (cmp_eps == 0.0f) return delta > 0.0f;
    if (fabs((double)delta) < (double)cmp_eps) return 0;
    return delta > 0.0f;
}

/* surrogate derivative up(m) = +-0.5 / (1+|m|)^2, zero counts as negative
 * (lut_runtime_kernels_logic.proto:1339-1345) */
static inline double orc_up(float m) {
    double du = (double)m;
    if (du > 0) {
        du = 1.0 / (1.0 + fabs(du));
        du *= 0.5 * du;
    } else {
        du = 1.0 / (1.0 + fabs(du));
        du *= -0.5 * du;
    }
    return du;
}

/* convert_integers_to_floats_logic, proto:200-213 */
void orc_int_to_float(float *buf, int64_t n, double rescaler) {
    for (int64_t i = 0; i < n; i++) {
        double y = (double)(*(int32_t *)(buf + i)) * ORC_DENOM_RECIP;
        buf[i] = (float)(y / rescaler);
    }
}

/*
 * check_detectors_logic / check_detectors_eval_logic / check_detectors_seq*_logic
 * (proto:1050-1158, 1589-1707).  rows = B for non-sequence layers, B*S for sequence layers.
 * min_delta / min_k may be NULL (eval variant).
 */
void orc_check_detectors(const float *x, int64_t rows, int I, const int32_t *anchors, int Nt, int Nc,
                         float cmp_eps, int32_t *idx, float *min_delta, int32_t *min_k) {
    ORC_PARALLEL_FOR
    for (int64_t r = 0; r < rows; r++) {
        const float *xr = x + r * (int64_t)I;
        for (int t = 0; t < Nt; t++) {
            const int32_t *ap = anchors + (int64_t)t * Nc * 2;
            int32_t li = 0;
            float md = 0.0f;
            int32_t mk = -1;
            for (int k = 0; k < Nc; k++) {
                int32_t a1 = ap[2 * k], a2 = ap[2 * k + 1];
                if (a1 == ORC_NO_ANCHOR || a2 == ORC_NO_ANCHOR) continue;
                float delta = xr[a1] - xr[a2];
                if (orc_greater(delta, cmp_eps)) li |= (1 << k);
                if (mk == -1 || fabsf(delta) < fabsf(md)) {
                    md = delta;
                    mk = k;
                }
            }
            idx[r * Nt + t] = li;
            if (min_delta) min_delta[r * Nt + t] = md;
            if (min_k) min_k[r * Nt + t] = mk;
        }
    }
}

/*
 * check_positional_embeddings[_eval]_logic (proto:1709-1805): sign bits of pe[d][t][:],
 * first minimal |value| and its dimension.  pe is [(S-1)][Nt][Npe].
 */
void orc_check_positional(const float *pe, int S, int Nt, int Npe, float cmp_eps, int32_t *pidx,
                          float *pmin, int32_t *pmin_k) {
    int64_t n = (int64_t)(S - 1) * Nt;
    for (int64_t i = 0; i < n; i++) {
        const float *p = pe + i * Npe;
        int32_t li = 0, mk = -1;
        float md = 0.0f;
        for (int d = 0; d < Npe; d++) {
            float v = p[d];
            if (orc_greater(v, cmp_eps)) li |= (1 << d);
            if (mk == -1 || fabsf(v) < fabsf(md)) {
                md = v;
                mk = d;
            }
        }
        pidx[i] = li;
        if (pmin) pmin[i] = md;
        if (pmin_k) pmin_k[i] = mk;
    }
}

/*
 * fill_outputs_non_seq_fc_logic (proto:1214-1299) + the int->float pass of
 * LUTRuntimeContext::forward_step (lut_runtime.cu:200-210).
 * y is accumulated into (caller zero-fills).  Gb = backward_group_size: detectors are summed in
 * double inside blocks of Gb, each block sum is rounded (fp32) or truncated (int32 fixed point)
 * and then added to y.
 */
void orc_nonseq_fc_forward(const float *W, const int32_t *idx, float *y, int64_t B, int O, int Nt, int T,
                           int Gb, int int_mode, double rescaler) {
    int n_blocks = (Nt + Gb - 1) / Gb;
    ORC_PARALLEL_FOR
    for (int64_t b = 0; b < B; b++) {
        const int32_t *li = idx + b * Nt;
        float *yb = y + b * O;
        for (int blk = 0; blk < n_blocks; blk++) {
            int t0 = blk * Gb, t1 = t0 + Gb < Nt ? t0 + Gb : Nt;
            for (int o = 0; o < O; o++) {
                double s = 0.0;
                for (int t = t0; t < t1; t++) s += (double)W[((int64_t)t * T + li[t]) * O + o];
                if (int_mode)
                    *(int32_t *)(yb + o) += (int32_t)(s * ORC_DENOM * rescaler);
                else
                    yb[o] += (float)s;
            }
        }
    }
    if (int_mode) orc_int_to_float(y, B * O, rescaler);
}

/*
 * int8-table inference (no reference counterpart): fill_outputs_non_seq_fc_logic in int32 fixed-point mode
 * (proto:1214-1299) on the de-quantised table.  exact = 0: entries are the fp32 numbers f32(scale * q), i.e.
 * orc_nonseq_fc_forward(int_mode = 1) on that fp32 table; exact = 1: entries are the exact reals scale * q
 * (the 24 x 8 bit product is exact in double).  acc is accumulated into and left as int32.
 */
void orc_infer_int8(const int8_t *Q, const float *scales, const int32_t *idx, int32_t *acc, int64_t B, int O, int Nt,
                    int T, int Gb, double rescaler, int exact) {
    int n_blocks = (Nt + Gb - 1) / Gb;
    ORC_PARALLEL_FOR
    for (int64_t b = 0; b < B; b++) {
        const int32_t *li = idx + b * Nt;
        for (int blk = 0; blk < n_blocks; blk++) {
            int t0 = blk * Gb, t1 = t0 + Gb < Nt ? t0 + Gb : Nt;
            for (int o = 0; o < O; o++) {
                double s = 0.0;
                for (int t = t0; t < t1; t++) {
                    int q = Q[((int64_t)t * T + li[t]) * O + o];
                    if (exact) s += (double)scales[t] * (double)q;
                    else { volatile float w = scales[t] * (float)q; s += (double)w; }
                }
                acc[b * O + o] += (int32_t)(s * ORC_DENOM * rescaler);
            }
        }
    }
}

/*
 * propagate_through_detectors_non_seq_fc_logic (proto:1421-1499) followed by
 * gather_w_gradients_non_seq_fc_logic (proto:1547-1585, helper :716-819) and the int->float passes
 * of LUTRuntimeContext::backward_backprop (lut_runtime.cu:365-396).
 *   G        forward_group_size: outputs are processed in blocks of G; every block issues its own
 *            (rounded / truncated) contribution to dX
 *   lr_meta  SynapseMeta.learning_rate
 *   ext_lr   < 0: write lr_meta*dY into dW (caller zero-fills);  >= 0: "Internal" policy, dW must be
 *            NULL and W is updated in place by -ext_lr*lr_meta*dY (lut_runtime.cu:236-238, 343-361)
 * dX is accumulated into (caller zero-fills).
 */
void orc_nonseq_fc_backward(float *W, const float *dY, const int32_t *anchors, const int32_t *idx,
                            const float *min_delta, const int32_t *min_k, float *dX, float *dW, int64_t B,
                            int I, int O, int Nt, int Nc, int T, int G, double lr_meta, double ext_lr,
                            int int_mode, double rescaler) {
    int n_ob = (O + G - 1) / G;
    ORC_PARALLEL_FOR
    for (int64_t b = 0; b < B; b++) {
        const float *dy = dY + b * O;
        float *dx = dX + b * (int64_t)I;
        for (int t = 0; t < Nt; t++) {
            int32_t li = idx[b * Nt + t];
            int32_t k = min_k[b * Nt + t];
            int64_t row = ((int64_t)t * T + li) * O;
            int64_t alt = ((int64_t)t * T + (li ^ (1 << k))) * O;
            for (int ob = 0; ob < n_ob; ob++) {
                int o0 = ob * G, o1 = o0 + G < O ? o0 + G : O;
                double du = orc_up(min_delta[b * Nt + t]);
                double ms = 0.0, as = 0.0;
                for (int o = o0; o < o1; o++) {
                    double g = (double)dy[o];
                    ms += (double)W[row + o] * g;
                    as += (double)W[alt + o] * g;
                }
                du *= ms - as;
                if (fabs(du) > ORC_EPS) {
                    int32_t a1 = anchors[((int64_t)t * Nc + k) * 2], a2 = anchors[((int64_t)t * Nc + k) * 2 + 1];
                    if (int_mode) {
                        int32_t d = (int32_t)(du * ORC_DENOM * rescaler);
                        *(int32_t *)(dx + a1) += d;
                        *(int32_t *)(dx + a2) -= d;
                    } else {
                        dx[a1] += du;
                        dx[a2] -= du;
                    }
                }
            }
        }
    }
    double lr = lr_meta;
    if (ext_lr >= 0) lr *= -ext_lr;
    float *target = ext_lr >= 0 ? W : dW;
    /* every cell belongs to one detector and receives its contributions in batch order, exactly as
     * in the reference's batch-outermost loop; detectors are therefore independent */
    ORC_PARALLEL_FOR
    for (int t = 0; t < Nt; t++) {
        for (int64_t b = 0; b < B; b++) {
            const float *dy = dY + b * O;
            int64_t row = ((int64_t)t * T + idx[b * Nt + t]) * O;
            for (int o = 0; o < O; o++) {
                double g = (double)dy[o];
                if (fabs(g) > ORC_EPS) {
                    if (int_mode)
                        *(int32_t *)(target + row + o) += (int32_t)(g * lr * ORC_DENOM * rescaler);
                    else
                        target[row + o] += (float)(g * lr);
                }
            }
        }
    }
    if (int_mode) {
        orc_int_to_float(dX, B * (int64_t)I, rescaler);
        if (dW) orc_int_to_float(dW, (int64_t)Nt * T * O, rescaler);
    }
}

/* ------------------------------------------------------------------------------------------
 * Sparse (projection / convolution) lookup -> output connectivity.
 *
 * The reference stores, per lookup neuron, a run of "forward synapse groups": an 8-byte header
 * followed by up to G 4-byte target ids (spiky_cuda/connections_manager/connections_manager.h:39-66).
 * The weight of a synapse lives in a separate fp32 array at the index of its target id inside the
 * arena, counted in 4-byte words from the first synapse (lut_runtime_kernels_logic.proto:227), so
 * every group header leaves two unused weight slots.  In all reference layer types the lookup
 * neurons of one detector share one target list, and neurons are laid out in id order; the oracle
 * therefore takes the connectivity per detector:
 *   det_wbase[t]   weight index of synapse 0 of row 0
 *   det_stride[t]  weight-index distance between consecutive rows (= P + 2*ceil(P/G))
 *   det_count[t]   P, synapses per row
 *   det_toff[t]    offset of the detector's target list (output indices, synapse order) in `targets`
 * Synapse p of a row sits at row_base + p + 2*(p/G); group `ob` holds synapses [ob*G, ob*G+G).
 * ------------------------------------------------------------------------------------------ */
static inline int64_t orc_syn_slot(int64_t row_base, int p, int G) { return row_base + p + 2 * (p / G); }

/* fill_outputs_non_seq_sparse_logic + fire_single_synapse_group (proto:1160-1212, 215-313) */
void orc_nonseq_sparse_forward(const float *W, const int32_t *idx, float *y, int64_t B, int O, int Nt,
                               const int64_t *det_wbase, const int32_t *det_stride, const int32_t *det_count,
                               const int32_t *det_toff, const int32_t *targets, int G, int int_mode,
                               double rescaler) {
    ORC_PARALLEL_FOR
    for (int64_t b = 0; b < B; b++) {
        float *yb = y + b * O;
        for (int t = 0; t < Nt; t++) {
            int64_t row = det_wbase[t] + (int64_t)idx[b * Nt + t] * det_stride[t];
            const int32_t *tg = targets + det_toff[t];
            for (int p = 0; p < det_count[t]; p++) {
                double w = (double)W[orc_syn_slot(row, p, G)];
                if (int_mode)
                    *(int32_t *)(yb + tg[p]) += (int32_t)(w * ORC_DENOM * rescaler);
                else
                    yb[tg[p]] += (float)w;
            }
        }
    }
    if (int_mode) orc_int_to_float(y, B * O, rescaler);
}

/* propagate_through_detectors_non_seq_sparse_logic (proto:1303-1419, helper :315-395) and
 * gather_w_gradients_non_seq_sparse_logic (proto:1501-1545, helper :584-714).
 * n_weights is the length of W / dW. */
void orc_nonseq_sparse_backward(float *W, const float *dY, const int32_t *anchors, const int32_t *idx,
                                const float *min_delta, const int32_t *min_k, float *dX, float *dW, int64_t B,
                                int I, int O, int Nt, int Nc, const int64_t *det_wbase,
                                const int32_t *det_stride, const int32_t *det_count, const int32_t *det_toff,
                                const int32_t *targets, int G, int64_t n_weights, double lr_meta, double ext_lr,
                                int int_mode, double rescaler) {
    ORC_PARALLEL_FOR
    for (int64_t b = 0; b < B; b++) {
        const float *dy = dY + b * O;
        float *dx = dX + b * (int64_t)I;
        for (int t = 0; t < Nt; t++) {
            int32_t li = idx[b * Nt + t];
            int32_t k = min_k[b * Nt + t];
            int P = det_count[t];
            int64_t row = det_wbase[t] + (int64_t)li * det_stride[t];
            int64_t alt = det_wbase[t] + (int64_t)(li ^ (1 << k)) * det_stride[t];
            const int32_t *tg = targets + det_toff[t];
            int n_groups = (P + G - 1) / G;
            for (int ob = 0; ob < n_groups; ob++) {
                int p0 = ob * G, p1 = p0 + G < P ? p0 + G : P;
                double du = orc_up(min_delta[b * Nt + t]);
                double ms = 0.0, as = 0.0;
                for (int p = p0; p < p1; p++) ms += (double)W[orc_syn_slot(row, p, G)] * (double)dy[tg[p]];
                for (int p = p0; p < p1; p++) as += (double)W[orc_syn_slot(alt, p, G)] * (double)dy[tg[p]];
                du *= ms - as;
                if (fabs(du) > ORC_EPS) {
                    int32_t a1 = anchors[((int64_t)t * Nc + k) * 2], a2 = anchors[((int64_t)t * Nc + k) * 2 + 1];
                    if (int_mode) {
                        int32_t d = (int32_t)(du * ORC_DENOM * rescaler);
                        *(int32_t *)(dx + a1) += d;
                        *(int32_t *)(dx + a2) -= d;
                    } else {
                        dx[a1] += du;
                        dx[a2] -= du;
                    }
                }
            }
        }
    }
    double lr = lr_meta;
    if (ext_lr >= 0) lr *= -ext_lr;
    float *target = ext_lr >= 0 ? W : dW;
    ORC_PARALLEL_FOR
    for (int t = 0; t < Nt; t++) {
        const int32_t *tg = targets + det_toff[t];
        for (int64_t b = 0; b < B; b++) {
            const float *dy = dY + b * O;
            int64_t row = det_wbase[t] + (int64_t)idx[b * Nt + t] * det_stride[t];
            for (int p = 0; p < det_count[t]; p++) {
                double g = (double)dy[tg[p]];
                if (fabs(g) > ORC_EPS) {
                    int64_t slot = orc_syn_slot(row, p, G);
                    if (int_mode)
                        *(int32_t *)(target + slot) += (int32_t)(g * lr * ORC_DENOM * rescaler);
                    else
                        target[slot] += (float)(g * lr);
                }
            }
        }
    }
    if (int_mode) {
        orc_int_to_float(dX, B * (int64_t)I, rescaler);
        if (dW) orc_int_to_float(dW, n_weights, rescaler);
    }
}

/* ------------------------------------------------------------------------------------------
 * Product-mode sequence layers: the table index is computed per causal pair (i < j) from the
 * virtual vector [x1[b,i,:] | x2[b,j,:] | pe[j-i-1, t, :]] (sliced mode: interleaved, anchor id =
 * 3 * slot + component) with the non-sequence rule, tables have 2^Nc rows.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    int comp;   /* 0: x1 at position i, 1: x2 at position j, 2: positional embedding */
    int index;  /* element inside that source */
} orc_src;

/* anchor id -> (source, element), proto:60-66 (sliced) and :82-88 (sequential layout) */
static inline orc_src orc_product_src(int32_t id, int sliced, int E1, int E2) {
    orc_src s;
    if (sliced) {
        s.index = id / 3;
        s.comp = id % 3;
    } else {
        s.comp = id < E1 ? 0 : (id < E1 + E2 ? 1 : 2);
        s.index = id - (s.comp == 0 ? 0 : (s.comp == 1 ? E1 : E1 + E2));
    }
    return s;
}

/* calculate_product_lookup_index_backprop, proto:102-198 (the forward-only variant :32-100 computes
 * the same index: val1 > val2 and (val1 - val2) > 0 agree in IEEE arithmetic with denormals kept).
 * Returns the index; *alt, the two flipped sources and the minimal delta are optional outputs. */
static inline int32_t orc_product_index(const int32_t *ap, int Nc, int sliced, int E1, int E2, const float *v1,
                                        const float *v2, const float *pe, float cmp_eps, int32_t *alt,
                                        orc_src *first, orc_src *second, float *min_delta) {
    const float *src[3] = {v1, v2, pe};
    int32_t li = 0;
    float md = 3.402823466e+38F;
    int flip = -1;
    orc_src f1 = {-1, -1}, f2 = {-1, -1};
    for (int k = 0; k < Nc; k++) {
        int32_t a1 = ap[2 * k], a2 = ap[2 * k + 1];
        if (a1 == ORC_NO_ANCHOR || a2 == ORC_NO_ANCHOR) continue;
        orc_src s1 = orc_product_src(a1, sliced, E1, E2), s2 = orc_product_src(a2, sliced, E1, E2);
        float delta = src[s1.comp][s1.index] - src[s2.comp][s2.index];
        if (orc_greater(delta, cmp_eps)) li |= (1 << k);
        if (fabsf(delta) < fabsf(md)) {
            md = delta;
            flip = k;
            f1 = s1;
            f2 = s2;
        }
    }
    if (alt) *alt = flip >= 0 ? (li ^ (1 << flip)) : li;
    if (first) *first = f1;
    if (second) *second = f2;
    if (min_delta) *min_delta = md;
    return li;
}

/* fill_outputs_product_cpu_logic, proto:2148-2264 (fully connected branch) */
void orc_product_forward(const float *W, const float *x1, const float *x2, const float *pe, const int32_t *anchors,
                         float *y, int64_t B, int S, int E1, int E2, int Npe, int O, int Nt, int Nc, int sliced,
                         float cmp_eps, int int_mode, double rescaler) {
    int T = 1 << Nc;
    ORC_PARALLEL_FOR
    for (int64_t b = 0; b < B; b++) {
        for (int j = 0; j < S; j++) {
            float *yo = y + (b * S + j) * O;
            for (int t = 0; t < Nt; t++) {
                const int32_t *ap = anchors + (int64_t)t * Nc * 2;
                for (int i = 0; i < j; i++) {
                    const float *p = Npe > 0 ? pe + ((int64_t)(j - i - 1) * Nt + t) * Npe : NULL;
                    int32_t li = orc_product_index(ap, Nc, sliced, E1, E2, x1 + (b * S + i) * E1, x2 + (b * S + j) * E2, p,
                                                   cmp_eps, NULL, NULL, NULL, NULL);
                    const float *row = W + ((int64_t)t * T + li) * O;
                    for (int o = 0; o < O; o++) {
                        double w = (double)row[o];
                        if (int_mode)
                            *(int32_t *)(yo + o) += (int32_t)(w * ORC_DENOM * rescaler);
                        else
                            yo[o] += (float)w;
                    }
                }
            }
        }
    }
    if (int_mode) orc_int_to_float(y, B * S * O, rescaler);
}

static inline void orc_route(orc_src s, double du, float *dX1, float *dX2, float *dPE, int64_t b, int S, int i, int j,
                             int E1, int E2, int Npe, int Nt, int t, int int_mode, double rescaler) {
    float *cell;
    if (s.comp == 0) cell = dX1 + (b * S + i) * E1 + s.index;
    else if (s.comp == 1) cell = dX2 + (b * S + j) * E2 + s.index;
    else if (s.comp == 2) cell = dPE + ((int64_t)(j - i - 1) * Nt + t) * Npe + s.index;
    else return;
    if (int_mode) *(int32_t *)cell += (int32_t)(du * ORC_DENOM * rescaler);
    else *cell += (float)du;
}

/*
 * propagate_backward_product_cpu_logic (proto:2396-2628, helper propagate_through_detector_product :869-1014)
 * and, for the internal policy, gather_w_gradients_internal_product_cpu_logic (proto:2630-2744).
 * dX1 / dX2 may alias (the layer passes the same buffer twice).  Not thread-parallel over samples when
 * dPE is given (dPE is shared by the batch), to keep the reference's accumulation order.
 */
void orc_product_backward(float *W, const float *x1, const float *x2, const float *pe, const int32_t *anchors,
                          const float *dY, float *dX1, float *dX2, float *dPE, float *dW, int64_t B, int S, int E1,
                          int E2, int Npe, int O, int Nt, int Nc, int sliced, float cmp_eps, double lr_meta,
                          double ext_lr, int int_mode, double rescaler) {
    int T = 1 << Nc;
    for (int64_t b = 0; b < B; b++) {
        for (int j = 0; j < S; j++) {
            const float *dy = dY + (b * S + j) * O;
            for (int t = 0; t < Nt; t++) {
                const int32_t *ap = anchors + (int64_t)t * Nc * 2;
                for (int i = 0; i < j; i++) {
                    const float *p = Npe > 0 ? pe + ((int64_t)(j - i - 1) * Nt + t) * Npe : NULL;
                    int32_t alt_li;
                    orc_src f1, f2;
                    float md;
                    int32_t li = orc_product_index(ap, Nc, sliced, E1, E2, x1 + (b * S + i) * E1, x2 + (b * S + j) * E2, p,
                                                   cmp_eps, &alt_li, &f1, &f2, &md);
                    const float *row = W + ((int64_t)t * T + li) * O;
                    const float *alt = W + ((int64_t)t * T + alt_li) * O;
                    double ms = 0.0, as = 0.0;
                    for (int o = 0; o < O; o++) ms += (double)row[o] * (double)dy[o];
                    for (int o = 0; o < O; o++) as += (double)alt[o] * (double)dy[o];
                    double du = orc_up(md) * (ms - as);
                    if (fabs(du) > ORC_EPS) {
                        orc_route(f1, du, dX1, dX2, dPE, b, S, i, j, E1, E2, Npe, Nt, t, int_mode, rescaler);
                        orc_route(f2, -du, dX1, dX2, dPE, b, S, i, j, E1, E2, Npe, Nt, t, int_mode, rescaler);
                    }
                    if (dW) {
                        float *drow = dW + ((int64_t)t * T + li) * O;
                        for (int o = 0; o < O; o++) {
                            double g = (double)dy[o];
                            if (fabs(g) > ORC_EPS) {
                                if (int_mode) *(int32_t *)(drow + o) += (int32_t)(g * lr_meta * ORC_DENOM * rescaler);
                                else drow[o] += (float)(g * lr_meta);
                            }
                        }
                    }
                }
            }
        }
    }
    if (ext_lr >= 0) {
        double lr = lr_meta * -ext_lr;
        for (int64_t b = 0; b < B; b++)
            for (int j = 0; j < S; j++) {
                const float *dy = dY + (b * S + j) * O;
                for (int t = 0; t < Nt; t++) {
                    const int32_t *ap = anchors + (int64_t)t * Nc * 2;
                    for (int i = 0; i < j; i++) {
                        const float *p = Npe > 0 ? pe + ((int64_t)(j - i - 1) * Nt + t) * Npe : NULL;
                        int32_t li = orc_product_index(ap, Nc, sliced, E1, E2, x1 + (b * S + i) * E1, x2 + (b * S + j) * E2,
                                                       p, cmp_eps, NULL, NULL, NULL, NULL);
                        float *wrow = W + ((int64_t)t * T + li) * O;
                        for (int o = 0; o < O; o++) {
                            double g = (double)dy[o];
                            if (fabs(g) > ORC_EPS) wrow[o] += (float)(g * lr);
                        }
                    }
                }
            }
    }
    if (int_mode) {
        orc_int_to_float(dX1, B * S * (int64_t)E1, rescaler);
        if (dX2 != dX1) orc_int_to_float(dX2, B * S * (int64_t)E2, rescaler);
        if (dW) orc_int_to_float(dW, (int64_t)Nt * T * O, rescaler);
        if (Npe > 0 && dPE) orc_int_to_float(dPE, (int64_t)(S - 1) * Nt * Npe, rescaler);
    }
}

/* ------------------------------------------------------------------------------------------
 * Concatenation-mode sequence layers: every token gets its own index (orc_check_detectors over
 * B*S rows), every (distance, detector) its positional index (orc_check_positional); a causal pair
 * (i < j) selects row (Q_j << (Nc + Npe)) | (K_i << Npe) | PE_{j-i-1} of a table with 2^(2Nc+Npe) rows.
 * ------------------------------------------------------------------------------------------ */
static inline int64_t orc_concat_row(int32_t Q, int32_t K, int32_t PE, int Nc, int Npe) {
    return (int64_t)(((uint32_t)Q << (Nc + Npe)) | ((uint32_t)K << Npe) | (uint32_t)PE);
}

/* fill_outputs_fully_connected_seq_logic, proto:1807-1904 */
void orc_concat_forward(const float *W, const int32_t *idx, const int32_t *pidx, float *y, int64_t B, int S, int O,
                        int Nt, int Nc, int Npe, int int_mode, double rescaler) {
    int64_t T = (int64_t)1 << (2 * Nc + Npe);
    ORC_PARALLEL_FOR
    for (int64_t b = 0; b < B; b++) {
        const int32_t *ib = idx + b * S * Nt;
        for (int j = 1; j < S; j++)
            for (int t = 0; t < Nt; t++) {
                int32_t Q = ib[j * Nt + t];
                for (int o = 0; o < O; o++) {
                    double s = 0.0;
                    for (int i = 0; i < j; i++) {
                        int32_t PE = Npe > 0 ? pidx[(j - i - 1) * Nt + t] : 0;
                        s += (double)W[((int64_t)t * T + orc_concat_row(Q, ib[i * Nt + t], PE, Nc, Npe)) * O + o];
                    }
                    float *cell = y + (b * S + j) * O + o;
                    if (int_mode) *(int32_t *)cell += (int32_t)(s * ORC_DENOM * rescaler);
                    else *cell += (float)s;
                }
            }
    }
    if (int_mode) orc_int_to_float(y, B * S * O, rescaler);
}

/*
 * propagate_through_detectors_seq_fc_logic (proto:3629-3835) followed by gather_w_gradients_seq_fc_cpu_logic
 * (proto:3944-4044); loop nest = the reference's host grid: (sample, output block) outermost, then 32x32
 * pair tiles row-major, detectors, and inside a tile the query index outer / key index inner
 * (lut_runtime.cu:639-799, 32 = TILE of lut_runtime.cuh:68).
 */
void orc_concat_backward(float *W, const float *dY, const int32_t *anchors, const int32_t *idx,
                         const float *min_delta, const int32_t *min_k, const int32_t *pidx, const float *pmin,
                         const int32_t *pmin_k, float *dX, float *dPE, float *dW, int64_t B, int S, int I, int O,
                         int Nt, int Nc, int Npe, int G, double lr_meta, double ext_lr, int int_mode,
                         double rescaler) {
    int64_t T = (int64_t)1 << (2 * Nc + Npe);
    int n_ob = (O + G - 1) / G;
    int tiles = (S + 31) / 32;
    double lr = lr_meta;
    if (ext_lr >= 0) lr *= -ext_lr;
    float *target = ext_lr >= 0 ? W : dW;
    for (int pass = 0; pass < 2; pass++)  /* 0: input + positional gradients, 1: table gradients */
        for (int64_t b = 0; b < B; b++)
            for (int ob = 0; ob < n_ob; ob++) {
                int o0 = ob * G, o1 = o0 + G < O ? o0 + G : O;
                for (int ti = 0; ti < tiles; ti++)
                    for (int tj = 0; tj < tiles; tj++) {
                        if (ti > tj) continue;
                        for (int t = 0; t < Nt; t++)
                            for (int jl = 0; jl < 32; jl++)
                                for (int il = 0; il < 32; il++) {
                                    int i = ti * 32 + il, j = tj * 32 + jl;
                                    if (i >= j || i >= S || j >= S) continue;
                                    const float *dy = dY + (b * S + j) * O;
                                    int64_t ko = (b * S + i) * Nt + t, qo = (b * S + j) * Nt + t;
                                    int32_t K = idx[ko], Q = idx[qo];
                                    int32_t PE = 0, pk = -1;
                                    float pm = 0.0f;
                                    int64_t po = (int64_t)(j - i - 1) * Nt + t;
                                    if (Npe > 0) { PE = pidx[po]; pk = pmin_k[po]; pm = pmin[po]; }
                                    int64_t row = (int64_t)t * T + orc_concat_row(Q, K, PE, Nc, Npe);
                                    if (pass == 1) {
                                        for (int o = o0; o < o1; o++) {
                                            double g = (double)dy[o];
                                            if (fabs(g) > ORC_EPS) {
                                                if (int_mode) *(int32_t *)(target + row * O + o) += (int32_t)(g * lr * ORC_DENOM * rescaler);
                                                else target[row * O + o] += (float)(g * lr);
                                            }
                                        }
                                        continue;
                                    }
                                    float qm = min_delta[qo], km = min_delta[ko];
                                    int64_t alt;
                                    double du;
                                    int flip, pos;
                                    if (fabsf(qm) < fabsf(km)) {
                                        alt = (int64_t)t * T + orc_concat_row(Q ^ (1 << min_k[qo]), K, PE, Nc, Npe);
                                        du = orc_up(qm); flip = min_k[qo]; pos = j;
                                    } else {
                                        alt = (int64_t)t * T + orc_concat_row(Q, K ^ (1 << min_k[ko]), PE, Nc, Npe);
                                        du = orc_up(km); flip = min_k[ko]; pos = i;
                                    }
                                    double ms = 0.0, as = 0.0;
                                    for (int o = o0; o < o1; o++) {
                                        double g = (double)dy[o];
                                        ms += (double)W[row * O + o] * g;
                                        as += (double)W[alt * O + o] * g;
                                    }
                                    du *= ms - as;
                                    if (fabs(du) > ORC_EPS) {
                                        int32_t a1 = anchors[((int64_t)t * Nc + flip) * 2], a2 = anchors[((int64_t)t * Nc + flip) * 2 + 1];
                                        float *dx = dX + (b * S + pos) * (int64_t)I;
                                        if (int_mode) {
                                            int32_t d = (int32_t)(du * ORC_DENOM * rescaler);
                                            *(int32_t *)(dx + a1) += d;
                                            *(int32_t *)(dx + a2) -= d;
                                        } else {
                                            dx[a1] += du;
                                            dx[a2] -= du;
                                        }
                                    }
                                    if (Npe > 0 && fabsf(pm) < fabsf(qm) && fabsf(pm) < fabsf(km)) {
                                        int64_t palt = (int64_t)t * T + orc_concat_row(Q, K, PE ^ (1 << pk), Nc, Npe);
                                        double dp = orc_up(pm);
                                        double ps = 0.0;
                                        for (int o = o0; o < o1; o++) ps += (double)W[palt * O + o] * (double)dy[o];
                                        dp *= ms - ps;
                                        float *cell = dPE + po * Npe + pk;
                                        if (int_mode) *(int32_t *)cell += (int32_t)(dp * ORC_DENOM * rescaler);
                                        else *cell += dp;
                                    }
                                }
                    }
            }
    if (int_mode) {
        orc_int_to_float(dX, B * S * (int64_t)I, rescaler);
        if (dW) orc_int_to_float(dW, (int64_t)Nt * T * O, rescaler);
        if (Npe > 0) orc_int_to_float(dPE, (int64_t)(S - 1) * Nt * Npe, rescaler);
    }
}

/* ------------------------------------------------------------------------------------------
 * Concatenation-mode sequence layers with sparse lookup -> output connectivity: the pair (i < j) selects
 * lookup neuron t * T + row(i, j) as in the fully connected case, and that neuron's synapse groups are walked
 * like in the non-sequence sparse layer (same arrays: det_wbase / det_stride / det_count / det_toff / targets).
 * Host loop nest of the reference: (sample, synapse group) outermost, 32x32 pair tiles row-major, detectors,
 * inside a tile key index outer / query index inner (i = thread / TILE, j = thread % TILE).
 * ------------------------------------------------------------------------------------------ */

/* fill_outputs_sparse_seq_logic (proto:1906-2013) + fire_single_synapse_group (:215-313) */
void orc_concat_sparse_forward(const float *W, const int32_t *idx, const int32_t *pidx, float *y, int64_t B, int S, int O,
                               int Nt, int Nc, int Npe, const int64_t *det_wbase, const int32_t *det_stride,
                               const int32_t *det_count, const int32_t *det_toff, const int32_t *targets, int G,
                               int int_mode, double rescaler) {
    int max_groups = 0;
    for (int t = 0; t < Nt; t++) {
        int g = (det_count[t] + G - 1) / G;
        if (g > max_groups) max_groups = g;
    }
    int tiles = (S + 31) / 32;
    for (int64_t b = 0; b < B; b++)
        for (int ob = 0; ob < max_groups; ob++)
            for (int ti = 0; ti < tiles; ti++)
                for (int tj = 0; tj < tiles; tj++) {
                    if (ti > tj) continue;
                    for (int t = 0; t < Nt; t++) {
                        int P = det_count[t];
                        int p0 = ob * G, p1 = p0 + G < P ? p0 + G : P;
                        if (p0 >= P) continue;
                        const int32_t *tg = targets + det_toff[t];
                        for (int il = 0; il < 32; il++)
                            for (int jl = 0; jl < 32; jl++) {
                                int i = ti * 32 + il, j = tj * 32 + jl;
                                if (i >= j || i >= S || j >= S) continue;
                                int32_t K = idx[(b * S + i) * Nt + t], Q = idx[(b * S + j) * Nt + t];
                                int32_t PE = Npe > 0 ? pidx[(int64_t)(j - i - 1) * Nt + t] : 0;
                                int64_t row = det_wbase[t] + orc_concat_row(Q, K, PE, Nc, Npe) * det_stride[t];
                                float *yb = y + (b * S + j) * O;
                                for (int p = p0; p < p1; p++) {
                                    double w = (double)W[orc_syn_slot(row, p, G)];
                                    if (int_mode) *(int32_t *)(yb + tg[p]) += (int32_t)(w * ORC_DENOM * rescaler);
                                    else yb[tg[p]] += (float)w;
                                }
                            }
                    }
                }
    if (int_mode) orc_int_to_float(y, B * S * O, rescaler);
}

/* propagate_through_detectors_seq_sparse_logic (proto:3371-3627, helper accumulate_grad_sum_sparse :315-395) and
 * gather_w_gradients_seq_sparse_logic (proto:3837-3942, helper gather_weight_gradients_sparse :584-714). */
void orc_concat_sparse_backward(float *W, const float *dY, const int32_t *anchors, const int32_t *idx,
                                const float *min_delta, const int32_t *min_k, const int32_t *pidx, const float *pmin,
                                const int32_t *pmin_k, float *dX, float *dPE, float *dW, int64_t B, int S, int I, int O,
                                int Nt, int Nc, int Npe, const int64_t *det_wbase, const int32_t *det_stride,
                                const int32_t *det_count, const int32_t *det_toff, const int32_t *targets, int G,
                                int64_t n_weights, double lr_meta, double ext_lr, int int_mode, double rescaler) {
    int max_groups = 0;
    for (int t = 0; t < Nt; t++) {
        int g = (det_count[t] + G - 1) / G;
        if (g > max_groups) max_groups = g;
    }
    int tiles = (S + 31) / 32;
    double lr = lr_meta;
    if (ext_lr >= 0) lr *= -ext_lr;
    float *target = ext_lr >= 0 ? W : dW;
    for (int pass = 0; pass < 2; pass++)  /* 0: input + positional gradients, 1: table gradients */
        for (int64_t b = 0; b < B; b++)
            for (int ob = 0; ob < max_groups; ob++)
                for (int ti = 0; ti < tiles; ti++)
                    for (int tj = 0; tj < tiles; tj++) {
                        if (ti > tj) continue;
                        for (int t = 0; t < Nt; t++) {
                            int P = det_count[t];
                            int p0 = ob * G, p1 = p0 + G < P ? p0 + G : P;
                            if (p0 >= P) continue;
                            const int32_t *tg = targets + det_toff[t];
                            for (int il = 0; il < 32; il++)
                                for (int jl = 0; jl < 32; jl++) {
                                    int i = ti * 32 + il, j = tj * 32 + jl;
                                    if (i >= j || i >= S || j >= S) continue;
                                    const float *dy = dY + (b * S + j) * O;
                                    int64_t ko = (b * S + i) * Nt + t, qo = (b * S + j) * Nt + t;
                                    int32_t K = idx[ko], Q = idx[qo];
                                    int32_t PE = 0, pk = -1;
                                    float pm = 0.0f;
                                    int64_t po = (int64_t)(j - i - 1) * Nt + t;
                                    if (Npe > 0) { PE = pidx[po]; pk = pmin_k[po]; pm = pmin[po]; }
                                    int64_t row = det_wbase[t] + orc_concat_row(Q, K, PE, Nc, Npe) * det_stride[t];
                                    if (pass == 1) {
                                        for (int p = p0; p < p1; p++) {
                                            double g = (double)dy[tg[p]];
                                            if (fabs(g) > ORC_EPS) {
                                                int64_t slot = orc_syn_slot(row, p, G);
                                                if (int_mode) *(int32_t *)(target + slot) += (int32_t)(g * lr * ORC_DENOM * rescaler);
                                                else target[slot] += (float)(g * lr);
                                            }
                                        }
                                        continue;
                                    }
                                    float qm = min_delta[qo], km = min_delta[ko];
                                    int64_t alt;
                                    double du;
                                    int flip, pos;
                                    if (fabsf(qm) < fabsf(km)) {
                                        alt = det_wbase[t] + orc_concat_row(Q ^ (1 << min_k[qo]), K, PE, Nc, Npe) * det_stride[t];
                                        du = orc_up(qm); flip = min_k[qo]; pos = j;
                                    } else {
                                        alt = det_wbase[t] + orc_concat_row(Q, K ^ (1 << min_k[ko]), PE, Nc, Npe) * det_stride[t];
                                        du = orc_up(km); flip = min_k[ko]; pos = i;
                                    }
                                    double ms = 0.0, as = 0.0;
                                    for (int p = p0; p < p1; p++) ms += (double)W[orc_syn_slot(row, p, G)] * (double)dy[tg[p]];
                                    for (int p = p0; p < p1; p++) as += (double)W[orc_syn_slot(alt, p, G)] * (double)dy[tg[p]];
                                    du *= ms - as;
                                    if (fabs(du) > ORC_EPS) {
                                        int32_t a1 = anchors[((int64_t)t * Nc + flip) * 2], a2 = anchors[((int64_t)t * Nc + flip) * 2 + 1];
                                        float *dx = dX + (b * S + pos) * (int64_t)I;
                                        if (int_mode) {
                                            int32_t d = (int32_t)(du * ORC_DENOM * rescaler);
                                            *(int32_t *)(dx + a1) += d;
                                            *(int32_t *)(dx + a2) -= d;
                                        } else {
                                            dx[a1] += du;
                                            dx[a2] -= du;
                                        }
                                    }
                                    if (Npe > 0 && fabsf(pm) < fabsf(qm) && fabsf(pm) < fabsf(km)) {
                                        int64_t palt = det_wbase[t] + orc_concat_row(Q, K, PE ^ (1 << pk), Nc, Npe) * det_stride[t];
                                        double dp = orc_up(pm);
                                        double ps = 0.0;
                                        for (int p = p0; p < p1; p++) ps += (double)W[orc_syn_slot(palt, p, G)] * (double)dy[tg[p]];
                                        dp *= ms - ps;
                                        float *cell = dPE + po * Npe + pk;
                                        if (int_mode) *(int32_t *)cell += (int32_t)(dp * ORC_DENOM * rescaler);
                                        else *cell += dp;
                                    }
                                }
                        }
                    }
    if (int_mode) {
        orc_int_to_float(dX, B * S * (int64_t)I, rescaler);
        if (dW) orc_int_to_float(dW, n_weights, rescaler);
        if (Npe > 0) orc_int_to_float(dPE, (int64_t)(S - 1) * Nt * Npe, rescaler);
    }
}
