// Pair evaluation shared by the product-mode kernels: a block owns one (sample, detector), stages the input
// elements its anchors read from every token once, and evaluates the S*(S-1)/2 causal pairs out of shared memory.
//
// An anchor pair compares two elements of the virtual vector [x_i | x_j | pe(j-i-1)].  Anchors whose two ends
// read the same source (both the key token i, both the query token j, or both the positional embedding) do not
// depend on the pair: their bits and their first-minimum |delta| are evaluated once per token (or distance)
// while staging.  Only the "mixed" anchors are evaluated per pair.
//
// Reference: calculate_product_lookup_index[_backprop] (lut_runtime_kernels_logic.proto:32-198).
#pragma once

#include "lutb_common.cuh"

namespace lutb {

constexpr int kMaxPairs = 16;  // anchor pairs per detector supported by the pair kernels (table of 2^16 rows)
constexpr float kFltMax = 3.402823466e+38F;

struct PairStage {
    float *U;        // [S][ustride]  U[s][2k+e] = x[b, s, element(k, e)] for ends that read a token
    float *PE;       // [S-1][pstride] positional embedding of (distance, this detector); PE = U + S * ustride
    int ustride, pstride;
    // per anchor end (shared memory): source (0: token i, 1: token j, 2: positional embedding, 3: unused
    // pair) and element inside that source
    int *comp;       // [2 * kMaxPairs]
    int *elem;       // [2 * kMaxPairs]
    // mixed anchors: {k, source of end 0 | source of end 1 << 2, column of end 0, column of end 1}; columns are
    // offsets from U (row offset of the source added per pair)
    int4 *mixed;     // [kMaxPairs]
    int n_mixed;
    // the same anchors as address arithmetic (MixedPlan below): end e of mixed anchor m reads
    // U[i * lin[m].x/.y + j * jmul + off] with {jmul, off} = jplan[2 * m + e]
    int2 *lin;       // [kMaxPairs]  i-multipliers of the two ends
    int2 *jplan;     // [2 * kMaxPairs]
    // pair-independent anchors, per token / distance: bits | (first-min anchor + 1) << 16, and that delta
    uint32_t *tokI, *tokJ, *posP;
    float *tokId, *tokJd, *posPd;
    float *scratch;  // 16-byte aligned start of the per-warp scratch area behind the staged data
};

__device__ __forceinline__ void decode_anchor(int32_t id, bool sliced, int e1, int e2, int &comp, int &elem) {
    if (id == kNoAnchor) { comp = 3; elem = 0; return; }
    if (sliced) { elem = id / 3; comp = id % 3; }
    else if (id < e1) { comp = 0; elem = id; }
    else if (id < e1 + e2) { comp = 1; elem = id - e1; }
    else { comp = 2; elem = id - e1 - e2; }
}

// Candidate (d, k) replaces the running first-minimum (md, mk) when |d| is smaller, or equal with a smaller
// anchor number: together with the strict '<' inside each group this reproduces "first anchor of minimal
// |delta| in anchor order, starting from FLT_MAX" (reference proto:166-173) for any evaluation order.
__device__ __forceinline__ void consider(float &md, int &mk, float d, int k) {
    const float a = fabsf(d), b = fabsf(md);
    if (k >= 0 && (a < b || (a == b && mk >= 0 && k < mk))) { md = d; mk = k; }
}

// Evaluates the anchors of one pair (i, j).  Returns the table index; when TRACK also the first anchor of
// minimal |delta| and that delta (kmin = -1 when the detector has no usable anchor).
template <bool TRACK>
__device__ __forceinline__ int32_t eval_pair(const PairStage &st, int /*n_anchors*/, int i, int j, float cmp_eps,
                                             int &kmin, float &dmin) {
    const int dist = j - i - 1;
    const uint32_t pi = st.tokI[i], pj = st.tokJ[j], pp = st.posP[dist];
    int32_t li = (int32_t)((pi | pj | pp) & 0xffffu);
    float md = kFltMax;
    int mk = -1;
    if (TRACK) {
        consider(md, mk, st.tokId[i], (int)(pi >> 16) - 1);
        consider(md, mk, st.tokJd[j], (int)(pj >> 16) - 1);
        consider(md, mk, st.posPd[dist], (int)(pp >> 16) - 1);
    }
    const int ri = i * st.ustride, rj = j * st.ustride, rp = dist * st.pstride;
    for (int m = 0; m < st.n_mixed; m++) {
        const int4 e = st.mixed[m];
        const int s1 = e.y & 3, s2 = e.y >> 2;
        const float v1 = st.U[(s1 == 0 ? ri : (s1 == 1 ? rj : rp)) + e.z];
        const float v2 = st.U[(s2 == 0 ? ri : (s2 == 1 ? rj : rp)) + e.w];
        const float d = __fsub_rn(v1, v2);
        if (greater_than_zero(d, cmp_eps)) li |= (1 << e.x);
        if (TRACK) consider(md, mk, d, e.x);
    }
    if (TRACK) { kmin = mk; dmin = md; }
    return li;
}

// The mixed anchors of a detector held in registers for one query j: end e of anchor m reads U[i * imul + base],
// base = j * jmul + off folded per query (a source row is i, j or j - i - 1, so the address is linear in i).  MAXM
// bounds the unrolled loops; anchors beyond n are skipped by a block-uniform test.
template <int MAXM>
struct MixedPlan {
    int n;
    int k[MAXM];
    int imul1[MAXM], imul2[MAXM];
    int base1[MAXM], base2[MAXM];

    __device__ __forceinline__ void load(const PairStage &st) {
        n = st.n_mixed;
#pragma unroll
        for (int m = 0; m < MAXM; m++) {
            k[m] = 0; imul1[m] = imul2[m] = 0; base1[m] = base2[m] = 0;
            if (m < n) {
                k[m] = st.mixed[m].x;
                const int2 l = st.lin[m];
                imul1[m] = l.x;
                imul2[m] = l.y;
            }
        }
    }
    __device__ __forceinline__ void set_query(const PairStage &st, int j) {
#pragma unroll
        for (int m = 0; m < MAXM; m++)
            if (m < n) {
                const int2 p1 = st.jplan[2 * m], p2 = st.jplan[2 * m + 1];
                base1[m] = j * p1.x + p1.y;
                base2[m] = j * p2.x + p2.y;
            }
    }
};

// Per-query part of a pair: the query token's pair-independent anchors.
struct QueryPart {
    uint32_t word;
    float delta;
};
__device__ __forceinline__ QueryPart query_part(const PairStage &st, int j) { return QueryPart{st.tokJ[j], st.tokJd[j]}; }

// eval_pair with the mixed anchors taken from a MixedPlan and the query token's part loaded once per query: the same
// comparisons on the same operands (the first-minimum rule of `consider` does not depend on the evaluation order).
template <bool TRACK, int MAXM>
__device__ __forceinline__ int32_t eval_pair_planned(const PairStage &st, const MixedPlan<MAXM> &mp, const QueryPart &qp,
                                                     int i, int j, float cmp_eps, int &kmin, float &dmin) {
    const int dist = j - i - 1;
    const uint32_t pi = st.tokI[i], pp = st.posP[dist];
    int32_t li = (int32_t)((pi | qp.word | pp) & 0xffffu);
    float md = kFltMax;
    int mk = -1;
    if (TRACK) {
        consider(md, mk, st.tokId[i], (int)(pi >> 16) - 1);
        consider(md, mk, qp.delta, (int)(qp.word >> 16) - 1);
        consider(md, mk, st.posPd[dist], (int)(pp >> 16) - 1);
    }
#pragma unroll
    for (int m = 0; m < MAXM; m++) {
        if (m < mp.n) {
            const float d = __fsub_rn(st.U[i * mp.imul1[m] + mp.base1[m]], st.U[i * mp.imul2[m] + mp.base2[m]]);
            if (greater_than_zero(d, cmp_eps)) li |= 1 << mp.k[m];
            if (TRACK) consider(md, mk, d, mp.k[m]);
        }
    }
    if (TRACK) { kmin = mk; dmin = md; }
    return li;
}

// ints of shared memory stage_pairs lays out in front of the per-warp scratch area
inline size_t pair_stage_floats(int S, int n_anchors, int npe) {
    // anchor metadata + U + PE + per-token / per-distance tables, plus slack for 16-byte alignment
    return 14 * kMaxPairs + (size_t)S * ((2 * n_anchors) | 1) + (size_t)(S > 1 ? S - 1 : 0) * (npe | 1) + 6 * (size_t)S + 12;
}

__device__ __forceinline__ void stage_pairs(PairStage &st, float *smem, const float *__restrict__ x1b,
                                            const float *__restrict__ x2b, const float *__restrict__ pe,
                                            const int32_t *__restrict__ anchors_t, int S, int e1, int e2, int npe,
                                            int n_anchors, int n_detectors, int t, bool sliced, float cmp_eps) {
    st.ustride = (2 * n_anchors) | 1;  // odd strides keep the per-token reads conflict free
    st.pstride = npe | 1;
    st.mixed = reinterpret_cast<int4 *>(smem);
    st.comp = reinterpret_cast<int *>(smem) + 4 * kMaxPairs;
    st.elem = st.comp + 2 * kMaxPairs;
    st.lin = reinterpret_cast<int2 *>(smem + 8 * kMaxPairs);
    st.jplan = reinterpret_cast<int2 *>(smem + 10 * kMaxPairs);
    st.U = smem + 14 * kMaxPairs;
    st.PE = st.U + S * st.ustride;
    float *p = st.PE + (S - 1) * st.pstride;
    st.tokI = reinterpret_cast<uint32_t *>(p); p += S;
    st.tokJ = reinterpret_cast<uint32_t *>(p); p += S;
    st.posP = reinterpret_cast<uint32_t *>(p); p += S;
    st.tokId = p; p += S;
    st.tokJd = p; p += S;
    st.posPd = p; p += S;
    st.scratch = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(p) + 15) & ~(uintptr_t)15);
    __shared__ int n_mixed_s;
    if (threadIdx.x < 2 * kMaxPairs) {
        int c = 3, e = 0;
        if (threadIdx.x < 2 * n_anchors) decode_anchor(__ldg(anchors_t + threadIdx.x), sliced, e1, e2, c, e);
        st.comp[threadIdx.x] = c;
        st.elem[threadIdx.x] = e;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int nm = 0;
        const int pe_col = S * st.ustride;
        for (int k = 0; k < n_anchors; k++) {
            const int c1 = st.comp[2 * k], c2 = st.comp[2 * k + 1];
            if (c1 == 3 || c2 == 3 || c1 == c2) continue;
            const int col1 = c1 == 2 ? pe_col + st.elem[2 * k] : 2 * k;
            const int col2 = c2 == 2 ? pe_col + st.elem[2 * k + 1] : 2 * k + 1;
            // U[(row of the source) * stride + col] with row = i, j or j - i - 1: linear in i and j
            const int cs[2] = {c1, c2}, cols[2] = {col1, col2};
            int imul[2];
            for (int e = 0; e < 2; e++) {
                const int a = cs[e] == 0 ? st.ustride : 0, b = cs[e] == 1 ? st.ustride : 0;
                const int c = cs[e] == 2 ? st.pstride : 0;
                imul[e] = a - c;
                st.jplan[2 * nm + e] = make_int2(b + c, cols[e] - c);
            }
            st.lin[nm] = make_int2(imul[0], imul[1]);
            st.mixed[nm++] = make_int4(k, c1 | (c2 << 2), col1, col2);
        }
        n_mixed_s = nm;
    }
    for (int w = threadIdx.x; w < S * 2 * n_anchors; w += blockDim.x) {
        const int s = w / (2 * n_anchors), q = w - s * (2 * n_anchors);
        float v = 0.f;
        // an end reads the same element whether its token plays the "i" or the "j" part
        if (st.comp[q] == 0) v = __ldg(x1b + (size_t)s * e1 + st.elem[q]);
        else if (st.comp[q] == 1) v = __ldg(x2b + (size_t)s * e2 + st.elem[q]);
        st.U[s * st.ustride + q] = v;
    }
    if (npe > 0) {
        for (int w = threadIdx.x; w < (S - 1) * npe; w += blockDim.x) {
            const int d = w / npe, c = w - d * npe;
            st.PE[d * st.pstride + c] = __ldg(pe + ((size_t)d * n_detectors + t) * npe + c);
        }
    }
    __syncthreads();
    st.n_mixed = n_mixed_s;
    // pair-independent anchors: source 0 per key token, source 1 per query token, source 2 per distance
    for (int w = threadIdx.x; w < 3 * S; w += blockDim.x) {
        const int src = w / S, s = w - src * S;
        if (src == 2 && s >= S - 1) continue;
        uint32_t bits = 0;
        float md = kFltMax;
        int mk = -1;
        for (int k = 0; k < n_anchors; k++) {
            if (st.comp[2 * k] != src || st.comp[2 * k + 1] != src) continue;
            float v1, v2;
            if (src == 2) {
                v1 = st.PE[s * st.pstride + st.elem[2 * k]];
                v2 = st.PE[s * st.pstride + st.elem[2 * k + 1]];
            } else {
                v1 = st.U[s * st.ustride + 2 * k];
                v2 = st.U[s * st.ustride + 2 * k + 1];
            }
            const float d = __fsub_rn(v1, v2);
            if (greater_than_zero(d, cmp_eps)) bits |= (1u << k);
            if (fabsf(d) < fabsf(md)) { md = d; mk = k; }
        }
        uint32_t *word = src == 0 ? st.tokI : (src == 1 ? st.tokJ : st.posP);
        float *delta = src == 0 ? st.tokId : (src == 1 ? st.tokJd : st.posPd);
        word[s] = bits | ((uint32_t)(mk + 1) << 16);
        delta[s] = md;
    }
    __syncthreads();
}

// Note on U: an end with source "token i" is read from row i of U, an end with source "token j" from
// row j; both rows hold x at the end's element, taken from x1 for "i" ends and x2 for "j" ends.

}  // namespace lutb
