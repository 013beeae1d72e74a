// Pair evaluation shared by the product-mode kernels: a block owns one (sample, detector), stages the input
// elements its anchors read from every token once, and evaluates the S*(S-1)/2 causal pairs out of shared memory.
//
// Reference: calculate_product_lookup_index[_backprop] (lut_runtime_kernels_logic.proto:32-198).
#pragma once

#include "lutb_common.cuh"

namespace lutb {

constexpr int kMaxPairs = 16;  // anchor pairs per detector supported by the pair kernels (table of 2^16 rows)

// Per-block staging shared by forward and backward.  A block owns one (sample, detector): it gathers
// the 2*Nc input elements its anchors read from every token of the sample once, so the S*(S-1)/2 pair
// evaluations run entirely out of shared memory.
struct PairStage {
    float *U;        // [S][ustride]  U[s][2k+e] = x[b, s, element(k, e)] for ends that read a token
    float *PE;       // [S-1][pstride] positional embedding of (distance, this detector)
    int ustride, pstride;
    // per anchor end (shared memory): source (0: token i, 1: token j, 2: positional embedding, 3: unused
    // pair) and element inside that source
    int *comp;       // [2 * kMaxPairs]
    int *elem;       // [2 * kMaxPairs]
    float *scratch;  // 16-byte aligned start of the per-warp scratch area behind the staged data
};

__device__ __forceinline__ void decode_anchor(int32_t id, bool sliced, int e1, int e2, int &comp, int &elem) {
    if (id == kNoAnchor) { comp = 3; elem = 0; return; }
    if (sliced) { elem = id / 3; comp = id % 3; }
    else if (id < e1) { comp = 0; elem = id; }
    else if (id < e1 + e2) { comp = 1; elem = id - e1; }
    else { comp = 2; elem = id - e1 - e2; }
}

// Evaluates the anchors of one pair (i, j).  Returns the table index; when TRACK also the first anchor of
// minimal |delta| (strict '<' from FLT_MAX, reference proto:166-173) and that delta.
template <bool TRACK>
__device__ __forceinline__ int32_t eval_pair(const PairStage &st, int n_anchors, int i, int j, float cmp_eps,
                                             int &kmin, float &dmin) {
    const float *ui = st.U + i * st.ustride;
    const float *uj = st.U + j * st.ustride;
    const float *pe = st.PE + (j - i - 1) * st.pstride;
    int32_t li = 0;
    float md = 3.402823466e+38F;
    int mk = -1;
    for (int k = 0; k < n_anchors; k++) {
        const int c1 = st.comp[2 * k], c2 = st.comp[2 * k + 1];
        if (c1 == 3 || c2 == 3) continue;
        const float v1 = c1 == 0 ? ui[2 * k] : (c1 == 1 ? uj[2 * k] : pe[st.elem[2 * k]]);
        const float v2 = c2 == 0 ? ui[2 * k + 1] : (c2 == 1 ? uj[2 * k + 1] : pe[st.elem[2 * k + 1]]);
        const float d = __fsub_rn(v1, v2);
        if (greater_than_zero(d, cmp_eps)) li |= (1 << k);
        if (TRACK && fabsf(d) < fabsf(md)) { md = d; mk = k; }
    }
    if (TRACK) { kmin = mk; dmin = md; }
    return li;
}

__device__ __forceinline__ void stage_pairs(PairStage &st, float *smem, const float *__restrict__ x1b,
                                            const float *__restrict__ x2b, const float *__restrict__ pe,
                                            const int32_t *__restrict__ anchors_t, int S, int e1, int e2, int npe,
                                            int n_anchors, int n_detectors, int t, bool sliced) {
    st.ustride = (2 * n_anchors) | 1;  // odd strides keep the per-token reads conflict free
    st.pstride = npe | 1;
    st.comp = reinterpret_cast<int *>(smem);
    st.elem = st.comp + 2 * kMaxPairs;
    st.U = smem + 4 * kMaxPairs;
    st.PE = st.U + S * st.ustride;
    st.scratch = st.PE + (((S - 1) * st.pstride + 3) & ~3) + ((4 - ((S * st.ustride) & 3)) & 3);
    if (threadIdx.x < 2 * kMaxPairs) {
        int c = 3, e = 0;
        if (threadIdx.x < 2 * n_anchors) decode_anchor(__ldg(anchors_t + threadIdx.x), sliced, e1, e2, c, e);
        st.comp[threadIdx.x] = c;
        st.elem[threadIdx.x] = e;
    }
    __syncthreads();
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
}

// Note on U: an end with source "token i" is read from row i of U, an end with source "token j" from
// row j; both rows hold x at the end's element, taken from x1 for "i" ends and x2 for "j" ends.

// floats of shared memory stage_pairs lays out in front of the per-warp scratch area
inline size_t pair_stage_floats(int S, int n_anchors, int npe) {
    // anchor metadata + U + PE, plus slack for the 16-byte alignment of the scratch area behind them
    return 4 * kMaxPairs + (size_t)S * ((2 * n_anchors) | 1) + (size_t)(S > 1 ? S - 1 : 0) * (npe | 1) + 8;
}

}  // namespace lutb
