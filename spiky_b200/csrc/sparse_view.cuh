// Device-side view of the sparse lookup -> output index (lutb_sparse_index) shared by the sparse-layer kernels.
#pragma once

#include "lutb_common.cuh"

namespace lutb {

struct SparseView {
    const int64_t *det_wbase;
    const int32_t *det_stride;
    const int32_t *det_count;
    const int32_t *det_sstart;
    const int32_t *syn_target;
    const int4 *chunks;   // two int4 per chunk, see lutb_sparse_index::chunk_info
    int64_t n_chunks;
    int32_t group;
    int32_t group_shift;  // log2(group) when group is a power of two, else -1
};

__device__ __forceinline__ int hole_offset(int p, const SparseView &sp) {
    // two unused slots in front of every group of `group` synapses (the first pair lies before the row base)
    return 2 * (sp.group_shift >= 0 ? (p >> sp.group_shift) : (p / sp.group));
}

struct ChunkStatic {
    int det0, ndet, toff, P, stride, table;
    int64_t wbase0;
};

__device__ __forceinline__ ChunkStatic load_chunk(const SparseView &sp, int64_t c) {
    const int4 a = __ldg(sp.chunks + 2 * c);
    const int4 w = __ldg(sp.chunks + 2 * c + 1);
    ChunkStatic cs;
    cs.det0 = a.x; cs.ndet = a.y; cs.toff = a.z; cs.P = a.w;
    cs.stride = w.x; cs.table = w.y;
    cs.wbase0 = (int64_t)(((uint64_t)(uint32_t)w.w << 32) | (uint32_t)w.z);
    return cs;
}

inline SparseView make_view(const lutb_sparse_index *sp) {
    SparseView v;
    v.det_wbase = sp->det_wbase; v.det_stride = sp->det_stride; v.det_count = sp->det_count;
    v.det_sstart = sp->det_sstart; v.syn_target = sp->syn_target;
    v.chunks = reinterpret_cast<const int4 *>(sp->chunk_info); v.n_chunks = sp->n_chunks; v.group = sp->group_size;
    v.group_shift = -1;
    for (int s = 0; s < 31; s++) if ((1 << s) == sp->group_size) v.group_shift = s;
    return v;
}


}  // namespace lutb
