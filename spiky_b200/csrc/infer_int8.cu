// Forward-only inference with int8 tables and one fp32 scale per table.  The reference has no quantised
// tables; the arithmetic is defined as its int32 fixed-point accumulator mode (LUTDataManagerI, forward:
// fill_outputs_non_seq_fc_logic with INTEGERS_INSTEAD_OF_FLOATS, lut_runtime_kernels_logic.proto:1214-1299)
// applied to the de-quantised table f32(scale[t] * q[t][row][o]): inside every block of `backward_group`
// detectors the selected entries are summed in double, the block sum is scaled by 0xFFFFF * int_rescaler,
// truncated toward zero and added to an int32 accumulator.  Integer accumulators make the result independent
// of summation order, so detector shards computed on different GPUs combine bit-exactly with an integer
// all-reduce before the final conversion to fp32 (convert_integers_to_floats_logic, proto:200-213).
//
// Two de-quantisation rules (cfg-independent argument `dequant`):
//   LUTB_INT8_DEQUANT_F32    entry = f32(scale * q): exactly the fp32 table the reference would be given; costs two
//                            conversions per entry (int8 -> fp32 -> fp64) on the conversion unit, which bound the kernel
//   LUTB_INT8_DEQUANT_EXACT  entry = scale * q as an exact real (24 x 8 bit product, exact in fp64): one int8 -> fp64
//                            conversion and one fp64 FMA per entry (the scale is converted once per detector);
//                            building the double from integer operations instead measured the same within 3 %
#include "lutb_common.cuh"
#include "nonseq_fc.cuh"

namespace lutb {

// One warp per (sample, 128-output chunk): lane groups of LG lanes cover a row 4 int8 at a time (one 32-bit
// load per lane), NG = 32 / LG groups take the detectors of a block round-robin; the per-group double sums
// are exact (<= 32 fp32 terms of similar magnitude), so combining them across groups before the truncation
// gives the same bits as the sequential sum.
template <int LG, bool EXACT>
__global__ void __launch_bounds__(256) int8_gather_kernel(const int8_t *__restrict__ Q, const float *__restrict__ scales,
                                                         const int32_t *__restrict__ idx, int32_t *__restrict__ acc,
                                                         int64_t batch, int n_outputs, int n_detectors, int table_rows,
                                                         int det_block, double fixed_scale, int det_begin, int det_end) {
    constexpr int NG = 32 / LG;   // lane groups; group g takes detectors g, g + NG, ... of every 32
    constexpr int IT = 32 / NG;   // = LG row loads per lane and 32 detectors, all issued before the first use
    const int lane = threadIdx.x & 31;
    const int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= batch) return;
    const int g = lane / LG, j = lane - g * LG;
    const int col = blockIdx.y * (LG * 4) + j * 4;
    const bool active = col < n_outputs;   // n_outputs is a multiple of 4
    const int32_t *idx_b = idx + b * n_detectors;
    const int8_t *Qc = Q + col;
    int32_t iacc[4] = {0, 0, 0, 0};
    // [det_begin, det_end) starts on a block boundary: one launch covers a range of detectors whose tables stay in L2
    for (int tb = det_begin; tb < det_end; tb += det_block) {
        const int tend = min(tb + det_block, det_end);
        double s[4] = {0.0, 0.0, 0.0, 0.0};
        for (int t0 = tb; t0 < tend; t0 += 32) {
            const int nvalid = min(32, tend - t0);
            int32_t my_idx = 0;
            float my_scale = 0.f;
            if (lane < nvalid) { my_idx = __ldg(idx_b + t0 + lane); my_scale = __ldg(scales + t0 + lane); }
            int32_t packed[IT];
#pragma unroll
            for (int i = 0; i < IT; i++) {
                const int d = i * NG + g;
                const int32_t li = __shfl_sync(0xffffffffu, my_idx, d);
                packed[i] = (active && d < nvalid)
                                ? __ldg(reinterpret_cast<const int32_t *>(Qc + ((size_t)(t0 + d) * table_rows + li) * n_outputs))
                                : 0;
            }
#pragma unroll
            for (int i = 0; i < IT; i++) {
                const float sc = __shfl_sync(0xffffffffu, my_scale, i * NG + g);   // 0 beyond nvalid
                if (EXACT) {
                    const double sd = (double)sc;
                    s[0] = fma(sd, (double)(int8_t)(packed[i] & 0xff), s[0]);
                    s[1] = fma(sd, (double)(int8_t)((packed[i] >> 8) & 0xff), s[1]);
                    s[2] = fma(sd, (double)(int8_t)((packed[i] >> 16) & 0xff), s[2]);
                    s[3] = fma(sd, (double)(int8_t)((packed[i] >> 24) & 0xff), s[3]);
                } else {
                    s[0] += (double)__fmul_rn(sc, (float)(int8_t)(packed[i] & 0xff));
                    s[1] += (double)__fmul_rn(sc, (float)(int8_t)((packed[i] >> 8) & 0xff));
                    s[2] += (double)__fmul_rn(sc, (float)(int8_t)((packed[i] >> 16) & 0xff));
                    s[3] += (double)__fmul_rn(sc, (float)(int8_t)((packed[i] >> 24) & 0xff));
                }
            }
        }
#pragma unroll
        for (int m = LG; m < 32; m <<= 1) {
#pragma unroll
            for (int e = 0; e < 4; e++) s[e] += __shfl_xor_sync(0xffffffffu, s[e], m);
        }
#pragma unroll
        for (int e = 0; e < 4; e++) iacc[e] += to_fixed(s[e], fixed_scale);
    }
    if (active && g == 0) {
        int32_t *out = acc + b * n_outputs + col;
#pragma unroll
        for (int e = 0; e < 4; e++) out[e] += iacc[e];
    }
}

}  // namespace lutb

using namespace lutb;

extern "C" int lutb_infer_int8_accumulate(const lutb_layer_cfg *cfg, int64_t batch, const int8_t *q_tables,
                                          const float *scales, const float *x, const int32_t *anchors,
                                          int32_t *acc, int32_t *idx, int dequant, void *stream) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->seq_len == 1, LUTB_ERR_MODE, "int8 inference is defined for non-sequence layers");
    LUTB_REQUIRE(batch > 0, LUTB_ERR_SHAPE, "batch_size == 0");
    LUTB_REQUIRE(q_tables && scales && x && anchors && acc && idx, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE(cfg->n_outputs % 4 == 0, LUTB_ERR_SHAPE, "int8 inference needs n_outputs to be a multiple of 4");
    LUTB_REQUIRE((reinterpret_cast<uintptr_t>(q_tables) & 3) == 0, LUTB_ERR_ALIGN, "q_tables must be 4-byte aligned");
    LUTB_REQUIRE(cfg->int_rescaler > 0.0, LUTB_ERR_MODE, "int_rescaler must be positive");
    LUTB_REQUIRE(dequant == LUTB_INT8_DEQUANT_F32 || dequant == LUTB_INT8_DEQUANT_EXACT, LUTB_ERR_MODE,
                 "unknown de-quantisation rule %d", dequant);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = launch_check_detectors(x, batch, cfg->n_inputs, anchors, cfg->n_detectors, cfg->n_anchors, cfg->cmp_eps, idx,
                                nullptr, nullptr, st);
    if (rc) return rc;
    const int vpr = cfg->n_outputs / 4;
    int lanes = 1;
    while (lanes < 32 && lanes < vpr) lanes <<= 1;
    const int n_chunks = (cfg->n_outputs + lanes * 4 - 1) / (lanes * 4);
    const int64_t blocks = (batch + 7) / 8;
    LUTB_REQUIRE(blocks <= 0x7FFFFFFF && n_chunks <= 65535, LUTB_ERR_SHAPE, "grid too large");
    const dim3 grid((unsigned)blocks, (unsigned)n_chunks);
    // detector ranges of at most 40 MB of tables (whole blocks): the rows of a range are fetched from DRAM once and
    // then served by L2 while the batch streams through
    const size_t table_bytes = ((size_t)1 << cfg->n_anchors) * cfg->n_outputs;
    int64_t per_range = (int64_t)((size_t)(40u << 20) / table_bytes);
    per_range = per_range / cfg->backward_group * cfg->backward_group;
    if (per_range < cfg->backward_group) per_range = cfg->backward_group;
    for (int64_t t0 = 0; t0 < cfg->n_detectors; t0 += per_range) {
    const int det_begin = (int)t0, det_end = (int)(t0 + per_range < cfg->n_detectors ? t0 + per_range : cfg->n_detectors);
    KernelScope scope(K_INT8_GATHER, st);
#define LUTB_INT8(LGV)                                                                                                  \
    do {                                                                                                               \
        if (dequant == LUTB_INT8_DEQUANT_EXACT)                                                                        \
            int8_gather_kernel<LGV, true><<<grid, 256, 0, st>>>(q_tables, scales, idx, acc, batch, cfg->n_outputs,     \
                cfg->n_detectors, 1 << cfg->n_anchors, cfg->backward_group, cfg->int_rescaler, det_begin, det_end);    \
        else                                                                                                           \
            int8_gather_kernel<LGV, false><<<grid, 256, 0, st>>>(q_tables, scales, idx, acc, batch, cfg->n_outputs,    \
                cfg->n_detectors, 1 << cfg->n_anchors, cfg->backward_group, cfg->int_rescaler, det_begin, det_end);    \
    } while (0)
    switch (lanes) {
        case 32: LUTB_INT8(32); break;
        case 16: LUTB_INT8(16); break;
        case 8: LUTB_INT8(8); break;
        case 4: LUTB_INT8(4); break;
        case 2: LUTB_INT8(2); break;
        default: LUTB_INT8(1); break;
    }
    LUTB_LAUNCH_CHECK();
    }
#undef LUTB_INT8
    return LUTB_OK;
}

extern "C" int lutb_fixed_to_float(float *buffer, int64_t n, double int_rescaler, void *stream) {
    LUTB_REQUIRE(buffer != nullptr, LUTB_ERR_NULL, "buffer is NULL");
    LUTB_REQUIRE(n >= 0 && int_rescaler > 0.0, LUTB_ERR_SHAPE, "bad size or rescaler");
    return launch_fixed_to_float(buffer, n, int_rescaler, static_cast<cudaStream_t>(stream));
}
