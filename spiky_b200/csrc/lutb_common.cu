// Error reporting, configuration checks and small utility kernels shared by all entry points.
#include <stdarg.h>
#include <string.h>

#include "lutb_common.cuh"

namespace lutb {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

DeviceInfo device_info() {
    static int sm_counts[64] = {0};
    DeviceInfo d{0, 0};
    if (cudaGetDevice(&d.device) != cudaSuccess) return d;
    if (d.device < 64 && sm_counts[d.device] > 0) {
        d.sm_count = sm_counts[d.device];
        return d;
    }
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d.device) != cudaSuccess || n <= 0) n = 148;
    if (d.device < 64) sm_counts[d.device] = n;
    d.sm_count = n;
    return d;
}

int validate_cfg(const lutb_layer_cfg *cfg) {
    LUTB_REQUIRE(cfg != nullptr, LUTB_ERR_NULL, "cfg is NULL");
    LUTB_REQUIRE(cfg->n_inputs > 0, LUTB_ERR_SHAPE, "n_inputs == 0");
    LUTB_REQUIRE(cfg->n_outputs > 0, LUTB_ERR_SHAPE, "n_outputs == 0");
    LUTB_REQUIRE(cfg->n_detectors > 0, LUTB_ERR_SHAPE, "n_detectors == 0");
    LUTB_REQUIRE(cfg->n_anchors > 0 && cfg->n_anchors <= 30, LUTB_ERR_SHAPE, "n_anchors_per_detector must be in 1..30");
    LUTB_REQUIRE(cfg->seq_len > 0, LUTB_ERR_SHAPE, "sequence_length == 0");
    LUTB_REQUIRE(cfg->pos_dim >= 0, LUTB_ERR_SHAPE, "positional_dim < 0");
    LUTB_REQUIRE(cfg->forward_group > 0, LUTB_ERR_SHAPE, "forward_group_size == 0");
    LUTB_REQUIRE(cfg->backward_group > 0, LUTB_ERR_SHAPE, "backward_group_size == 0");
    LUTB_REQUIRE(cfg->int_mode == 0 || cfg->int_mode == 1, LUTB_ERR_MODE, "int_mode must be 0 or 1");
    LUTB_REQUIRE(cfg->int_mode == 0 || cfg->int_rescaler > 0.0, LUTB_ERR_MODE, "int_rescaler must be positive");
    return LUTB_OK;
}

__global__ void fixed_to_float_kernel(float *buf, int64_t n, double rescaler) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        double y = (double)__float_as_int(buf[i]) * kDenomRecip;
        buf[i] = (float)(y / rescaler);
    }
}

int launch_fixed_to_float(float *buf, int64_t n, double rescaler, cudaStream_t stream) {
    if (n <= 0) return LUTB_OK;
    int64_t blocks = (n + 255) / 256;
    int64_t cap = (int64_t)device_info().sm_count * 16;
    if (blocks > cap) blocks = cap;
    fixed_to_float_kernel<<<(unsigned)blocks, 256, 0, stream>>>(buf, n, rescaler);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

}  // namespace lutb

extern "C" int lutb_version(void) { return 100; }
extern "C" const char *lutb_last_error(void) { return lutb::g_error; }
