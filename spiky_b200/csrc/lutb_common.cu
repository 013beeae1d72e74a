// Error reporting, configuration checks and small utility kernels shared by all entry points.
#include <stdarg.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <vector>

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
    KernelScope scope(K_FIXED_TO_FLOAT, stream);
    fixed_to_float_kernel<<<(unsigned)blocks, 256, 0, stream>>>(buf, n, rescaler);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

// ------------------------------------------------------------------------------ profiler
static const char *const kKernelNames[K_COUNT] = {
    "check_detectors", "fc_gather_forward", "fc_input_grad", "fc_weight_grad", "fixed_to_float",
    "sparse_forward", "sparse_input_grad", "sparse_weight_grad", "sparse_backward_fused",
    "product_forward", "product_backward", "product_weight_update",
    "check_positional", "concat_forward", "concat_backward", "concat_weight_update",
    "int8_gather",
    "product_hist", "product_hist_forward", "product_row_dots", "product_route", "product_hist_weight_grad",
    "dense_to_sparse", "fp32_gemm", "peer_sgd_update", "peer_barrier", "peer_broadcast",
};

struct EventPair {
    cudaEvent_t start, stop;
    int id;
};
static std::mutex g_prof_mutex;
static std::atomic<int> g_prof_enabled{0};
static std::atomic<long long> g_launches[K_COUNT];
static std::vector<EventPair> g_pairs;      // recorded since the last reset
static std::vector<EventPair> g_free;       // recycled events
static double g_total_ms[K_COUNT];           // resolved time
static long long g_timed[K_COUNT];           // launches with resolved time
constexpr size_t kMaxPendingPairs = 1 << 16;

static thread_local int g_no_events = 0;
NoEventsGuard::NoEventsGuard() { ++g_no_events; }
NoEventsGuard::~NoEventsGuard() { --g_no_events; }

KernelScope::KernelScope(KernelId id, cudaStream_t stream) : stream_(stream), stop_(nullptr) {
    g_launches[id].fetch_add(1, std::memory_order_relaxed);
    if (!g_prof_enabled.load(std::memory_order_relaxed) || g_no_events > 0) return;
    std::lock_guard<std::mutex> lock(g_prof_mutex);
    if (g_pairs.size() >= kMaxPendingPairs) return;
    EventPair p;
    if (!g_free.empty()) {
        p = g_free.back();
        g_free.pop_back();
    } else {
        if (cudaEventCreate(&p.start) != cudaSuccess) return;
        if (cudaEventCreate(&p.stop) != cudaSuccess) { cudaEventDestroy(p.start); return; }
    }
    p.id = id;
    cudaEventRecord(p.start, stream);
    g_pairs.push_back(p);
    stop_ = p.stop;
}

KernelScope::~KernelScope() {
    if (stop_) cudaEventRecord(stop_, stream_);
}

static void resolve_pending_locked() {
    for (EventPair &p : g_pairs) {
        float ms = 0.f;
        if (cudaEventSynchronize(p.stop) == cudaSuccess && cudaEventElapsedTime(&ms, p.start, p.stop) == cudaSuccess) {
            g_total_ms[p.id] += ms;
            g_timed[p.id] += 1;
        }
        g_free.push_back(p);
    }
    g_pairs.clear();
}

}  // namespace lutb

extern "C" int lutb_profiler_enable(int on) {
    lutb::g_prof_enabled.store(on ? 1 : 0);
    return LUTB_OK;
}

extern "C" int lutb_profiler_reset(void) {
    std::lock_guard<std::mutex> lock(lutb::g_prof_mutex);
    lutb::resolve_pending_locked();
    for (int i = 0; i < lutb::K_COUNT; i++) {
        lutb::g_total_ms[i] = 0.0;
        lutb::g_timed[i] = 0;
        lutb::g_launches[i].store(0);
    }
    return LUTB_OK;
}

extern "C" int lutb_profiler_kernel_count(void) { return lutb::K_COUNT; }

extern "C" const char *lutb_profiler_kernel_name(int kernel_id) {
    return (kernel_id >= 0 && kernel_id < lutb::K_COUNT) ? lutb::kKernelNames[kernel_id] : "";
}

extern "C" int lutb_profiler_read(int kernel_id, double *total_ms, int64_t *timed_launches, int64_t *launches) {
    if (kernel_id < 0 || kernel_id >= lutb::K_COUNT) {
        lutb::set_error("unknown kernel id %d", kernel_id);
        return LUTB_ERR_SHAPE;
    }
    std::lock_guard<std::mutex> lock(lutb::g_prof_mutex);
    lutb::resolve_pending_locked();
    if (total_ms) *total_ms = lutb::g_total_ms[kernel_id];
    if (timed_launches) *timed_launches = lutb::g_timed[kernel_id];
    if (launches) *launches = lutb::g_launches[kernel_id].load();
    return LUTB_OK;
}

extern "C" int lutb_version(void) { return 100; }
extern "C" const char *lutb_last_error(void) { return lutb::g_error; }
