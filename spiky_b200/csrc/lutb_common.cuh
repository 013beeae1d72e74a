// Shared host/device helpers of the LUT runtime kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/spiky_b200.h"

namespace lutb {

// Fixed-point constants of the int32 accumulator mode (reference: spiky_cuda/misc/misc.h:90-103).
constexpr double kDenom = 1048575.0;                  // DENOMINATOR32 = 0xFFFFF
constexpr double kDenomRecip = 9.536752259018191e-07;  // DENOMINATOR32_RECIPROC
constexpr double kEps = 0.00000000000000001;           // EPS: contributions with |v| <= EPS are dropped
// largest float not above EPS: for a float g, fabsf(g) > kEpsF is the same predicate as fabs((double)g) > kEps
constexpr float kEpsF = 1e-17f;
constexpr int32_t kNoAnchor = -1;                      // 0xFFFFFFFF marks an unused anchor pair

constexpr int kMaxSmemPerBlock = 227 * 1024;  // opt-in dynamic shared memory limit on sm_100

void set_error(const char *fmt, ...);

struct DeviceInfo {
    int sm_count;
    int device;
};
// SM count of the current device (cached per device).
DeviceInfo device_info();

#define LUTB_REQUIRE(cond, code, ...)      \
    do {                                    \
        if (!(cond)) {                      \
            lutb::set_error(__VA_ARGS__);   \
            return (code);                  \
        }                                   \
    } while (0)

#define LUTB_CUDA(expr)                                                                  \
    do {                                                                                 \
        cudaError_t _e = (expr);                                                         \
        if (_e != cudaSuccess) {                                                         \
            lutb::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return (int)_e;                                                              \
        }                                                                                \
    } while (0)

#define LUTB_LAUNCH_CHECK()                                                                       \
    do {                                                                                          \
        cudaError_t _e = cudaGetLastError();                                                      \
        if (_e != cudaSuccess) {                                                                  \
            lutb::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), __FILE__, __LINE__); \
            return (int)_e;                                                                       \
        }                                                                                         \
    } while (0)

int validate_cfg(const lutb_layer_cfg *cfg);

// While an instance lives on a thread, KernelScope only counts launches on that thread and never creates
// CUDA events (event creation allocates); used by entry points that promise not to allocate.
class NoEventsGuard {
public:
    NoEventsGuard();
    ~NoEventsGuard();
};

// Kernel families, as reported by the opt-in profiler (lutb_profiler_*) and the launch counter.
enum KernelId {
    K_CHECK_DETECTORS = 0,
    K_FC_GATHER_FORWARD,
    K_FC_INPUT_GRAD,
    K_FC_WEIGHT_GRAD,
    K_FIXED_TO_FLOAT,
    K_SPARSE_FORWARD,
    K_SPARSE_INPUT_GRAD,
    K_SPARSE_WEIGHT_GRAD,
    K_SPARSE_BACKWARD_FUSED,
    K_PRODUCT_FORWARD,
    K_PRODUCT_BACKWARD,
    K_PRODUCT_WEIGHT_UPDATE,
    K_CHECK_POSITIONAL,
    K_CONCAT_FORWARD,
    K_CONCAT_BACKWARD,
    K_CONCAT_WEIGHT_UPDATE,
    K_INT8_GATHER,
    K_PRODUCT_HIST,
    K_PRODUCT_HIST_FORWARD,
    K_PRODUCT_ROW_DOTS,
    K_PRODUCT_ROUTE,
    K_PRODUCT_HIST_WEIGHT_GRAD,
    K_DENSE_TO_SPARSE,
    K_FP32_GEMM,
    K_PEER_SGD_UPDATE,
    K_PEER_BARRIER,
    K_PEER_BROADCAST,
    K_COUNT
};

// RAII marker around one kernel launch: always bumps the launch counter; when the profiler is enabled
// it also brackets the launch with CUDA events on the launching stream (no synchronisation here, the
// events are resolved when the profiler is read).
class KernelScope {
public:
    KernelScope(KernelId id, cudaStream_t stream);
    ~KernelScope();
    KernelScope(const KernelScope &) = delete;
    KernelScope &operator=(const KernelScope &) = delete;

private:
    cudaStream_t stream_;
    cudaEvent_t stop_;
};

// Dead-band comparison "delta > 0" (reference: ROUNDED_COMPARISON_GREATER, misc.h:16).
__device__ __forceinline__ bool greater_than_zero(float delta, float cmp_eps) {
    if (cmp_eps == 0.0f) return delta > 0.0f;
    return fabsf(delta) < cmp_eps ? false : delta > 0.0f;
}

// Surrogate derivative up(m) = sign(m) * 0.5 / (1 + |m|)^2 with up(0) negative
// (reference: lut_runtime_kernels_logic.proto:1339-1345), evaluated in double like the reference;
// (+-0.5 * r) * r rounds exactly as the reference's r * (+-0.5 * r) because the scaling by 0.5 is exact.
__device__ __forceinline__ double surrogate_up(float m) {
    double du = (double)m;
    double r = 1.0 / (1.0 + fabs(du));
    return (du > 0 ? 0.5 : -0.5) * r * r;
}

__device__ __forceinline__ int32_t to_fixed(double v, double scale) {
    return (int32_t)(v * kDenom * scale);  // cvt.rzi: truncation toward zero like the C cast
}

// Bounded waits of the peer-memory barrier that ran out on the current device (peer_update.cu).
int peer_wait_errors(int *count_out);

// In-place conversion of int32 fixed-point accumulators to fp32
// (reference: convert_integers_to_floats_logic, proto:200-213).
int launch_fixed_to_float(float *buf, int64_t n, double rescaler, cudaStream_t stream);

}  // namespace lutb
