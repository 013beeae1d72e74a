// fp32 GEMMs on the sm_100a tensor cores for the contractions of the product-mode histogram path.
//
// The contractions (product_hist.cuh) multiply exact small integers (row counts) or fp32 tables / gradients and must
// keep fp32 accuracy (parity bar 1e-5), so plain TF32 or BF16 inputs are not an option.  Two routes, both CUTLASS 3
// collectives instantiated for sm_100a (operands arrive in shared memory by TMA - cluster 1x1x1: plain copies of this
// GPU's own memory -, tcgen05.mma accumulates in fp32 in tensor memory, the epilogue reads the accumulators back with
// tcgen05.ld and applies alpha / beta):
//
//   split TF32 (default)  every fp32 operand x is written once as hi = x rounded to TF32 and lo = x - hi (exact)
//                         rounded to TF32, and the product is formed as hi.hi + hi.lo + lo.hi; concatenated copies
//                         make that ONE TF32 GEMM wherever the layouts allow.  An operand that holds integers below
//                         2048 (row counts) is exact in TF32 and needs no split.  The dropped lo.lo term and the
//                         rounding of lo are each below 2^-22 relative.
//   fast fp32             one GEMM whose mainloop splits the operands into three BF16 terms on the fly (CUTLASS'
//                         "FastF32" schedule); simpler, no scratch, but bound by the conversion work: 80-90 TFLOP/s on
//                         the contraction shapes against 2-3 times that for the split TF32 route.
//
// Results agree with an fp32 FMA contraction to about 1e-6 relative; the summation order differs.
// All matrices are fp32 with 16-byte aligned base pointers and leading dimensions that are multiples of 4.
#include "fp32_gemm_sm100.cuh"

#ifdef LUTB_NO_CUTLASS
// built without a CUTLASS header tree: the callers keep their fp32 FMA contractions
namespace lutb {
bool tc_gemm_available() { return false; }
size_t tc_gemm_workspace(TcGemmKind, int, int, int, bool) { return 0; }
size_t tc_gemm_fast_workspace(int, int, int) { return 0; }
int tc_gemm(TcGemmKind, int, int, int, const float *, int64_t, const float *, int64_t, float *, int64_t, float, float, bool,
            void *, size_t, cudaStream_t) {
    set_error("the library was built without the tensor-core contractions (no CUTLASS headers at build time)");
    return LUTB_ERR_MODE;
}
int tc_gemm_fast(TcGemmKind, int, int, int, const float *, int64_t, const float *, int64_t, float *, int64_t, float, float,
                 void *, size_t, cudaStream_t) {
    set_error("the library was built without the tensor-core contractions (no CUTLASS headers at build time)");
    return LUTB_ERR_MODE;
}
}  // namespace lutb
#else

#include "cutlass/cutlass.h"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/util/packed_stride.hpp"

namespace lutb {

using namespace cute;

template <class LayoutA, class LayoutB>
struct FastF32Gemm {
    using Element = float;
    using LayoutC = cutlass::layout::RowMajor;
    static constexpr int kAlign = 4;   // 16 bytes
    using MmaTile = Shape<_128, _128, _16>;
    using Cluster = Shape<_1, _1, _1>;
    using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, MmaTile, Cluster,
        cutlass::epilogue::collective::EpilogueTileAuto, float, float, Element, LayoutC, kAlign, Element, LayoutC, kAlign,
        cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;
    using Mainloop = typename cutlass::gemm::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, Element, LayoutA, kAlign, Element, LayoutB, kAlign, float, MmaTile,
        Cluster, cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
        cutlass::gemm::KernelTmaWarpSpecialized1SmFastFP32Sm100>::CollectiveOp;
    using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Mainloop, Epilogue>;
    using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;
    using StrideA = typename Kernel::StrideA;
    using StrideB = typename Kernel::StrideB;
    using StrideC = typename Kernel::StrideC;
    using StrideD = typename Kernel::StrideD;
};

template <class LayoutA, class LayoutB>
struct Tf32Gemm {
    using Element = cutlass::tfloat32_t;   // fp32 storage; the MMA reads sign, exponent and the top 10 mantissa bits
    using LayoutC = cutlass::layout::RowMajor;
    static constexpr int kAlign = 4;
    using MmaTile = Shape<_128, _128, _32>;
    using Cluster = Shape<_1, _1, _1>;
    using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, MmaTile, Cluster,
        cutlass::epilogue::collective::EpilogueTileAuto, float, float, float, LayoutC, kAlign, float, LayoutC, kAlign,
        cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;
    using Mainloop = typename cutlass::gemm::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, Element, LayoutA, kAlign, Element, LayoutB, kAlign, float, MmaTile,
        Cluster, cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
        cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;
    using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Mainloop, Epilogue>;
    using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;
    using StrideA = typename Kernel::StrideA;
    using StrideB = typename Kernel::StrideB;
    using StrideC = typename Kernel::StrideC;
    using StrideD = typename Kernel::StrideD;
};

template <class Cfg>
static size_t workspace_of(int M, int N, int K) {
    typename Cfg::Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm, {M, N, K, 1}};
    return Cfg::Gemm::get_workspace_size(args);
}

// `batches` independent GEMMs of the same shape in one launch; operand b of batch l starts batch_b * l elements
// after the first (and so on); one batch by default.
struct Batches {
    int count = 1;
    int64_t a = 0, b = 0, c = 0;
};

template <class Cfg>
static int run(int M, int N, int K, const float *A, int64_t lda, const float *B, int64_t ldb, float *C, int64_t ldc,
               float alpha, float beta, void *workspace, size_t workspace_bytes, cudaStream_t stream,
               Batches batches = Batches{}) {
    typename Cfg::StrideA sa;
    typename Cfg::StrideB sb;
    typename Cfg::StrideC sc;
    // the dynamic (non unit) mode of every stride is the leading dimension
    if constexpr (cute::is_same_v<decltype(get<1>(sa)), cute::Int<1>>) sa = make_stride(lda, Int<1>{}, batches.a);
    else sa = make_stride(Int<1>{}, lda, batches.a);
    if constexpr (cute::is_same_v<decltype(get<1>(sb)), cute::Int<1>>) sb = make_stride(ldb, Int<1>{}, batches.b);
    else sb = make_stride(Int<1>{}, ldb, batches.b);
    sc = make_stride(ldc, Int<1>{}, batches.c);
    using ElementAB = typename Cfg::Element;
    typename Cfg::Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm,
                                       {M, N, K, batches.count},
                                       {reinterpret_cast<const ElementAB *>(A), sa, reinterpret_cast<const ElementAB *>(B), sb},
                                       {{alpha, beta}, C, sc, C, sc}};
    typename Cfg::Gemm gemm;
    LUTB_REQUIRE(gemm.can_implement(args) == cutlass::Status::kSuccess, LUTB_ERR_SHAPE,
                 "tensor-core contraction: shapes or alignments not supported (M=%d N=%d K=%d)", M, N, K);
    const size_t need = Cfg::Gemm::get_workspace_size(args);
    LUTB_REQUIRE(need <= workspace_bytes, LUTB_ERR_WORKSPACE, "tensor-core contraction needs %zu bytes of workspace", need);
    cutlass::Status st = gemm.initialize(args, workspace, stream);
    LUTB_REQUIRE(st == cutlass::Status::kSuccess, LUTB_ERR_MODE, "tensor-core contraction: initialisation failed (%d)", (int)st);
    st = gemm.run(stream);
    LUTB_REQUIRE(st == cutlass::Status::kSuccess, LUTB_ERR_MODE, "tensor-core contraction: launch failed (%d)", (int)st);
    return LUTB_OK;
}

// operand layouts: TN = A [M x K] row-major, B stored as [N x K] row-major; NN = A [M x K], B [K x N] row-major;
// TT = A stored as [K x M] row-major, B [K x N] row-major
using FastTN = FastF32Gemm<cutlass::layout::RowMajor, cutlass::layout::ColumnMajor>;
using FastNN = FastF32Gemm<cutlass::layout::RowMajor, cutlass::layout::RowMajor>;
using FastTT = FastF32Gemm<cutlass::layout::ColumnMajor, cutlass::layout::RowMajor>;
using Tf32TN = Tf32Gemm<cutlass::layout::RowMajor, cutlass::layout::ColumnMajor>;
using Tf32NN = Tf32Gemm<cutlass::layout::RowMajor, cutlass::layout::RowMajor>;
using Tf32TT = Tf32Gemm<cutlass::layout::ColumnMajor, cutlass::layout::RowMajor>;

bool tc_gemm_available() { return true; }

// Nearest value with a 10-bit mantissa (what a TF32 operand keeps; the MMA itself would truncate).
__device__ __forceinline__ float round_tf32(float x) {
    return __uint_as_float((__float_as_uint(x) + 0x00001000u) & 0xFFFFE000u);
}

// hi = x rounded to TF32 (|x - hi| <= 2^-11 |x|), lo = x - hi (exact in fp32) rounded to TF32 (error <= 2^-22 |x|).
// The two parts of a [rows x cols] matrix are written into a [rows x parts * cols] matrix, part p at columns
// [p * cols, (p + 1) * cols); `pattern` says which part goes where (bit p set: lo, clear: hi).  Concatenating along
// the contraction index turns hi.hi + hi.lo + lo.hi into ONE GEMM with three times the depth (A parts hi|hi|lo, B
// parts hi|lo|hi); concatenating B along its free index turns A.hi + A.lo into one GEMM with twice the width.
__global__ void split_tf32_kernel(const float *__restrict__ x, int64_t rows, int64_t cols, int64_t ld, float *__restrict__ out,
                                  int parts, unsigned pattern) {
    const int64_t n4 = rows * (cols / 4);
    const int64_t ldo = (int64_t)parts * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / (cols / 4), c = (i - r * (cols / 4)) * 4;
        const float4 v = *reinterpret_cast<const float4 *>(x + r * ld + c);
        float4 h, l;
        h.x = round_tf32(v.x); l.x = round_tf32(v.x - h.x);
        h.y = round_tf32(v.y); l.y = round_tf32(v.y - h.y);
        h.z = round_tf32(v.z); l.z = round_tf32(v.z - h.z);
        h.w = round_tf32(v.w); l.w = round_tf32(v.w - h.w);
        for (int p = 0; p < parts; p++)
            *reinterpret_cast<float4 *>(out + r * ldo + p * cols + c) = ((pattern >> p) & 1u) ? l : h;
    }
}

static int split(const float *x, int64_t rows, int64_t cols, int64_t ld, float *out, int parts, unsigned pattern,
                 cudaStream_t stream) {
    const int64_t n4 = rows * (cols / 4);
    int64_t blocks = (n4 + 255) / 256;
    const int64_t cap = (int64_t)device_info().sm_count * 16;
    if (blocks > cap) blocks = cap;
    split_tf32_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, rows, cols, ld, out, parts, pattern);
    LUTB_LAUNCH_CHECK();
    return LUTB_OK;
}

// C = alpha * sum over the slices s of (P_s[:, 0:N] + P_s[:, N:2N]) + beta * C, P_s = P + s * M * 2N; the lo halves are
// summed first (the smaller terms), then the hi halves, in rounded fp32.
__global__ void combine_halves_kernel(const float *__restrict__ P, float *__restrict__ C, int64_t M, int64_t N, int64_t ldc,
                                      float alpha, float beta, int slices) {
    const int64_t n4 = M * (N / 4);
    const int64_t slice = M * 2 * N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / (N / 4), c = (i - r * (N / 4)) * 4;
        float4 lo = *reinterpret_cast<const float4 *>(P + r * 2 * N + N + c);
        for (int s_ = 1; s_ < slices; s_++) {
            const float4 t = *reinterpret_cast<const float4 *>(P + s_ * slice + r * 2 * N + N + c);
            lo.x += t.x; lo.y += t.y; lo.z += t.z; lo.w += t.w;
        }
        float4 hi = *reinterpret_cast<const float4 *>(P + r * 2 * N + c);
        for (int s_ = 1; s_ < slices; s_++) {
            const float4 t = *reinterpret_cast<const float4 *>(P + s_ * slice + r * 2 * N + c);
            hi.x += t.x; hi.y += t.y; hi.z += t.z; hi.w += t.w;
        }
        float4 *dst = reinterpret_cast<float4 *>(C + r * ldc + c);
        float4 v = make_float4(alpha * (lo.x + hi.x), alpha * (lo.y + hi.y), alpha * (lo.z + hi.z), alpha * (lo.w + hi.w));
        if (beta != 0.f) {
            const float4 o = *dst;
            v.x += beta * o.x; v.y += beta * o.y; v.z += beta * o.z; v.w += beta * o.w;
        }
        *dst = v;
    }
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

template <class T3>
static size_t gemm_ws3(int M, int N, int K) {
    return workspace_of<T3>(M, N, K);
}

// Plan of one call.  TN (both operands contraction-major): one GEMM of depth 3K on concatenated copies.  NN / TT with an
// exact A: one GEMM of width 2N on B = [hi | lo], halves added in the epilogue pass.  Anything else: the generic
// sequence of two or three GEMMs on separate hi / lo copies.
struct SplitPlan {
    int mode;            // 0: deep TN, 1: wide (exact A), 2: generic
    int slices, kc;      // mode 1: the contraction index is cut into `slices` pieces of kc (see mode1_slices)
    size_t gemm_ws, a_bytes, b_bytes, p_bytes;
};

// How the wide plan cuts its contraction index.  Inside a slice the tensor core accumulates, truncating its fp32
// accumulator after every step (a bias that grows with the length of the chain); the slices' results are added in
// rounded fp32.  A . B with A [M x K] row-major (few output tiles, deep contraction: the forward pass of the histogram
// path): the slices are the batches of ONE launch, each into its own partial result, which also gives the launch
// K / kc times as many blocks.  A^T . B: the slices run one after the other and accumulate through the epilogue.  kc is
// at least 8 N, which keeps the traffic of the partial results below half of the slice's operand traffic.
static void mode1_slices(TcGemmKind kind, int N, int K, int *slices, int *kc) {
    int want = ((8 * N + 255) / 256) * 256;
    const int floor_ = kind == TC_A_ROWS_B_ROWS_OF_K ? 2048 : 8192;
    if (want < floor_) want = floor_;
    *slices = 1;
    *kc = K;
    if (kind == TC_A_ROWS_B_ROWS_OF_K) {
        // equal slices (one batched launch): the largest count of pieces of at least `want` that divides K evenly
        for (int l = K / want; l > 1; l--)
            if (K % l == 0 && (K / l) % 4 == 0) {
                *slices = l;
                *kc = K / l;
                break;
            }
    } else if (K > want) {
        *kc = want;
        *slices = (K + want - 1) / want;
    }
}

static SplitPlan split_plan(TcGemmKind kind, int M, int N, int K, bool a_exact) {
    SplitPlan p{};
    if (kind == TC_A_ROWS_B_ROWS_OF_N && !a_exact) {
        p.mode = 0;
        p.gemm_ws = align256(workspace_of<Tf32TN>(M, N, 3 * K));
        p.a_bytes = align256((size_t)M * 3 * K * 4);
        p.b_bytes = align256((size_t)N * 3 * K * 4);
    } else if (kind != TC_A_ROWS_B_ROWS_OF_N && a_exact && N % 4 == 0) {
        p.mode = 1;
        mode1_slices(kind, N, K, &p.slices, &p.kc);
        p.gemm_ws = align256(kind == TC_A_ROWS_B_ROWS_OF_K ? workspace_of<Tf32NN>(M, 2 * N, K) : workspace_of<Tf32TT>(M, 2 * N, K));
        p.b_bytes = align256((size_t)K * 2 * N * 4);
        p.p_bytes = align256((size_t)M * 2 * N * 4 * (kind == TC_A_ROWS_B_ROWS_OF_K ? p.slices : 1));
    } else {
        p.mode = 2;
        size_t w = workspace_of<Tf32TN>(M, N, K);
        const size_t w2 = workspace_of<Tf32NN>(M, N, K), w3 = workspace_of<Tf32TT>(M, N, K);
        w = w > w2 ? w : w2;
        p.gemm_ws = align256(w > w3 ? w : w3);
        p.a_bytes = a_exact ? 0 : align256((size_t)M * K * 4 * 2);
        p.b_bytes = align256((size_t)N * K * 4 * 2);
    }
    return p;
}

size_t tc_gemm_workspace(TcGemmKind kind, int M, int N, int K, bool a_exact) {
    const SplitPlan p = split_plan(kind, M, N, K, a_exact);
    return p.gemm_ws + p.a_bytes + p.b_bytes + p.p_bytes + 512;
}

template <class Cfg>
static int run3(int M, int N, int K, const float *Ah, const float *Al, int64_t lda, const float *Bh, const float *Bl, int64_t ldb,
                float *C, int64_t ldc, float alpha, float beta, void *ws, size_t ws_bytes, cudaStream_t stream) {
    // small terms first, so that they are added to each other before they meet the large one
    int rc = run<Cfg>(M, N, K, Ah, lda, Bl, ldb, C, ldc, alpha, beta, ws, ws_bytes, stream);
    if (rc) return rc;
    if (Al != nullptr) {
        rc = run<Cfg>(M, N, K, Al, lda, Bh, ldb, C, ldc, alpha, 1.f, ws, ws_bytes, stream);
        if (rc) return rc;
    }
    return run<Cfg>(M, N, K, Ah, lda, Bh, ldb, C, ldc, alpha, 1.f, ws, ws_bytes, stream);
}

int tc_gemm(TcGemmKind kind, int M, int N, int K, const float *A, int64_t lda, const float *B, int64_t ldb, float *C,
            int64_t ldc, float alpha, float beta, bool a_exact, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    const size_t need = tc_gemm_workspace(kind, M, N, K, a_exact);
    LUTB_REQUIRE(workspace_bytes >= need, LUTB_ERR_WORKSPACE, "tensor-core contraction needs %zu bytes of workspace", need);
    // stored extents of the operands: A is [ar x ac], B is [br x bc] (row-major, contiguous in the second)
    const int64_t ar = kind == TC_A_COLS_B_ROWS_OF_K ? K : M, ac = kind == TC_A_COLS_B_ROWS_OF_K ? M : K;
    const int64_t br = kind == TC_A_ROWS_B_ROWS_OF_N ? N : K, bc = kind == TC_A_ROWS_B_ROWS_OF_N ? K : N;
    LUTB_REQUIRE(ac % 4 == 0 && bc % 4 == 0, LUTB_ERR_ALIGN, "tensor-core contraction: row lengths must be multiples of 4");
    const SplitPlan plan = split_plan(kind, M, N, K, a_exact);
    unsigned char *p = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t)255);
    void *gw = p;
    p += plan.gemm_ws;
    float *Bs = reinterpret_cast<float *>(p);
    p += plan.b_bytes;
    float *As = reinterpret_cast<float *>(p);
    p += plan.a_bytes;
    float *P = reinterpret_cast<float *>(p);
    int rc;
    if (plan.mode == 0) {
        // A' = [hi | lo | hi], B' = [lo | hi | hi] along the contraction index: one GEMM of depth 3K.  The mainloop
        // walks the contraction index upwards and the tensor core truncates its fp32 accumulator after every step, an
        // error proportional to the accumulator's size: the two small products go first, while it is small.
        rc = split(A, M, K, lda, As, 3, 0b010u, stream);
        if (rc) return rc;
        rc = split(B, N, K, ldb, Bs, 3, 0b001u, stream);
        if (rc) return rc;
        return run<Tf32TN>(M, N, 3 * K, As, 3 * (int64_t)K, Bs, 3 * (int64_t)K, C, ldc, alpha, beta, gw, plan.gemm_ws, stream);
    }
    if (plan.mode == 1) {
        // B' = [hi | lo] along the free index: one GEMM of width 2N into P, then C = alpha * (P_hi + P_lo) + beta * C
        rc = split(B, K, N, ldb, Bs, 2, 0b10u, stream);
        if (rc) return rc;
        int p_slices = 1;
        if (kind == TC_A_ROWS_B_ROWS_OF_K) {
            // the slices of the contraction index as the batches of one launch, each into its own partial result
            Batches bt;
            bt.count = p_slices = plan.slices;
            bt.a = plan.kc;
            bt.b = (int64_t)plan.kc * 2 * N;
            bt.c = (int64_t)M * 2 * N;
            rc = run<Tf32NN>(M, 2 * N, plan.kc, A, lda, Bs, 2 * (int64_t)N, P, 2 * (int64_t)N, 1.f, 0.f, gw, plan.gemm_ws, stream, bt);
            if (rc) return rc;
        } else {
            for (int k0 = 0; k0 < K; k0 += plan.kc) {
                const int kn = K - k0 < plan.kc ? K - k0 : plan.kc;
                rc = run<Tf32TT>(M, 2 * N, kn, A + (int64_t)k0 * lda, lda, Bs + (int64_t)k0 * 2 * N, 2 * (int64_t)N, P,
                                 2 * (int64_t)N, 1.f, k0 == 0 ? 0.f : 1.f, gw, plan.gemm_ws, stream);
                if (rc) return rc;
            }
        }
        const int64_t n4 = (int64_t)M * (N / 4);
        int64_t blocks = (n4 + 255) / 256;
        const int64_t cap = (int64_t)device_info().sm_count * 16;
        if (blocks > cap) blocks = cap;
        combine_halves_kernel<<<(unsigned)blocks, 256, 0, stream>>>(P, C, M, N, ldc, alpha, beta, p_slices);
        LUTB_LAUNCH_CHECK();
        return LUTB_OK;
    }
    // generic: separate hi / lo copies (one matrix with two parts each), two or three GEMMs
    rc = split(B, br, bc, ldb, Bs, 2, 0b10u, stream);
    if (rc) return rc;
    const float *Ah = A, *Al = nullptr;
    int64_t lda_s = lda;
    if (!a_exact) {
        rc = split(A, ar, ac, lda, As, 2, 0b10u, stream);
        if (rc) return rc;
        Ah = As; Al = As + ac; lda_s = 2 * ac;
    }
    const float *Bh = Bs, *Bl = Bs + bc;
    const int64_t ldb_s = 2 * bc;
    switch (kind) {
        case TC_A_ROWS_B_ROWS_OF_N: return run3<Tf32TN>(M, N, K, Ah, Al, lda_s, Bh, Bl, ldb_s, C, ldc, alpha, beta, gw, plan.gemm_ws, stream);
        case TC_A_ROWS_B_ROWS_OF_K: return run3<Tf32NN>(M, N, K, Ah, Al, lda_s, Bh, Bl, ldb_s, C, ldc, alpha, beta, gw, plan.gemm_ws, stream);
        default: return run3<Tf32TT>(M, N, K, Ah, Al, lda_s, Bh, Bl, ldb_s, C, ldc, alpha, beta, gw, plan.gemm_ws, stream);
    }
}

size_t tc_gemm_fast_workspace(int M, int N, int K) {
    size_t w = workspace_of<FastTN>(M, N, K);
    const size_t w2 = workspace_of<FastNN>(M, N, K), w3 = workspace_of<FastTT>(M, N, K);
    w = w > w2 ? w : w2;
    return (w > w3 ? w : w3) + 256;
}

int tc_gemm_fast(TcGemmKind kind, int M, int N, int K, const float *A, int64_t lda, const float *B, int64_t ldb, float *C,
                 int64_t ldc, float alpha, float beta, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    switch (kind) {
        case TC_A_ROWS_B_ROWS_OF_N: return run<FastTN>(M, N, K, A, lda, B, ldb, C, ldc, alpha, beta, workspace, workspace_bytes, stream);
        case TC_A_ROWS_B_ROWS_OF_K: return run<FastNN>(M, N, K, A, lda, B, ldb, C, ldc, alpha, beta, workspace, workspace_bytes, stream);
        default: return run<FastTT>(M, N, K, A, lda, B, ldb, C, ldc, alpha, beta, workspace, workspace_bytes, stream);
    }
}

}  // namespace lutb
#endif  // LUTB_NO_CUTLASS

// C-ABI face of the contraction (used by the tests and by callers that want the same fp32-accurate tensor-core GEMM
// the histogram path uses).
extern "C" int lutb_fp32_gemm_available(void) { return lutb::tc_gemm_available() ? 1 : 0; }

extern "C" size_t lutb_fp32_gemm_workspace(int32_t m, int32_t n, int32_t k) {
    if (!(m > 0 && n > 0 && k > 0)) return 0;
    size_t a = 0;
    for (int kind = 0; kind < 3; kind++) {
        const size_t w = lutb::tc_gemm_workspace(static_cast<lutb::TcGemmKind>(kind), m, n, k, false);
        a = w > a ? w : a;
    }
    const size_t b = lutb::tc_gemm_fast_workspace(m, n, k);
    return a > b ? a : b;
}

extern "C" int lutb_fp32_gemm(int kind, int32_t m, int32_t n, int32_t k, const float *a, int64_t lda, const float *b,
                              int64_t ldb, float *c, int64_t ldc, float alpha, float beta, void *workspace,
                              size_t workspace_bytes, void *stream) {
    using namespace lutb;
    const bool fast = (kind & LUTB_GEMM_FAST_FP32) != 0;
    kind &= ~LUTB_GEMM_FAST_FP32;
    LUTB_REQUIRE(kind >= LUTB_GEMM_A_ROWS_B_ROWS_OF_N && kind <= LUTB_GEMM_A_COLS_B_ROWS_OF_K, LUTB_ERR_MODE, "unknown GEMM kind %d", kind);
    LUTB_REQUIRE(m > 0 && n > 0 && k > 0, LUTB_ERR_SHAPE, "empty GEMM");
    LUTB_REQUIRE(a && b && c, LUTB_ERR_NULL, "a matrix pointer is NULL");
    LUTB_REQUIRE(((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) == 0,
                 LUTB_ERR_ALIGN, "matrices must be 16-byte aligned");
    LUTB_REQUIRE(((lda | ldb | ldc) & 3) == 0, LUTB_ERR_ALIGN, "leading dimensions must be multiples of 4");
    KernelScope scope(K_FP32_GEMM, static_cast<cudaStream_t>(stream));
    if (fast)
        return tc_gemm_fast(static_cast<TcGemmKind>(kind), m, n, k, a, lda, b, ldb, c, ldc, alpha, beta, workspace,
                            workspace_bytes, static_cast<cudaStream_t>(stream));
    return tc_gemm(static_cast<TcGemmKind>(kind), m, n, k, a, lda, b, ldb, c, ldc, alpha, beta, false, workspace, workspace_bytes,
                   static_cast<cudaStream_t>(stream));
}

