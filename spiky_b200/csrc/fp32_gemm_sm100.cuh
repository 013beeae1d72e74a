// fp32 GEMMs on the tensor cores (tcgen05) for the histogram path of the product-mode layer; see fp32_gemm_sm100.cu.
#pragma once

#include "lutb_common.cuh"

namespace lutb {

enum TcGemmKind {
    TC_A_ROWS_B_ROWS_OF_N,   // A [M x K] row-major, B stored as [N x K] row-major:  C = A . B^T
    TC_A_ROWS_B_ROWS_OF_K,   // A [M x K] row-major, B stored as [K x N] row-major:  C = A . B
    TC_A_COLS_B_ROWS_OF_K,   // A stored as [K x M] row-major, B as [K x N] row-major: C = A^T . B
};

// false when the library was built without a CUTLASS header tree (tc_gemm then fails with LUTB_ERR_MODE)
bool tc_gemm_available();
// C [M x N] row-major = alpha * op(A) . op(B) + beta * C; all pointers 16-byte aligned, lda / ldb / ldc multiples of 4.
// Split-TF32 route: hi / lo copies of the operands in the workspace, concatenated so that one TF32 GEMM forms all the
// cross products wherever the layouts allow (else two or three GEMMs accumulate into C).
// a_exact: A holds integers below 2048 (row counts), which TF32 represents exactly: A is used as it is, two GEMMs.
size_t tc_gemm_workspace(TcGemmKind kind, int M, int N, int K, bool a_exact);
int tc_gemm(TcGemmKind kind, int M, int N, int K, const float *A, int64_t lda, const float *B, int64_t ldb, float *C,
            int64_t ldc, float alpha, float beta, bool a_exact, void *workspace, size_t workspace_bytes, cudaStream_t stream);
// Single-GEMM route: the mainloop splits the fp32 operands into BF16 terms on the fly.
size_t tc_gemm_fast_workspace(int M, int N, int K);
int tc_gemm_fast(TcGemmKind kind, int M, int N, int K, const float *A, int64_t lda, const float *B, int64_t ldb, float *C,
                 int64_t ldc, float alpha, float beta, void *workspace, size_t workspace_bytes, cudaStream_t stream);

}  // namespace lutb
