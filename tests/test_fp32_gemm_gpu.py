"""The tensor-core fp32 GEMM of the library (lutb_fp32_gemm: fp32 operands split into BF16 terms, tcgen05.mma with fp32
accumulators in tensor memory) against an fp64 product, through the C ABI, for the three operand layouts the histogram
path of the product-mode layer uses; the bar is the layers' own 1e-5."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

KINDS = {0: "A rows, B rows of n", 1: "A rows, B rows of k", 2: "A columns, B rows of k"}
FAST = 16   # LUTB_GEMM_FAST_FP32: the single-GEMM route (operands split into BF16 terms inside the mainloop)


def gemm(kind, A, B, C, alpha, beta, fast=False):
    from spiky_b200 import _native
    L = _native.lib()
    flags = FAST if fast else 0
    if kind == 0:
        m, k = A.shape
        n = B.shape[0]
    elif kind == 1:
        m, k = A.shape
        n = B.shape[1]
    else:
        k, m = A.shape
        n = B.shape[1]
    need = L.lutb_fp32_gemm_workspace(m, n, k)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=A.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    _native.check(L.lutb_fp32_gemm(kind | flags, m, n, k, ptr(A), A.stride(0), ptr(B), B.stride(0), ptr(C), C.stride(0), alpha, beta,
                                   ptr(ws), ws.numel(), stream))


@pytest.mark.parametrize("fast", [False, True], ids=["split_tf32", "fast_fp32"])
@pytest.mark.parametrize("kind", sorted(KINDS))
@pytest.mark.parametrize("shape", [(256, 256, 512), (300, 200, 520), (128, 1024, 64), (1000, 8, 36)])
def test_fp32_gemm_matches_fp64_product(kind, shape, fast):
    from spiky_b200 import _native
    if not _native.lib().lutb_fp32_gemm_available():
        pytest.skip("library built without the CUTLASS headers")
    m, n, k = shape
    g = torch.Generator().manual_seed(m + n + k + kind)
    A = torch.randn((m, k) if kind != 2 else (k, m), generator=g).cuda()
    B = torch.randn((n, k) if kind == 0 else (k, n), generator=g).cuda()
    if kind == 2:
        A = torch.randint(0, 1024, A.shape, generator=g).float().cuda()   # row counts: exact small integers
    C0 = torch.randn(m, n, generator=g).cuda()
    C = C0.clone()
    gemm(kind, A, B, C, 0.5, 1.0, fast)
    a64 = A.double() if kind != 2 else A.double().t()
    b64 = B.double().t() if kind == 0 else B.double()
    ref = 0.5 * (a64 @ b64) + C0.double()
    err = (C.double() - ref).abs().max().item()
    assert err <= 1e-5 * ref.abs().max().item(), f"{KINDS[kind]} {shape}: max err {err:.3e} of {ref.abs().max().item():.3e}"
    # beta = 0 overwrites
    C.fill_(float("nan"))
    gemm(kind, A, B, C, 1.0, 0.0, fast)
    ref = a64 @ b64
    assert (C.double() - ref).abs().max().item() <= 1e-5 * ref.abs().max().item()


def test_fp32_gemm_rejects_misaligned_leading_dimensions():
    from spiky_b200 import _native
    if not _native.lib().lutb_fp32_gemm_available():
        pytest.skip("library built without the CUTLASS headers")
    A = torch.zeros(8, 6, device="cuda")
    B = torch.zeros(8, 6, device="cuda")
    C = torch.zeros(8, 8, device="cuda")
    with pytest.raises(ValueError, match="multiples of 4"):
        gemm(0, A, B, C, 1.0, 0.0)
