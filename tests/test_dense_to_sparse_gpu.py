"""Dense -> sparse compaction kernel (the Sparse gradient policy's converter) against numpy."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def make(n, density, seed, dtype=np.float32):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(n).astype(np.float32)
    x[rng.random(n) >= density] = 0.0
    if dtype == np.int32:
        return (x * 1000).astype(np.int32)
    return x


@pytest.mark.parametrize("n,density", [(4, 1.0), (8, 0.0), (2048, 0.5), (2052, 0.3), (1 << 20, 0.01), (3 * 2048 * 256 + 12, 0.7)])
def test_compaction_matches_numpy_and_is_sorted(n, density):
    from spiky_b200.torch_utils import DenseToSparseConverter

    conv = DenseToSparseConverter()
    x = make(n, density, 5 + n % 97)
    if n >= 8 and density > 0:
        x[3] = -0.0          # bit pattern 0x80000000 is a non-zero word, as in the reference
        x[n - 1] = 1.5       # last word of a ragged tail
    t = torch.from_numpy(x.copy()).cuda()
    want = np.flatnonzero(x.view(np.uint32))
    assert conv.count_nonzero(t) == want.size
    idx, val = conv.dense_to_sparse_32(t)
    if want.size == 0:
        assert idx is None and val is None
        return
    assert np.array_equal(idx.cpu().numpy(), want)                       # sorted, exact
    assert np.array_equal(val.cpu().numpy().view(np.uint32), x.view(np.uint32)[want])
    assert np.array_equal(t.cpu().numpy().view(np.uint32), x.view(np.uint32))  # source untouched


def test_erase_preallocated_buffers_and_int32():
    from spiky_b200.torch_utils import DenseToSparseConverter

    conv = DenseToSparseConverter()
    x = make(40000, 0.2, 11, np.int32)
    t = torch.from_numpy(x.copy()).cuda()
    want = np.flatnonzero(x)
    bufs = (torch.empty(want.size + 100, dtype=torch.int64, device="cuda"),
            torch.empty(want.size + 100, dtype=torch.int32, device="cuda"))
    idx, val = conv.dense_to_sparse_32(t, erase_input=True, densify_buffers=bufs)
    assert np.array_equal(idx.cpu().numpy(), want) and np.array_equal(val.cpu().numpy(), x[want])
    assert not t.any()                                                    # erased
    small = (torch.empty(3, dtype=torch.int64, device="cuda"), torch.empty(3, dtype=torch.int32, device="cuda"))
    with pytest.raises(ValueError, match="non-zero words"):
        conv.dense_to_sparse_32(torch.from_numpy(x.copy()).cuda(), densify_buffers=small)
    with pytest.raises(ValueError, match="divisable by 4"):
        conv.dense_to_sparse_32(torch.zeros(6, device="cuda"))
    with pytest.raises(ValueError, match="32-bit"):
        conv.dense_to_sparse_32(torch.zeros(8, device="cuda", dtype=torch.float64))
