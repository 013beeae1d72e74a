"""Dense -> sparse conversion of 32-bit tensors (reference: src/spiky/util/torch_utils.py:7-131, the Python face of
``DenseToSparseConverterNative``).  Same call shape; the lists come back sorted by index and deterministic."""
import ctypes

import torch

from . import _native


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


class DenseToSparseConverter:
    """Reusable converter: keeps its scratch between calls.

    >>> conv = DenseToSparseConverter()
    >>> idx, val = conv.dense_to_sparse_32(torch.tensor([1., 0., 2., 0.], device="cuda"))
    >>> idx.tolist(), val.tolist()
    ([0, 2], [1.0, 2.0])
    """

    def __init__(self, use_new_kernel=True):
        self._counter = None
        self._workspace = None

    def _scratch(self, source):
        need = _native.lib().lutb_dense_to_sparse_workspace(source.numel())
        if self._workspace is None or self._workspace.device != source.device or self._workspace.numel() < need:
            self._workspace = torch.empty(need, dtype=torch.uint8, device=source.device)
        if self._counter is None or self._counter.device != source.device:
            self._counter = torch.zeros(1, dtype=torch.int64, device=source.device)
        return self._workspace, self._counter

    @staticmethod
    def _check(source):
        if source.element_size() != 4:
            raise ValueError(f"source tensor must be 32-bit (element_size == 4), got {source.element_size()}")
        if source.dim() != 1:
            raise ValueError("source tensor must be 1D")
        if not source.is_contiguous():
            raise ValueError("source tensor must be contiguous")
        if (source.numel() % 4) != 0:
            raise ValueError("source tensor size must be divisable by 4")
        if source.device.type != "cuda":
            raise RuntimeError("spiky_b200 has no CPU path: the source must be a CUDA tensor")

    def count_nonzero(self, source, stream=None):
        self._check(source)
        ws, counter = self._scratch(source)
        with torch.cuda.device(source.device):
            s = (stream or torch.cuda.current_stream(source.device)).cuda_stream
            _native.check(_native.lib().lutb_count_nonzero_32(_ptr(source), source.numel(), _ptr(counter), _ptr(ws),
                                                              ws.numel(), ctypes.c_void_p(s)))
        return int(counter.item())

    def dense_to_sparse_32(self, source, erase_input=False, densify_buffers=None, stream=None, decouple=True):
        """(indices int64, values) of the non-zero words of ``source`` or (None, None); ``densify_buffers`` are
        preallocated (indices, values) to fill instead of allocating exactly-sized ones (which costs a host read of the
        count first); ``decouple`` returns exactly-sized copies instead of views into them."""
        self._check(source)
        ws, counter = self._scratch(source)
        if densify_buffers is not None:
            indices, values = densify_buffers
            if values.dim() != 1 or indices.dim() != 1:
                raise ValueError("densify_buffers tensors must be 1D")
            if values.dtype != source.dtype:
                raise ValueError("densify_buffers values tensor must match source dtype")
            if indices.dtype != torch.int64:
                raise ValueError("densify_buffers indices tensor must be int64")
            if values.device != source.device or indices.device != source.device:
                raise ValueError("densify_buffers tensors must be on the same device as source")
            if not values.is_contiguous() or not indices.is_contiguous():
                raise ValueError("densify_buffers tensors must be contiguous")
            if values.numel() != indices.numel():
                raise ValueError("densify_buffers tensors must have the same length")
        else:
            assert decouple
            nnz = self.count_nonzero(source, stream)
            if nnz == 0:
                return None, None
            indices = torch.empty(nnz, dtype=torch.int64, device=source.device)
            values = torch.empty(nnz, dtype=source.dtype, device=source.device)
        with torch.cuda.device(source.device):
            s = (stream or torch.cuda.current_stream(source.device)).cuda_stream
            _native.check(_native.lib().lutb_dense_to_sparse_32(
                _ptr(source), source.numel(), _ptr(indices), _ptr(values), indices.numel(), _ptr(counter),
                int(bool(erase_input)), _ptr(ws), ws.numel(), ctypes.c_void_p(s)))
        if densify_buffers is None:
            return indices, values
        if not decouple:
            return indices, values
        n = int(counter.item())
        if n > indices.numel():
            raise ValueError(f"densify_buffers hold {indices.numel()} entries, the source has {n} non-zero words")
        if n == 0:
            return None, None
        return indices[:n].clone(), values[:n].clone()

    def get_profiling_stats(self):
        prof = _native.profiler_read().get("dense_to_sparse", {"ms": 0.0, "launches": 0})
        return f"torch_utils::dense_to_sparse_32: {prof['launches']} launches, {prof['ms']:.3f} ms"
