"""ctypes binding of libspiky_b200.so, the C-ABI CUDA library (include/spiky_b200.h).

The library is the only compute path: there is no CPU or PyTorch fallback.  Loading fails loudly
when the library has not been built (``python -m spiky_b200.build``).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libspiky_b200.so")

# dW kernel variants (include/spiky_b200.h)
DW_AUTO, DW_ATOMIC, DW_SORTED = 0, 1, 3
SKIP_TABLE_GRADIENT = -2.0  # external_lr value: input gradient only (lutb_nonseq_sparse_backward)
# product-mode kernel variants (include/spiky_b200.h)
PRODUCT_AUTO, PRODUCT_DIRECT, PRODUCT_HIST, PRODUCT_HIST_FMA = 0, 1, 2, 3
PRODUCT_KEEP_HIST, PRODUCT_REUSE_HIST = 0x100, 0x200   # flags or'ed into the variant
# de-quantisation rules of the int8 inference path (include/spiky_b200.h)
INT8_DEQUANT_F32, INT8_DEQUANT_EXACT = 0, 1
# kernel family of the sparse forward / input-gradient passes (include/spiky_b200.h)
SPARSE_AUTO, SPARSE_GATHER, SPARSE_STAGED = 0, 1, 2


class LayerCfg(ctypes.Structure):
    """Mirror of ``lutb_layer_cfg``."""

    _fields_ = [
        ("n_inputs", ctypes.c_int32),
        ("n_outputs", ctypes.c_int32),
        ("n_detectors", ctypes.c_int32),
        ("n_anchors", ctypes.c_int32),
        ("seq_len", ctypes.c_int32),
        ("pos_dim", ctypes.c_int32),
        ("forward_group", ctypes.c_int32),
        ("backward_group", ctypes.c_int32),
        ("int_mode", ctypes.c_int32),
        ("sliced_product", ctypes.c_int32),
        ("cmp_eps", ctypes.c_float),
        ("reserved0", ctypes.c_float),
        ("int_rescaler", ctypes.c_double),
        ("lr_meta", ctypes.c_double),
    ]


class SparseIndexC(ctypes.Structure):
    """Mirror of ``lutb_sparse_index`` (device pointers)."""

    _fields_ = [
        ("det_wbase", ctypes.c_void_p),
        ("det_stride", ctypes.c_void_p),
        ("det_count", ctypes.c_void_p),
        ("det_sstart", ctypes.c_void_p),
        ("syn_det", ctypes.c_void_p),
        ("syn_target", ctypes.c_void_p),
        ("chunk_info", ctypes.c_void_p),
        ("n_chunks", ctypes.c_int64),
        ("n_syn_per_sample", ctypes.c_int64),
        ("n_weights", ctypes.c_int64),
        ("group_size", ctypes.c_int32),
        ("max_count", ctypes.c_int32),
        ("max_table_slots", ctypes.c_int32),
        ("tables_aligned16", ctypes.c_int32),
    ]


_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int
_dbl = ctypes.c_double
_size = ctypes.c_size_t
_cfgp = ctypes.POINTER(LayerCfg)
_spp = ctypes.POINTER(SparseIndexC)

# name -> (restype, argtypes); every symbol include/spiky_b200.h declares is listed here
SIGNATURES = {
    "lutb_version": (_int, []),
    "lutb_last_error": (ctypes.c_char_p, []),
    "lutb_profiler_enable": (_int, [_int]),
    "lutb_profiler_reset": (_int, []),
    "lutb_profiler_kernel_count": (_int, []),
    "lutb_profiler_kernel_name": (ctypes.c_char_p, [_int]),
    "lutb_profiler_read": (_int, [_int, ctypes.POINTER(_dbl), ctypes.POINTER(_i64), ctypes.POINTER(_i64)]),
    "lutb_nonseq_fc_forward": (_int, [_cfgp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "lutb_nonseq_fc_backward_workspace": (_size, [_cfgp, _i64, _int]),
    "lutb_nonseq_fc_backward": (_int, [_cfgp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _dbl, _int, _vp, _size, _vp]),
    "lutb_concat_forward": (_int, [_cfgp, _i64] + [_vp] * 12),
    "lutb_concat_backward": (_int, [_cfgp, _i64] + [_vp] * 12 + [_dbl, _vp]),
    "lutb_check_detectors": (_int, [_cfgp, _i64, _vp, _vp, _vp, _vp, _vp, _vp]),
    "lutb_check_positional": (_int, [_cfgp, _vp, _vp, _vp, _vp, _vp]),
    "lutb_concat_pairs_forward": (_int, [_cfgp, _i64, _vp, _vp, _vp, _vp, ctypes.c_int32, ctypes.c_int32, _vp]),
    "lutb_concat_pairs_backward": (_int, [_cfgp, _i64] + [_vp] * 12 + [_dbl, ctypes.c_int32, ctypes.c_int32, _vp]),
    "lutb_concat_sparse_forward": (_int, [_cfgp, _spp, _i64] + [_vp] * 12),
    "lutb_concat_sparse_backward": (_int, [_cfgp, _spp, _i64] + [_vp] * 12 + [_dbl, _vp]),
    "lutb_product_workspace": (_size, [_cfgp, _i64, ctypes.c_int32, _int]),
    "lutb_product_forward": (_int, [_cfgp, _i64, ctypes.c_int32, _vp, _vp, _vp, ctypes.c_int32, ctypes.c_int32, _vp, _vp, _vp,
                                    _int, _vp, _size, _vp]),
    "lutb_product_backward": (_int, [_cfgp, _i64, ctypes.c_int32, _vp, _vp, _vp, ctypes.c_int32, ctypes.c_int32, _vp, _vp,
                                     _vp, _vp, _vp, _vp, _vp, _dbl, _int, _vp, _size, _vp]),
    "lutb_product_keeps_histogram": (_int, [_cfgp, _i64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, _int, _vp, _size]),
    "lutb_nonseq_fc_table_grad_rows_workspace": (_size, [_cfgp, _i64]),
    "lutb_nonseq_fc_table_grad_rows": (_int, [_cfgp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _size, _vp]),
    "lutb_nonseq_fc_backward_noalloc": (_int, [_cfgp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _dbl, _vp]),
    "lutb_infer_int8_accumulate": (_int, [_cfgp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _int, _vp]),
    "lutb_fixed_to_float": (_int, [_vp, _i64, _dbl, _vp]),
    "lutb_dense_to_sparse_workspace": (_size, [_i64]),
    "lutb_count_nonzero_32": (_int, [_vp, _i64, _vp, _vp, _size, _vp]),
    "lutb_dense_to_sparse_32": (_int, [_vp, _i64, _vp, _vp, _i64, _vp, _int, _vp, _size, _vp]),
    "lutb_sparse_kernel_select": (_int, [_int, _int]),
    "lutb_device_wait_errors": (_int, [ctypes.POINTER(_int)]),
    "lutb_fp32_gemm_available": (_int, []),
    "lutb_fp32_gemm_workspace": (_size, [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]),
    "lutb_fp32_gemm": (_int, [_int, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, _vp, _i64, _vp, _i64, _vp, _i64,
                              ctypes.c_float, ctypes.c_float, _vp, _size, _vp]),
    "lutb_peer_alloc": (_int, [_size, ctypes.POINTER(_vp), ctypes.c_char_p]),
    "lutb_peer_free": (_int, [_vp]),
    "lutb_peer_open": (_int, [ctypes.c_char_p, ctypes.POINTER(_vp)]),
    "lutb_peer_close": (_int, [_vp]),
    "lutb_peer_broadcast": (_int, [ctypes.c_int32, ctypes.POINTER(_vp), _i64, _vp, _i64, _vp]),
    "lutb_peer_copy": (_int, [_vp, _vp, _size, _vp]),
    "lutb_peer_barrier": (_int, [ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(_vp), ctypes.c_uint64, _vp]),
    "lutb_peer_sgd_update": (_int, [ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i64, _i64,
                                    ctypes.c_float, _vp]),
    "lutb_nonseq_sparse_forward": (_int, [_cfgp, _spp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "lutb_nonseq_sparse_backward": (_int, [_cfgp, _spp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _dbl, _vp]),
    "lutb_nonseq_sparse_table_grad": (_int, [_cfgp, _spp, _i64, _vp, _vp, _int, _vp, _dbl, _i64, _i64, _vp]),
}

_lib = None


def lib():
    """The loaded library; raises RuntimeError when it is missing (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA library with `python -m spiky_b200.build` "
                "(spiky_b200 has no CPU or PyTorch fallback)"
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class LutbError(RuntimeError):
    pass


def check(status):
    """Translate a C-ABI status into the exception type the reference raises for the same mistake:
    argument errors -> ValueError (py::value_error in spiky_cuda/lut/lut.cu), CUDA errors -> RuntimeError."""
    if status == 0:
        return
    msg = lib().lutb_last_error().decode(errors="replace")
    if status < 0:
        raise ValueError(msg)
    raise LutbError(f"CUDA error {status}: {msg}")


def profiler_enable(on=True):
    check(lib().lutb_profiler_enable(int(bool(on))))


def profiler_reset():
    check(lib().lutb_profiler_reset())


def profiler_read():
    """{kernel family: {"ms": resolved device time, "timed": launches timed, "launches": launches counted}}."""
    L = lib()
    out = {}
    for k in range(L.lutb_profiler_kernel_count()):
        ms, timed, launches = _dbl(0.0), _i64(0), _i64(0)
        check(L.lutb_profiler_read(k, ctypes.byref(ms), ctypes.byref(timed), ctypes.byref(launches)))
        out[L.lutb_profiler_kernel_name(k).decode()] = {"ms": ms.value, "timed": timed.value, "launches": launches.value}
    return out


def sparse_kernel_select(forward, input_grad=None):
    """Force the gather or the staged kernels for the forward and the input-gradient pass of sparse layers
    (SPARSE_AUTO restores the library's choice; one argument sets both passes)."""
    check(lib().lutb_sparse_kernel_select(int(forward), int(forward if input_grad is None else input_grad)))


PEER_HANDLE_BYTES = 64
MAX_PEER_RANKS = 16


def peer_alloc(nbytes):
    """Device memory other processes of the node can map: (device pointer, 64-byte handle)."""
    ptr = _vp()
    handle = ctypes.create_string_buffer(PEER_HANDLE_BYTES)
    check(lib().lutb_peer_alloc(int(nbytes), ctypes.byref(ptr), handle))
    return ptr.value, handle.raw


def peer_free(ptr):
    check(lib().lutb_peer_free(_vp(ptr)))


def peer_open(handle):
    """Maps a buffer another process of the node allocated with peer_alloc; returns the device pointer."""
    assert len(handle) == PEER_HANDLE_BYTES
    ptr = _vp()
    check(lib().lutb_peer_open(bytes(handle), ctypes.byref(ptr)))
    return ptr.value


def peer_close(ptr):
    check(lib().lutb_peer_close(_vp(ptr)))


def peer_broadcast(dst_ptrs, dst_offset, src_ptr, nbytes, stream):
    """Copies nbytes from src_ptr (local) to dst_ptrs[r] + dst_offset of every listed buffer (own or mapped)."""
    n = len(dst_ptrs)
    check(lib().lutb_peer_broadcast(n, (_vp * n)(*dst_ptrs), int(dst_offset), _vp(src_ptr), int(nbytes), _vp(stream)))


def peer_copy(dst_ptr, src_ptr, nbytes, stream):
    """One asynchronous device-to-device copy (a copy engine carries it when one side is another rank's buffer)."""
    check(lib().lutb_peer_copy(_vp(dst_ptr), _vp(src_ptr), int(nbytes), _vp(stream)))


def peer_barrier(rank, flag_ptrs, epoch, stream):
    """Stream-ordered barrier over the ranks through flags in peer memory (flag_ptrs[r]: rank r's flag array)."""
    n = len(flag_ptrs)
    check(lib().lutb_peer_barrier(n, int(rank), (_vp * n)(*flag_ptrs), int(epoch), _vp(stream)))


def peer_sgd_update(rank, grad_ptrs, weight_ptrs, begin, end, scale, stream):
    """weights[r][begin:end] = weights[rank][begin:end] - scale * sum_r grads[r][begin:end] on every rank r; the
    pointers are device addresses (own or mapped), one per rank."""
    n = len(grad_ptrs)
    assert len(weight_ptrs) == n
    arr = _vp * n
    check(lib().lutb_peer_sgd_update(n, int(rank), arr(*grad_ptrs), arr(*weight_ptrs), int(begin), int(end),
                                     float(scale), _vp(stream)))


def device_wait_errors():
    """Bounded device-side waits that ran out on the current device (0 in a healthy run); synchronises the device."""
    n = _int(0)
    check(lib().lutb_device_wait_errors(ctypes.byref(n)))
    return n.value
