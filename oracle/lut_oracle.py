"""numpy front-end of the CPU oracle (``lut_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke test and the benchmark's CPU-baseline leg may import this module;
the product package never does.  Every function takes and returns numpy arrays and mirrors one
runtime call of the reference's ``LUTDataManagerF`` / ``LUTDataManagerI``
(spiky_cuda/lut/lut.cu:629-1180).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liblut_oracle.so")
_lib = None

_f = ctypes.c_float
_d = ctypes.c_double
_i = ctypes.c_int
_l = ctypes.c_int64
_p = ctypes.c_void_p


def build(force=False):
    """Compile the C oracle with the host gcc (a few seconds)."""
    src = os.path.join(_HERE, "lut_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
        subprocess.check_call(["make", "-C", _HERE, "-B", f"CC={cc}"], stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
    return _lib


def _ptr(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def set_threads(n):
    """Number of OpenMP threads used by the batch-parallel baseline loops (1 = reference-like)."""
    lib().orc_set_threads(_i(int(n)))


def check_detectors(x, anchors, n_detectors, n_anchors, cmp_eps=0.0, train=True):
    """x [rows, I] -> idx int32 [rows, Nt] (+ min_delta f32, min_k int32 when train)."""
    x = _f32(x)
    rows, n_in = x.shape
    anchors = _i32(anchors).reshape(-1)
    idx = np.zeros((rows, n_detectors), np.int32)
    md = np.zeros((rows, n_detectors), np.float32) if train else None
    mk = np.zeros((rows, n_detectors), np.int32) if train else None
    lib().orc_check_detectors(_ptr(x), _l(rows), _i(n_in), _ptr(anchors), _i(n_detectors), _i(n_anchors),
                              _f(cmp_eps), _ptr(idx), _ptr(md), _ptr(mk))
    return (idx, md, mk) if train else idx


def check_positional(pe, seq_len, n_detectors, pos_dim, cmp_eps=0.0, train=True):
    pe = _f32(pe).reshape(-1)
    n = (seq_len - 1) * n_detectors
    pidx = np.zeros(n, np.int32)
    pm = np.zeros(n, np.float32) if train else None
    pk = np.zeros(n, np.int32) if train else None
    lib().orc_check_positional(_ptr(pe), _i(seq_len), _i(n_detectors), _i(pos_dim), _f(cmp_eps), _ptr(pidx),
                               _ptr(pm), _ptr(pk))
    return (pidx, pm, pk) if train else pidx


def nonseq_fc_forward(W, x, anchors, n_detectors, n_anchors, n_outputs, cmp_eps=0.0, train=True,
                      backward_group_size=32, int_mode=False, int_rescaler=0.001):
    """One ``forward_step`` of a fully connected non-sequence layer.

    Returns (y [B,O], idx [B,Nt], min_delta, min_k); the last two are None when train is False.
    """
    x = _f32(x)
    B = x.shape[0]
    T = 1 << n_anchors
    W = _f32(W).reshape(-1)
    assert W.size == n_detectors * T * n_outputs
    res = check_detectors(x, anchors, n_detectors, n_anchors, cmp_eps, train)
    idx, md, mk = res if train else (res, None, None)
    y = np.zeros((B, n_outputs), np.float32)
    lib().orc_nonseq_fc_forward(_ptr(W), _ptr(idx), _ptr(y), _l(B), _i(n_outputs), _i(n_detectors), _i(T),
                                _i(backward_group_size), _i(int(int_mode)), _d(int_rescaler))
    return y, idx, md, mk


def int_to_float(acc, int_rescaler):
    """int32 fixed-point accumulators -> fp32 (convert_integers_to_floats_logic); returns a new array."""
    out = np.ascontiguousarray(acc, np.int32).copy().view(np.float32)
    lib().orc_int_to_float(_ptr(out), _l(out.size), _d(int_rescaler))
    return out


def infer_int8(q, scales, x, anchors, n_detectors, n_anchors, n_outputs, cmp_eps=0.0, backward_group_size=32,
               int_rescaler=0.001, exact=True):
    """int8-table inference: (int32 accumulators [B,O], idx [B,Nt]).  exact=False de-quantises to the fp32 numbers
    f32(scale * q) (identical to the fixed-point forward on that fp32 table), exact=True to the exact reals."""
    x = _f32(x)
    B = x.shape[0]
    T = 1 << n_anchors
    q = np.ascontiguousarray(q, np.int8).reshape(-1)
    scales = _f32(scales).reshape(-1)
    assert q.size == n_detectors * T * n_outputs and scales.size == n_detectors
    idx = check_detectors(x, anchors, n_detectors, n_anchors, cmp_eps, False)
    acc = np.zeros((B, n_outputs), np.int32)
    lib().orc_infer_int8(_ptr(q), _ptr(scales), _ptr(idx), _ptr(acc), _l(B), _i(n_outputs), _i(n_detectors), _i(T),
                         _i(backward_group_size), _d(int_rescaler), _i(int(exact)))
    return acc, idx


def nonseq_fc_backward(W, dY, anchors, idx, min_delta, min_k, n_inputs, n_anchors, lr_meta=1.0,
                       external_lr=-1.0, forward_group_size=32, int_mode=False, int_rescaler=0.001):
    """One ``backward_backprop`` of a fully connected non-sequence layer.

    Returns (dX [B,I], dW [Nt*T*O] or None).  With external_lr >= 0 the weights array ``W`` is
    updated in place (it must then be a writable contiguous float32 array) and dW is None.
    """
    dY = _f32(dY)
    B, O = dY.shape
    Nt = idx.shape[1]
    T = 1 << n_anchors
    if external_lr >= 0:
        assert W.dtype == np.float32 and W.flags["C_CONTIGUOUS"] and W.flags["WRITEABLE"]
        Wf = W.reshape(-1)
        dW = None
    else:
        Wf = _f32(W).reshape(-1)
        dW = np.zeros(Wf.size, np.float32)
    dX = np.zeros((B, n_inputs), np.float32)
    anchors = _i32(anchors).reshape(-1)
    lib().orc_nonseq_fc_backward(_ptr(Wf), _ptr(dY), _ptr(anchors), _ptr(_i32(idx)), _ptr(_f32(min_delta)),
                                 _ptr(_i32(min_k)), _ptr(dX), _ptr(dW), _l(B), _i(n_inputs), _i(O), _i(Nt),
                                 _i(n_anchors), _i(T), _i(forward_group_size),
                                 _d(float(np.float32(lr_meta))), _d(float(np.float32(external_lr))),
                                 _i(int(int_mode)), _d(int_rescaler))
    return dX, dW


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def nonseq_sparse_forward(W, x, anchors, sp, n_anchors, n_outputs, cmp_eps=0.0, train=True, int_mode=False,
                          int_rescaler=0.001):
    """One ``forward_step`` of a sparse non-sequence layer.  ``sp`` holds the per-detector connectivity:
    dict(det_wbase, det_stride, det_count, det_sstart, syn_target, group_size)."""
    x = _f32(x)
    B = x.shape[0]
    Nt = len(sp["det_count"])
    W = _f32(W).reshape(-1)
    res = check_detectors(x, anchors, Nt, n_anchors, cmp_eps, train)
    idx, md, mk = res if train else (res, None, None)
    y = np.zeros((B, n_outputs), np.float32)
    lib().orc_nonseq_sparse_forward(_ptr(W), _ptr(idx), _ptr(y), _l(B), _i(n_outputs), _i(Nt),
                                    _ptr(_i64(sp["det_wbase"])), _ptr(_i32(sp["det_stride"])),
                                    _ptr(_i32(sp["det_count"])), _ptr(_i32(sp["det_sstart"])),
                                    _ptr(_i32(sp["syn_target"])), _i(int(sp["group_size"])), _i(int(int_mode)),
                                    _d(int_rescaler))
    return y, idx, md, mk


def nonseq_sparse_backward(W, dY, anchors, idx, min_delta, min_k, sp, n_inputs, n_anchors, lr_meta=1.0,
                           external_lr=-1.0, int_mode=False, int_rescaler=0.001):
    """One ``backward_backprop`` of a sparse non-sequence layer; returns (dX, dW or None)."""
    dY = _f32(dY)
    B, O = dY.shape
    Nt = idx.shape[1]
    if external_lr >= 0:
        assert W.dtype == np.float32 and W.flags["C_CONTIGUOUS"] and W.flags["WRITEABLE"]
        Wf, dW = W.reshape(-1), None
    else:
        Wf = _f32(W).reshape(-1)
        dW = np.zeros(Wf.size, np.float32)
    dX = np.zeros((B, n_inputs), np.float32)
    anchors = _i32(anchors).reshape(-1)
    lib().orc_nonseq_sparse_backward(_ptr(Wf), _ptr(dY), _ptr(anchors), _ptr(_i32(idx)), _ptr(_f32(min_delta)),
                                     _ptr(_i32(min_k)), _ptr(dX), _ptr(dW), _l(B), _i(n_inputs), _i(O), _i(Nt),
                                     _i(n_anchors), _ptr(_i64(sp["det_wbase"])), _ptr(_i32(sp["det_stride"])),
                                     _ptr(_i32(sp["det_count"])), _ptr(_i32(sp["det_sstart"])),
                                     _ptr(_i32(sp["syn_target"])), _i(int(sp["group_size"])), _l(Wf.size),
                                     _d(float(np.float32(lr_meta))), _d(float(np.float32(external_lr))),
                                     _i(int(int_mode)), _d(int_rescaler))
    return dX, dW


def product_forward(W, x, pe, anchors, n_detectors, n_anchors, n_outputs, pos_dim, sliced=False, cmp_eps=0.0,
                    int_mode=False, int_rescaler=0.001):
    """One ``forward_step_product``: x [B,S,E] is used for both pair members (as the layer does),
    pe [(S-1), Nt, Npe] (already repeated over detectors for unified embeddings) or None."""
    x = _f32(x)
    B, S, E = x.shape
    W = _f32(W).reshape(-1)
    y = np.zeros((B, S, n_outputs), np.float32)
    pe_f = None if pe is None else _f32(pe).reshape(-1)
    lib().orc_product_forward(_ptr(W), _ptr(x), _ptr(x), _ptr(pe_f), _ptr(_i32(anchors).reshape(-1)), _ptr(y),
                              _l(B), _i(S), _i(E), _i(E), _i(pos_dim), _i(n_outputs), _i(n_detectors),
                              _i(n_anchors), _i(int(sliced)), _f(cmp_eps), _i(int(int_mode)), _d(int_rescaler))
    return y


def product_backward(W, x, pe, anchors, dY, n_detectors, n_anchors, pos_dim, sliced=False, cmp_eps=0.0,
                     lr_meta=1.0, external_lr=-1.0, int_mode=False, int_rescaler=0.001):
    """One ``backward_backprop_product``; returns (dX [B,S,E], dW or None, dPE or None)."""
    x = _f32(x)
    dY = _f32(dY)
    B, S, E = x.shape
    O = dY.shape[-1]
    if external_lr >= 0:
        assert W.dtype == np.float32 and W.flags["C_CONTIGUOUS"] and W.flags["WRITEABLE"]
        Wf, dW = W.reshape(-1), None
    else:
        Wf = _f32(W).reshape(-1)
        dW = np.zeros(Wf.size, np.float32)
    dX = np.zeros((B, S, E), np.float32)
    pe_f = None if pe is None else _f32(pe).reshape(-1)
    dPE = None if pe is None else np.zeros(pe_f.size, np.float32)
    lib().orc_product_backward(_ptr(Wf), _ptr(x), _ptr(x), _ptr(pe_f), _ptr(_i32(anchors).reshape(-1)), _ptr(dY),
                               _ptr(dX), _ptr(dX), _ptr(dPE), _ptr(dW), _l(B), _i(S), _i(E), _i(E), _i(pos_dim),
                               _i(O), _i(n_detectors), _i(n_anchors), _i(int(sliced)), _f(cmp_eps),
                               _d(float(np.float32(lr_meta))), _d(float(np.float32(external_lr))),
                               _i(int(int_mode)), _d(int_rescaler))
    return dX, dW, dPE


def concat_forward(W, x, pe, anchors, n_detectors, n_anchors, n_outputs, pos_dim, cmp_eps=0.0, train=True,
                   int_mode=False, int_rescaler=0.001):
    """One ``forward_step_concat``: x [B,S,I], pe [(S-1), Nt, Npe] or None.
    Returns (y [B,S,O], state) with state = dict(idx, min_delta, min_k, pidx, pmin, pmin_k)."""
    x = _f32(x)
    B, S, I = x.shape
    res = check_detectors(x.reshape(B * S, I), anchors, n_detectors, n_anchors, cmp_eps, train)
    idx, md, mk = res if train else (res, None, None)
    pidx = pm = pk = None
    if pos_dim > 0:
        pres = check_positional(pe, S, n_detectors, pos_dim, cmp_eps, train)
        pidx, pm, pk = pres if train else (pres, None, None)
    y = np.zeros((B, S, n_outputs), np.float32)
    W = _f32(W).reshape(-1)
    lib().orc_concat_forward(_ptr(W), _ptr(idx), _ptr(pidx), _ptr(y), _l(B), _i(S), _i(n_outputs), _i(n_detectors),
                             _i(n_anchors), _i(pos_dim), _i(int(int_mode)), _d(int_rescaler))
    return y, dict(idx=idx, min_delta=md, min_k=mk, pidx=pidx, pmin=pm, pmin_k=pk)


def concat_pairs_forward(W, idx, pidx, batch, seq_len, n_detectors, n_anchors, n_outputs, pos_dim, int_mode=False,
                         int_rescaler=0.001):
    """The pair stage of ``forward_step_concat`` alone, from the table indices of all tokens
    (idx int32 [B*S, Nt], pidx int32 [(S-1)*Nt] or None); returns y [B,S,O]."""
    y = np.zeros((batch, seq_len, n_outputs), np.float32)
    W = _f32(W).reshape(-1)
    idx = _i32(idx)
    pidx = None if pidx is None else _i32(pidx)
    lib().orc_concat_forward(_ptr(W), _ptr(idx), _ptr(pidx), _ptr(y), _l(batch), _i(seq_len), _i(n_outputs),
                             _i(n_detectors), _i(n_anchors), _i(pos_dim), _i(int(int_mode)), _d(int_rescaler))
    return y


def concat_backward(W, dY, anchors, state, n_inputs, n_anchors, pos_dim, lr_meta=1.0, external_lr=-1.0,
                    forward_group_size=32, int_mode=False, int_rescaler=0.001):
    """One ``backward_backprop_concat``; returns (dX [B,S,I], dW or None, dPE [(S-1)*Nt*Npe] or None)."""
    dY = _f32(dY)
    B, S, O = dY.shape
    Nt = state["idx"].shape[1]
    if external_lr >= 0:
        assert W.dtype == np.float32 and W.flags["C_CONTIGUOUS"] and W.flags["WRITEABLE"]
        Wf, dW = W.reshape(-1), None
    else:
        Wf = _f32(W).reshape(-1)
        dW = np.zeros(Wf.size, np.float32)
    dX = np.zeros((B, S, n_inputs), np.float32)
    dPE = np.zeros((S - 1) * Nt * pos_dim, np.float32) if pos_dim > 0 else None
    lib().orc_concat_backward(_ptr(Wf), _ptr(dY), _ptr(_i32(anchors).reshape(-1)), _ptr(state["idx"]),
                              _ptr(state["min_delta"]), _ptr(state["min_k"]), _ptr(state["pidx"]),
                              _ptr(state["pmin"]), _ptr(state["pmin_k"]), _ptr(dX), _ptr(dPE), _ptr(dW), _l(B),
                              _i(S), _i(n_inputs), _i(O), _i(Nt), _i(n_anchors), _i(pos_dim),
                              _i(forward_group_size), _d(float(np.float32(lr_meta))),
                              _d(float(np.float32(external_lr))), _i(int(int_mode)), _d(int_rescaler))
    return dX, dW, dPE


def _sp_args(sp):
    return (_ptr(_i64(sp["det_wbase"])), _ptr(_i32(sp["det_stride"])), _ptr(_i32(sp["det_count"])),
            _ptr(_i32(sp["det_sstart"])), _ptr(_i32(sp["syn_target"])), _i(int(sp["group_size"])))


def concat_sparse_forward(W, x, pe, anchors, sp, n_anchors, n_outputs, pos_dim, cmp_eps=0.0, train=True,
                          int_mode=False, int_rescaler=0.001):
    """``forward_step_concat`` of a layer with sparse lookup -> output connectivity (``sp`` as in
    nonseq_sparse_forward, with 2^(2*Nc+Npe) rows per detector).  Returns (y [B,S,O], state)."""
    x = _f32(x)
    B, S, I = x.shape
    Nt = len(sp["det_count"])
    res = check_detectors(x.reshape(B * S, I), anchors, Nt, n_anchors, cmp_eps, train)
    idx, md, mk = res if train else (res, None, None)
    pidx = pm = pk = None
    if pos_dim > 0:
        pres = check_positional(pe, S, Nt, pos_dim, cmp_eps, train)
        pidx, pm, pk = pres if train else (pres, None, None)
    y = np.zeros((B, S, n_outputs), np.float32)
    W = _f32(W).reshape(-1)
    lib().orc_concat_sparse_forward(_ptr(W), _ptr(idx), _ptr(pidx), _ptr(y), _l(B), _i(S), _i(n_outputs), _i(Nt),
                                    _i(n_anchors), _i(pos_dim), *_sp_args(sp), _i(int(int_mode)), _d(int_rescaler))
    return y, dict(idx=idx, min_delta=md, min_k=mk, pidx=pidx, pmin=pm, pmin_k=pk)


def concat_sparse_backward(W, dY, anchors, state, sp, n_inputs, n_anchors, pos_dim, lr_meta=1.0, external_lr=-1.0,
                           int_mode=False, int_rescaler=0.001):
    """``backward_backprop_concat`` of a sparse sequence layer; returns (dX [B,S,I], dW or None, dPE or None)."""
    dY = _f32(dY)
    B, S, O = dY.shape
    Nt = len(sp["det_count"])
    if external_lr >= 0:
        assert W.dtype == np.float32 and W.flags["C_CONTIGUOUS"] and W.flags["WRITEABLE"]
        Wf, dW = W.reshape(-1), None
    else:
        Wf = _f32(W).reshape(-1)
        dW = np.zeros(Wf.size, np.float32)
    dX = np.zeros((B, S, n_inputs), np.float32)
    dPE = np.zeros((S - 1) * Nt * pos_dim, np.float32) if pos_dim > 0 else None
    lib().orc_concat_sparse_backward(_ptr(Wf), _ptr(dY), _ptr(_i32(anchors).reshape(-1)), _ptr(state["idx"]),
                                     _ptr(state["min_delta"]), _ptr(state["min_k"]), _ptr(state["pidx"]),
                                     _ptr(state["pmin"]), _ptr(state["pmin_k"]), _ptr(dX), _ptr(dPE), _ptr(dW), _l(B),
                                     _i(S), _i(n_inputs), _i(O), _i(Nt), _i(n_anchors), _i(pos_dim), *_sp_args(sp),
                                     _l(Wf.size), _d(float(np.float32(lr_meta))), _d(float(np.float32(external_lr))),
                                     _i(int(int_mode)), _d(int_rescaler))
    return dX, dW, dPE



def peer_sgd_update(weights, grads, scale):
    """Data-parallel SGD step of one table set (no reference counterpart: the reference trains on one device; this
    states what ``lutb_peer_sgd_update`` computes so that the kernel can be checked bit for bit): the ranks' fp32
    gradients are added in rank order, ``w - scale * sum`` with the product and the difference rounded separately."""
    acc = _f32(grads[0]).copy()
    for g in grads[1:]:
        acc += _f32(g)
    return _f32(weights) - np.float32(scale) * acc
