"""Test infrastructure: runs the Python layer mirror (spiky_b200.lut_layer / lut_transformer) on CPU tensors by
serving the data manager's runtime calls from the CPU oracle.  It lets the host-side logic - shapes, positional
embedding handling, gradient policies, autograd wiring, the transformer's block structure - be checked against the
reference's fixtures without a GPU.  Never used by the product: the real data manager refuses to run on CPU."""
import numpy as np
import torch

from oracle import lut_oracle as orc


def _np(t):
    return None if t is None else t.detach().numpy()


def _acc(dst, value):
    """Accumulates a numpy result into the caller's flat torch buffer (the runtime accumulates into its outputs)."""
    if dst is not None and value is not None:
        dst.view(-1).add_(torch.from_numpy(np.ascontiguousarray(value)).view(-1).to(dst.dtype))


def _put(dst, value):
    if dst is not None and value is not None:
        dst.view(-1).copy_(torch.from_numpy(np.ascontiguousarray(value)).view(-1))


class OracleDataManager:
    """Same runtime methods as spiky_b200.lut_data_manager._LUTDataManager, on CPU tensors, through the oracle."""

    def __init__(self, real):
        self._real = real
        self._seen = False

    def __getattr__(self, name):
        return getattr(self._real, name)

    def to_device(self, device):
        return None

    # ---- helpers
    def _kw(self):
        r = self._real
        return dict(int_mode=r._INT_MODE, int_rescaler=r._int_rescaler)

    def _sp(self):
        index = self._real._sparse
        return dict(index.numpy(), group_size=index.group_size)

    # ---- non-sequence layers
    def forward_step(self, r_weights, batch_size, r_input, r_detector_anchors, w_output, w_lookup_indices, cmp_eps=0.0,
                     r_stream_handles=None, w_min_anchor_deltas=None, w_min_anchor_delta_indices=None):
        r = self._real
        train = w_min_anchor_deltas is not None
        x = _np(r_input).reshape(batch_size, r._n_inputs)
        if r._fully_connected:
            res = orc.nonseq_fc_forward(_np(r_weights), x, _np(r_detector_anchors), r._n_detectors, r._n_anchors,
                                        r._n_outputs, cmp_eps=cmp_eps, train=train, backward_group_size=r._bwd_group,
                                        **self._kw())
        else:
            res = orc.nonseq_sparse_forward(_np(r_weights), x, _np(r_detector_anchors), self._sp(), r._n_anchors,
                                            r._n_outputs, cmp_eps=cmp_eps, train=train, **self._kw())
        y, idx, md, mk = res
        _acc(w_output, y)
        _put(w_lookup_indices, idx)
        _put(w_min_anchor_deltas, md)
        _put(w_min_anchor_delta_indices, mk)
        self._seen = True

    def backward_backprop(self, r_weights, batch_size, r_output_gradients, r_detector_anchors, r_lookup_indices,
                          r_min_anchor_deltas, r_min_anchor_delta_indices, w_input_gradients, external_lr,
                          w_weights_gradients=None, r_stream_handles=None, dw_variant=0, workspace=None):
        if not self._seen:
            raise ValueError("no active context")
        r = self._real
        B = batch_size
        dY = _np(r_output_gradients).reshape(B, r._n_outputs)
        idx = _np(r_lookup_indices).reshape(B, r._n_detectors)
        md = _np(r_min_anchor_deltas).reshape(B, r._n_detectors)
        mk = _np(r_min_anchor_delta_indices).reshape(B, r._n_detectors)
        W = r_weights.numpy() if external_lr >= 0 else _np(r_weights)  # in-place SGD writes through
        skip_table = external_lr == -2.0  # input gradient only (spiky_b200._native.SKIP_TABLE_GRADIENT)
        assert not (skip_table and w_weights_gradients is not None)
        common = dict(lr_meta=r._lr_meta(), external_lr=-1.0 if skip_table else external_lr, **self._kw())
        if r._fully_connected:
            dX, dW = orc.nonseq_fc_backward(W, dY, _np(r_detector_anchors), idx, md, mk, r._n_inputs, r._n_anchors,
                                            forward_group_size=r._fwd_group, **common)
        else:
            dX, dW = orc.nonseq_sparse_backward(W, dY, _np(r_detector_anchors), idx, md, mk, self._sp(), r._n_inputs,
                                                r._n_anchors, **common)
        _acc(w_input_gradients, dX)
        _acc(w_weights_gradients, dW)

    def table_gradient_rows(self, batch_size, r_output_gradients, r_lookup_indices):
        """(row_ids, values) of the rows the batch touched, from the oracle's dense table gradient."""
        r = self._real
        B, Nt, T, O = batch_size, r._n_detectors, 1 << r._n_anchors, r._n_outputs
        dY = _np(r_output_gradients).reshape(B, O)
        idx = _np(r_lookup_indices).reshape(B, Nt).astype(np.int32)
        anchors = np.zeros((Nt, r._n_anchors, 2), np.int32)  # only the (discarded) input gradient reads them
        W = np.zeros(Nt * T * O, np.float32)
        _, dW = orc.nonseq_fc_backward(W, dY, anchors, idx, np.ones(idx.shape, np.float32), np.zeros_like(idx),
                                       r._n_inputs, r._n_anchors, forward_group_size=r._fwd_group, lr_meta=r._lr_meta())
        rows = np.unique(np.arange(Nt, dtype=np.int64)[None, :] * T + idx)
        return torch.from_numpy(rows), torch.from_numpy(dW.reshape(Nt * T, O)[rows].copy())

    def table_gradient(self, batch_size, r_output_gradients, r_lookup_indices, w_target, scale, chunk_begin=0,
                       chunk_end=None):
        """w_target[row(t, idx) + p] += scale * lr_meta * dY[b, target(p)] for the detectors of the chunk range."""
        r = self._real
        index = r._sparse
        chunk_end = index.n_chunks if chunk_end is None else chunk_end
        if not 0 <= chunk_begin <= chunk_end <= index.n_chunks:
            raise ValueError("chunk range outside the index")
        B = batch_size
        dY = _np(r_output_gradients).reshape(B, r._n_outputs)
        idx = _np(r_lookup_indices).reshape(B, r._n_detectors)
        if idx.dtype == np.int16:
            idx = idx.view(np.uint16)
        idx = idx.astype(np.int32)
        ones = np.ones(idx.shape, np.float32)
        anchors = np.zeros((r._n_detectors, r._n_anchors, 2), np.int32)  # only the (discarded) input gradient reads them
        _, dW = orc.nonseq_sparse_backward(_np(w_target), dY, anchors, idx, ones,
                                           np.zeros_like(idx), self._sp(), r._n_inputs, r._n_anchors,
                                           lr_meta=r._lr_meta(), **self._kw())
        bounds = index.chunk_weight_bounds()
        lo, hi = int(bounds[chunk_begin]), int(bounds[chunk_end])
        w_target.view(-1)[lo:hi] += float(scale) * torch.from_numpy(dW[lo:hi])

    # ---- product-mode sequence layers
    def _pe3(self, pe, S):
        r = self._real
        return None if pe is None else _np(pe).reshape(S - 1, r._n_detectors, r._pos_dim)

    def forward_step_product(self, r_weights, batch_size, sequence_length, r_input_1, r_input_2, r_detector_anchors,
                             w_output, n_inputs_1, n_inputs_2, sliced_mode, cmp_eps=0.0, r_positional_embeddings=None,
                             r_stream_handles=None, variant=0, keep_histogram=False):
        r = self._real
        assert r_input_1.data_ptr() == r_input_2.data_ptr() and n_inputs_1 == n_inputs_2
        x = _np(r_input_1).reshape(batch_size, sequence_length, n_inputs_1)
        y = orc.product_forward(_np(r_weights), x, self._pe3(r_positional_embeddings, sequence_length),
                                _np(r_detector_anchors), r._n_detectors, r._n_anchors, r._n_outputs, r._pos_dim,
                                sliced=sliced_mode, cmp_eps=cmp_eps, **self._kw())
        _acc(w_output, y)
        self._seen = True

    def backward_backprop_product(self, r_weights, batch_size, sequence_length, r_input_1, r_input_2,
                                  r_detector_anchors, r_output_gradients, w_input_gradients_1, w_input_gradients_2,
                                  external_lr, n_inputs_1, n_inputs_2, sliced_mode, cmp_eps=0.0,
                                  w_weights_gradients=None, r_positional_embeddings=None,
                                  w_positional_embeddings_gradients=None, r_stream_handles=None, variant=0):
        if not self._seen:
            raise ValueError("no active context")
        r = self._real
        assert w_input_gradients_1.data_ptr() == w_input_gradients_2.data_ptr()
        x = _np(r_input_1).reshape(batch_size, sequence_length, n_inputs_1)
        dY = _np(r_output_gradients).reshape(batch_size, sequence_length, r._n_outputs)
        W = r_weights.numpy() if external_lr >= 0 else _np(r_weights)
        dX, dW, dPE = orc.product_backward(W, x, self._pe3(r_positional_embeddings, sequence_length),
                                           _np(r_detector_anchors), dY, r._n_detectors, r._n_anchors, r._pos_dim,
                                           sliced=sliced_mode, cmp_eps=cmp_eps, lr_meta=r._lr_meta(),
                                           external_lr=external_lr, **self._kw())
        _acc(w_input_gradients_1, dX)
        _acc(w_weights_gradients, dW)
        _acc(w_positional_embeddings_gradients, dPE)

    # ---- concatenation-mode sequence layers
    def forward_step_concat(self, r_weights, batch_size, r_input, r_detector_anchors, w_output, w_lookup_indices,
                            cmp_eps=0.0, r_positional_embeddings=None, w_positional_lookup_indices=None,
                            w_min_anchor_deltas=None, w_min_anchor_delta_indices=None, w_positional_min_deltas=None,
                            w_positional_min_delta_indices=None, r_stream_handles=None):
        r = self._real
        S = r._seq_len
        train = w_min_anchor_deltas is not None
        x = _np(r_input).reshape(batch_size, S, r._n_inputs)
        pe = self._pe3(r_positional_embeddings, S)
        if r._fully_connected:
            y, st = orc.concat_forward(_np(r_weights), x, pe, _np(r_detector_anchors), r._n_detectors, r._n_anchors,
                                       r._n_outputs, r._pos_dim, cmp_eps=cmp_eps, train=train, **self._kw())
        else:
            y, st = orc.concat_sparse_forward(_np(r_weights), x, pe, _np(r_detector_anchors), self._sp(), r._n_anchors,
                                              r._n_outputs, r._pos_dim, cmp_eps=cmp_eps, train=train, **self._kw())
        _acc(w_output, y)
        _put(w_lookup_indices, st["idx"])
        _put(w_min_anchor_deltas, st["min_delta"])
        _put(w_min_anchor_delta_indices, st["min_k"])
        _put(w_positional_lookup_indices, st["pidx"])
        _put(w_positional_min_deltas, st["pmin"])
        _put(w_positional_min_delta_indices, st["pmin_k"])
        self._seen = True

    def backward_backprop_concat(self, r_weights, batch_size, r_output_gradients, r_detector_anchors, r_lookup_indices,
                                 r_min_anchor_deltas, r_min_anchor_delta_indices, w_input_gradients, external_lr,
                                 r_positional_lookup_indices=None, r_positional_min_deltas=None,
                                 r_positional_min_delta_indices=None, w_positional_embeddings_gradients=None,
                                 w_weights_gradients=None, r_stream_handles=None):
        if not self._seen:
            raise ValueError("no active context")
        r = self._real
        S, Nt = r._seq_len, r._n_detectors
        dY = _np(r_output_gradients).reshape(batch_size, S, r._n_outputs)
        as_i32 = lambda t: None if t is None else np.ascontiguousarray(_np(t), dtype=np.int32)
        as_f32 = lambda t: None if t is None else np.ascontiguousarray(_np(t), dtype=np.float32)
        state = dict(idx=as_i32(r_lookup_indices).reshape(batch_size * S, Nt),
                     min_delta=as_f32(r_min_anchor_deltas).reshape(batch_size * S, Nt),
                     min_k=as_i32(r_min_anchor_delta_indices).reshape(batch_size * S, Nt),
                     pidx=as_i32(r_positional_lookup_indices), pmin=as_f32(r_positional_min_deltas),
                     pmin_k=as_i32(r_positional_min_delta_indices))
        W = r_weights.numpy() if external_lr >= 0 else _np(r_weights)
        common = dict(lr_meta=r._lr_meta(), external_lr=external_lr, **self._kw())
        if r._fully_connected:
            dX, dW, dPE = orc.concat_backward(W, dY, _np(r_detector_anchors), state, r._n_inputs, r._n_anchors,
                                              r._pos_dim, forward_group_size=r._fwd_group, **common)
        else:
            dX, dW, dPE = orc.concat_sparse_backward(W, dY, _np(r_detector_anchors), state, self._sp(), r._n_inputs,
                                                     r._n_anchors, r._pos_dim, **common)
        _acc(w_input_gradients, dX)
        _acc(w_weights_gradients, dW)
        _acc(w_positional_embeddings_gradients, dPE)


    # ---- stages of the concatenation-mode layer (query-range variants)
    def check_detectors(self, rows, r_input, r_detector_anchors, w_lookup_indices, cmp_eps=0.0,
                        w_min_anchor_deltas=None, w_min_anchor_delta_indices=None):
        r = self._real
        train = w_min_anchor_deltas is not None
        res = orc.check_detectors(_np(r_input).reshape(rows, r._n_inputs), _np(r_detector_anchors), r._n_detectors,
                                  r._n_anchors, cmp_eps, train)
        idx, md, mk = res if train else (res, None, None)
        _put(w_lookup_indices, idx)
        _put(w_min_anchor_deltas, md)
        _put(w_min_anchor_delta_indices, mk)

    def check_positional(self, r_positional_embeddings, w_positional_lookup_indices, cmp_eps=0.0,
                         w_positional_min_deltas=None, w_positional_min_delta_indices=None):
        r = self._real
        train = w_positional_min_deltas is not None
        res = orc.check_positional(_np(r_positional_embeddings), r._seq_len, r._n_detectors, r._pos_dim, cmp_eps, train)
        pidx, pm, pk = res if train else (res, None, None)
        _put(w_positional_lookup_indices, pidx)
        _put(w_positional_min_deltas, pm)
        _put(w_positional_min_delta_indices, pk)

    def concat_pairs_forward(self, r_weights, batch_size, r_lookup_indices, r_positional_lookup_indices, w_output,
                             j_begin, j_end):
        # every query's output depends on its own pairs only: the range is a slice of the full result
        r = self._real
        S = r._seq_len
        y = orc.concat_pairs_forward(_np(r_weights), _np(r_lookup_indices).reshape(batch_size * S, r._n_detectors),
                                     _np(r_positional_lookup_indices), batch_size, S, r._n_detectors, r._n_anchors,
                                     r._n_outputs, r._pos_dim, **self._kw())
        y[:, :j_begin] = 0.0
        y[:, j_end:] = 0.0
        _acc(w_output, y)
        self._seen = True

    def concat_pairs_backward(self, r_weights, batch_size, r_output_gradients, r_detector_anchors, r_lookup_indices,
                              r_min_anchor_deltas, r_min_anchor_delta_indices, w_input_gradients, external_lr,
                              r_positional_lookup_indices, r_positional_min_deltas, r_positional_min_delta_indices,
                              w_positional_embeddings_gradients, w_weights_gradients, j_begin, j_end):
        # a pair contributes through dY of its query only: zero gradients outside the range leave exactly the
        # range's pairs (contributions with |dY| <= 1e-17 are dropped by the arithmetic itself)
        r = self._real
        S = r._seq_len
        masked = r_output_gradients.detach().clone().view(batch_size, S, r._n_outputs)
        masked[:, :j_begin] = 0.0
        masked[:, j_end:] = 0.0
        self.backward_backprop_concat(r_weights, batch_size, masked.view(-1), r_detector_anchors, r_lookup_indices,
                                      r_min_anchor_deltas, r_min_anchor_delta_indices, w_input_gradients, external_lr,
                                      r_positional_lookup_indices, r_positional_min_deltas,
                                      r_positional_min_delta_indices, w_positional_embeddings_gradients,
                                      w_weights_gradients)


def use_oracle_backend(module):
    """Replaces the data manager of every LUT layer inside ``module`` (a layer or a model, on CPU) by the
    oracle-backed one; returns the module."""
    from spiky_b200.lut_layer import LUTLayerBasic

    for layer in module.modules():
        if isinstance(layer, LUTLayerBasic) and not isinstance(layer._lut_dm, OracleDataManager):
            layer._lut_dm = OracleDataManager(layer._lut_dm)
    return module
