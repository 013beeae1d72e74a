"""Host-side mirror of the reference's native data managers ``LUTDataManagerF`` / ``LUTDataManagerI``
(pybind11 classes of spiky_cuda/lut/lut.cu:12-1656), backed by the C-ABI CUDA library.

Method names, argument order and error behaviour follow the reference so that layer code written
against it runs unchanged: argument mistakes raise ``ValueError`` (the reference's
``py::value_error``), tensor dtype / layout / device mistakes raise ``RuntimeError``
(``checkTensor``, spiky_cuda/misc/misc.cpp:217-277).  Differences, all deliberate:

* kernels are enqueued on torch's CURRENT CUDA stream and the call returns without synchronising;
  ``r_stream_handles`` is accepted and ignored (the reference spreads work over three caller
  streams and the caller synchronises them);
* there is no CPU execution path: ``to_device(-1)`` is accepted during set-up, runtime calls on a
  CPU-resident manager raise ``RuntimeError``;
* fully connected layers need no native structure at all; sparse connectivity is attached as a
  compact per-detector index (``set_sparse_index``) instead of the reference's byte arena.
"""
import ctypes

import torch

from . import _native
from ._native import LayerCfg

_EPS = 0.00000000000000001
_DENOM32 = 0xFFFFF
_MAX_GROUP = 1024  # forward_group_size upper bound of the reference's launch configuration


def _check_tensor(t, name, real, device_index, int_bytes=4):
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name} must be a tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"tensor {name} must be contiguous")
    if t.dim() != 1:
        raise RuntimeError(f"tensor {name} must be flat and has stride = 1")
    want = torch.float32 if real else (torch.int32 if int_bytes == 4 else torch.int64)
    if t.dtype != want:
        raise RuntimeError(f"tensor {name} must have dtype {str(want).replace('torch.', '')}")
    if device_index == -1:
        if t.device.type != "cpu":
            raise RuntimeError(f"tensor {name} must be on CPU")
    else:
        if t.device.type != "cuda":
            raise RuntimeError(f"tensor {name} must be on CUDA")
        if t.device.index != device_index:
            raise RuntimeError(f"tensor {name} must be on CUDA device {device_index}")


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


class _LUTDataManager:
    _INT_MODE = False

    def __init__(self, n_inputs, n_outputs, n_detectors, n_anchors_per_detector, sequence_length, positional_dim,
                 initial_synapse_capacity, forward_group_size, backward_group_size, int_rescaler=1.0):
        for value, name in ((n_inputs, "n_inputs"), (n_outputs, "n_outputs"), (n_detectors, "n_detectors"),
                            (n_anchors_per_detector, "n_anchors_per_detector"), (sequence_length, "sequence_length"),
                            (forward_group_size, "forward_group_size"), (backward_group_size, "backward_group_size")):
            if int(value) <= 0:
                raise ValueError(f"{name} == 0")
        if forward_group_size > _MAX_GROUP:
            raise ValueError("forward_group_size > LUT_RUNTIME_KERNELS_TPB")
        self._n_inputs = int(n_inputs)
        self._n_outputs = int(n_outputs)
        self._n_detectors = int(n_detectors)
        self._n_anchors = int(n_anchors_per_detector)
        self._seq_len = int(sequence_length)
        self._pos_dim = int(positional_dim)
        self._fwd_group = int(forward_group_size)
        self._bwd_group = int(backward_group_size)
        self._int_rescaler = float(int_rescaler)
        bits = self._n_anchors + ((self._n_anchors + self._pos_dim) if self._seq_len > 1 else 0)
        if bits > 30:
            raise ValueError("lookup table too large: more than 2^30 rows per detector")
        self._rows_per_detector = 1 << bits
        self._n_lookup_neurons = self._n_detectors * self._rows_per_detector
        self._metas = []
        self._fully_connected = None
        self._device = -1
        self._forward_seen = False
        self._sparse = None
        self._timers = {}

    # ------------------------------------------------------------------ description
    def get_smallest_distinguishable_fraction(self):
        return (1.0 / _DENOM32) / self._int_rescaler if self._INT_MODE else 0.0

    def get_epsilon(self):
        return _EPS

    def get_summations_data_type(self):
        return "int32" if self._INT_MODE else "float32"

    def get_number_of_inputs(self):
        return self._n_inputs

    def get_number_of_outputs(self):
        return self._n_outputs

    def get_number_of_detectors(self):
        return self._n_detectors

    def get_number_of_lookup_neurons(self):
        return self._n_lookup_neurons

    def get_number_of_anchors_per_detector(self):
        return self._n_anchors

    def get_number_of_synapses(self):
        if self._fully_connected:
            return self._n_lookup_neurons * self._n_outputs
        return 0 if self._sparse is None else int(self._sparse.n_synapses)

    def count_synapses(self, neuron_indices_to_process):
        """Number of lookup -> output synapses of the given lookup neurons (reference: lut.cu:1182-1193)."""
        if self._fully_connected:
            raise ValueError("count_synapses: there is nothing to count in fully connected mode")
        if self._sparse is None:
            raise ValueError("sparse connectivity has not been attached yet")
        return int(self._sparse.synapses_of(neuron_indices_to_process)[0].numel())

    def export_synapses(self, weights, neuron_indices_to_process, target_internal_source_indices, target_weights,
                        target_internal_target_indices, target_synapse_meta_indices=None):
        """Fills the caller's tensors with one entry per synapse of the given lookup neurons: lookup neuron id,
        weight, and the output's neuron id (outputs are numbered after the lookup neurons), in neuron order and
        synapse order inside a neuron (reference: lut.cu:1195-1221).  Not a hot path: plain tensor indexing."""
        if self._fully_connected:
            raise ValueError("export_synapses: there is nothing to export in fully connected mode")
        if self._sparse is None:
            raise ValueError("sparse connectivity has not been attached yet")
        src, slot, tgt = self._sparse.synapses_of(neuron_indices_to_process)
        n = src.numel()
        for t, name in ((target_internal_source_indices, "target_internal_source_indices"),
                        (target_weights, "target_weights"),
                        (target_internal_target_indices, "target_internal_target_indices")):
            if t.numel() < n:
                raise ValueError(f"{name} holds {t.numel()} entries, {n} synapses to export")
        dev = target_weights.device
        target_internal_source_indices.view(-1)[:n] = src.to(dev).to(target_internal_source_indices.dtype)
        target_weights.view(-1)[:n] = weights.detach().view(-1)[slot.to(weights.device)].to(dev)
        target_internal_target_indices.view(-1)[:n] = (tgt + self._n_lookup_neurons).to(dev).to(
            target_internal_target_indices.dtype)
        if target_synapse_meta_indices is not None:
            target_synapse_meta_indices.view(-1)[:n] = 0

    def get_weights_dimension(self):
        if self._fully_connected:
            return self._n_lookup_neurons * self._n_outputs
        if self._sparse is None:
            raise ValueError("sparse connectivity has not been attached yet")
        return int(self._sparse.n_weights)

    def get_max_forward_groups_per_neuron(self):
        if self._fully_connected:
            return (self._n_outputs + self._fwd_group - 1) // self._fwd_group
        if self._sparse is None:
            return 0
        return int(self._sparse.max_groups_per_neuron)

    def __repr__(self):
        return (f"LUTDataManager(backend: spiky_b200; summation type: {self.get_summations_data_type()}; "
                f"smallest distinguishable fraction: {self.get_smallest_distinguishable_fraction()}; "
                f"n_synapses: {self.get_number_of_synapses() if self._fully_connected is not None else 0}; "
                f"n_detectors: {self._n_detectors}; n_lookup_neurons: {self._n_lookup_neurons})")

    def get_memory_stats(self):
        n = 0 if self._sparse is None else self._sparse.nbytes()
        return f"sparse index: {n // 1024} KB\n"

    def get_profiling_stats(self):
        # Timings are opt-in CUDA-event measurements collected by the layer (no forced synchronisation
        # inside runtime calls, unlike the reference's always-on profiler, spiky_cuda/misc/misc.h:14,170-214).
        lines = []
        for name, (total_ms, count) in sorted(self._timers.items()):
            lines.append(f"{name}: {total_ms:.4f} ms / {count} = {total_ms / max(count, 1):.4f} ms")
        return "\n".join(lines)

    def reset_profiler(self):
        self._timers = {}

    def _record_time(self, name, ms):
        total, count = self._timers.get(name, (0.0, 0))
        self._timers[name] = (total + ms, count + 1)

    # ------------------------------------------------------------------ set-up
    def register_synapse_meta(self, learning_rate, min_synaptic_weight, max_synaptic_weight, initial_noise_level,
                              initial_weight):
        if self._fully_connected is not None:
            raise ValueError("can't register new synapse metas after neurons were initialized")
        if learning_rate < 0.0:
            raise ValueError("learning_rate < 0")
        if learning_rate > 1.0:
            raise ValueError("learning_rate > 1")
        if self._INT_MODE and learning_rate > 0.0 and learning_rate * self._int_rescaler < 1.0 / _DENOM32:
            raise ValueError(f"too small value for 'learning_rate' {learning_rate} "
                             f"(less than smallest distinguishable fraction {1.0 / _DENOM32})")
        if min_synaptic_weight > max_synaptic_weight:
            raise ValueError("min_synaptic_weight > max_synaptic_weight")
        if initial_weight < min_synaptic_weight:
            raise ValueError("initial_weight < min_synaptic_weight")
        if initial_weight > max_synaptic_weight:
            raise ValueError("initial_weight > max_synaptic_weight")
        meta = (float(learning_rate), float(min_synaptic_weight), float(max_synaptic_weight),
                float(initial_noise_level), float(initial_weight))
        if meta in self._metas:
            return self._metas.index(meta)
        self._metas.append(meta)
        return len(self._metas) - 1

    def initialize_neurons(self, is_fully_connected):
        if not self._metas:
            raise ValueError("no synapse metas were registered")
        if is_fully_connected and len(self._metas) > 1:
            raise ValueError("fully connected mode is not compatible with multiple synapse metas")
        self._fully_connected = bool(is_fully_connected)

    def set_sparse_index(self, index):
        """Attach the compact connectivity of a sparse (projection / convolution) layer."""
        if self._fully_connected is not False:
            raise ValueError("sparse connectivity can only be attached in sparse mode")
        self._sparse = index

    def to_device(self, device):
        """device: CUDA ordinal, or -1 for host (set-up only)."""
        self._device = int(device)
        if self._sparse is not None:
            self._sparse.to_device(self._device)

    # ------------------------------------------------------------------ runtime helpers
    def _lr_meta(self):
        # the reference stores the rate as fp32 (BaseSynapseMeta.lr) and widens it to double
        return float(torch.tensor(self._metas[0][0], dtype=torch.float32).item())

    def _cfg(self, cmp_eps=0.0, sliced=False, seq_len=None):
        return LayerCfg(
            n_inputs=self._n_inputs, n_outputs=self._n_outputs, n_detectors=self._n_detectors,
            n_anchors=self._n_anchors, seq_len=self._seq_len if seq_len is None else seq_len, pos_dim=self._pos_dim,
            forward_group=self._fwd_group, backward_group=self._bwd_group, int_mode=int(self._INT_MODE),
            sliced_product=int(bool(sliced)), cmp_eps=float(cmp_eps), reserved0=0.0,
            int_rescaler=self._int_rescaler, lr_meta=self._lr_meta(),
        )

    def _require_cuda(self):
        if self._device < 0:
            raise RuntimeError("spiky_b200 has no CPU execution path: move the layer to a CUDA device first")

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self._device).cuda_stream)

    # ------------------------------------------------------------------ non-sequence runtime
    def forward_step(self, r_weights, batch_size, r_input, r_detector_anchors, w_output, w_lookup_indices,
                     cmp_eps=0.0, r_stream_handles=None, w_min_anchor_deltas=None, w_min_anchor_delta_indices=None):
        self._require_cuda()
        dev = self._device
        _check_tensor(r_weights, "r_weights", True, dev)
        _check_tensor(r_input, "r_input", True, dev)
        _check_tensor(r_detector_anchors, "r_detector_anchors", False, dev)
        _check_tensor(w_output, "w_output", True, dev)
        _check_tensor(w_lookup_indices, "w_lookup_indices", False, dev)
        if w_min_anchor_deltas is not None:
            _check_tensor(w_min_anchor_deltas, "w_min_anchor_deltas", True, dev)
        if w_min_anchor_delta_indices is not None:
            _check_tensor(w_min_anchor_delta_indices, "w_min_anchor_delta_indices", False, dev)
        if batch_size == 0:
            raise ValueError("batch_size == 0")
        if self._seq_len != 1:
            raise ValueError("forward_step should only be called when sequence_length == 1")
        B = int(batch_size)
        self._expect(r_input, B * self._n_inputs, "r_input")
        self._expect(w_output, B * self._n_outputs, "w_output")
        self._expect(w_lookup_indices, B * self._n_detectors, "w_lookup_indices")
        self._expect(r_detector_anchors, self._n_detectors * self._n_anchors * 2, "r_detector_anchors")
        self._expect(r_weights, self.get_weights_dimension(), "r_weights")
        cfg = self._cfg(cmp_eps)
        L = _native.lib()
        with torch.cuda.device(dev):
            if self._fully_connected:
                rc = L.lutb_nonseq_fc_forward(ctypes.byref(cfg), B, _ptr(r_weights), _ptr(r_input),
                                              _ptr(r_detector_anchors), _ptr(w_output), _ptr(w_lookup_indices),
                                              _ptr(w_min_anchor_deltas), _ptr(w_min_anchor_delta_indices),
                                              self._stream())
            else:
                rc = self._sparse_forward(L, cfg, B, r_weights, r_input, r_detector_anchors, w_output,
                                          w_lookup_indices, w_min_anchor_deltas, w_min_anchor_delta_indices)
        _native.check(rc)
        self._forward_seen = True

    def backward_backprop(self, r_weights, batch_size, r_output_gradients, r_detector_anchors, r_lookup_indices,
                          r_min_anchor_deltas, r_min_anchor_delta_indices, w_input_gradients, external_lr,
                          w_weights_gradients=None, r_stream_handles=None, dw_variant=_native.DW_AUTO,
                          workspace=None):
        if batch_size == 0:
            raise ValueError("batch_size == 0")
        if not self._forward_seen:
            raise ValueError("no active context")
        self._require_cuda()
        dev = self._device
        _check_tensor(r_weights, "r_weights", True, dev)
        # w_input_gradients=None (an extension of the reference's signature): the input gradient is not wanted, its
        # kernels are skipped
        if w_input_gradients is not None:
            _check_tensor(w_input_gradients, "w_input_gradients", True, dev)
        _check_tensor(r_output_gradients, "r_output_gradients", True, dev)
        _check_tensor(r_detector_anchors, "r_detector_anchors", False, dev)
        _check_tensor(r_lookup_indices, "r_lookup_indices", False, dev)
        _check_tensor(r_min_anchor_deltas, "r_min_anchor_deltas", True, dev)
        _check_tensor(r_min_anchor_delta_indices, "r_min_anchor_delta_indices", False, dev)
        if w_weights_gradients is not None:
            _check_tensor(w_weights_gradients, "w_weights_gradients", True, dev)
        if self._seq_len != 1:
            raise ValueError("backward_backprop should only be called when sequence_length == 1")
        if external_lr >= 0.0 and w_weights_gradients is not None:
            raise ValueError("in internal weight gradients mode w_weights_gradients should be nullptr")
        B = int(batch_size)
        self._expect(r_output_gradients, B * self._n_outputs, "r_output_gradients")
        if w_input_gradients is not None:
            self._expect(w_input_gradients, B * self._n_inputs, "w_input_gradients")
        self._expect(r_lookup_indices, B * self._n_detectors, "r_lookup_indices")
        if w_weights_gradients is not None and w_weights_gradients.numel() < self.get_weights_dimension():
            raise ValueError("w_weights_gradients is smaller than the weights")
        cfg = self._cfg()
        L = _native.lib()
        with torch.cuda.device(dev):
            if self._fully_connected:
                ws_bytes = L.lutb_nonseq_fc_backward_workspace(ctypes.byref(cfg), B, dw_variant)
                if ws_bytes and (workspace is None or workspace.numel() * workspace.element_size() < ws_bytes):
                    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=r_weights.device)
                rc = L.lutb_nonseq_fc_backward(ctypes.byref(cfg), B, _ptr(r_weights), _ptr(r_output_gradients),
                                               _ptr(r_detector_anchors), _ptr(r_lookup_indices),
                                               _ptr(r_min_anchor_deltas), _ptr(r_min_anchor_delta_indices),
                                               _ptr(w_input_gradients), _ptr(w_weights_gradients),
                                               float(external_lr), int(dw_variant), _ptr(workspace),
                                               0 if workspace is None else workspace.numel() * workspace.element_size(),
                                               self._stream())
            else:
                rc = self._sparse_backward(L, cfg, B, r_weights, r_output_gradients, r_detector_anchors,
                                           r_lookup_indices, r_min_anchor_deltas, r_min_anchor_delta_indices,
                                           w_input_gradients, external_lr, w_weights_gradients)
        _native.check(rc)

    def table_gradient_rows(self, batch_size, r_output_gradients, r_lookup_indices):
        """Table gradient of a fully connected non-sequence layer as a list of touched rows (not part of the
        reference's class, which forms the dense gradient and compacts it): returns ``(row_ids int64 [n],
        values fp32 [n, n_outputs])`` with ``row_ids = detector * 2^Nc + row`` ascending.  fp32 accumulators only.
        Reads the number of touched rows back from the device (like the reference's converter does)."""
        self._require_cuda()
        if not self._fully_connected or self._seq_len != 1:
            raise ValueError("the row-list table gradient exists for fully connected non-sequence layers")
        B, O, Nt = int(batch_size), self._n_outputs, self._n_detectors
        self._expect(r_output_gradients, B * O, "r_output_gradients")
        self._expect(r_lookup_indices, B * Nt, "r_lookup_indices")
        cfg = self._cfg()
        L = _native.lib()
        dev = r_output_gradients.device
        capacity = min(B, 1 << self._n_anchors) * Nt
        with torch.cuda.device(self._device):
            ws_bytes = L.lutb_nonseq_fc_table_grad_rows_workspace(ctypes.byref(cfg), B)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            row_ids = torch.empty(capacity, dtype=torch.int64, device=dev)
            values = torch.empty(capacity * O, dtype=torch.float32, device=dev)
            count = torch.zeros(1, dtype=torch.int64, device=dev)
            rc = L.lutb_nonseq_fc_table_grad_rows(ctypes.byref(cfg), B, _ptr(r_output_gradients), _ptr(r_lookup_indices),
                                                  _ptr(row_ids), _ptr(values), capacity, _ptr(count), _ptr(ws), ws_bytes,
                                                  self._stream())
        _native.check(rc)
        n = int(count.item())
        return row_ids[:n], values[:n * O].view(n, O)

    def table_gradient(self, batch_size, r_output_gradients, r_lookup_indices, w_target, scale, chunk_begin=0,
                       chunk_end=None):
        """Table-gradient pass alone (sparse layers, fp32) over the detector chunks [chunk_begin, chunk_end):
        ``w_target[row(t, idx[b, t]) + p] += scale * lr_meta * dY[b, target(p)]``.  ``w_target`` is a dense gradient
        or the weights themselves (``scale = -learning_rate``); ``r_lookup_indices`` may be uint8 / int16 / int32.
        Not part of the reference's class: used by the data-parallel sharded table update."""
        self._require_cuda()
        dev = self._device
        if self._fully_connected or self._sparse is None:
            raise ValueError("table_gradient needs a layer with sparse lookup connectivity")
        _check_tensor(r_output_gradients, "r_output_gradients", True, dev)
        _check_tensor(w_target, "w_target", True, dev)
        idx = r_lookup_indices
        if not (isinstance(idx, torch.Tensor) and idx.is_contiguous() and idx.dim() == 1 and idx.device.type == "cuda"
                and idx.device.index == dev and idx.dtype in (torch.uint8, torch.int16, torch.int32)):
            raise RuntimeError("r_lookup_indices must be a flat contiguous uint8 / int16 / int32 tensor on the layer's device")
        B = int(batch_size)
        self._expect(r_output_gradients, B * self._n_outputs, "r_output_gradients")
        self._expect(idx, B * self._n_detectors, "r_lookup_indices")
        if w_target.numel() < self.get_weights_dimension():
            raise ValueError("w_target is smaller than the weights")
        if chunk_end is None:
            chunk_end = self._sparse.n_chunks
        cfg = self._cfg()
        sp = self._sparse.c_struct()
        with torch.cuda.device(dev):
            rc = _native.lib().lutb_nonseq_sparse_table_grad(
                ctypes.byref(cfg), ctypes.byref(sp), B, _ptr(r_output_gradients), _ptr(idx), idx.element_size(),
                _ptr(w_target), float(scale), int(chunk_begin), int(chunk_end), self._stream())
        _native.check(rc)

    # ------------------------------------------------------------------ product-mode sequence runtime
    def forward_step_product(self, r_weights, batch_size, sequence_length, r_input_1, r_input_2, r_detector_anchors,
                             w_output, n_inputs_1, n_inputs_2, sliced_mode, cmp_eps=0.0, r_positional_embeddings=None,
                             r_stream_handles=None, variant=_native.PRODUCT_AUTO, keep_histogram=False):
        """keep_histogram (not in the reference): the caller will run backward_backprop_product on the same inputs
        next (a training step); the row histogram this pass counts is then left in a workspace of its own and the
        backward pass does not count it again.  Only where the whole batch fits one pass within
        ``product_keep_limit`` bytes; silently off otherwise."""
        self._require_cuda()
        dev = self._device
        _check_tensor(r_weights, "r_weights", True, dev)
        _check_tensor(r_input_1, "r_input_1", True, dev)
        _check_tensor(r_input_2, "r_input_2", True, dev)
        _check_tensor(r_detector_anchors, "r_detector_anchors", False, dev)
        _check_tensor(w_output, "w_output", True, dev)
        if r_positional_embeddings is not None:
            _check_tensor(r_positional_embeddings, "r_positional_embeddings", True, dev)
        if batch_size == 0:
            raise ValueError("batch_size == 0")
        if self._seq_len != 1:
            raise ValueError("forward_step_product: this is an experimental method, this->sequence_length should be "
                             "equal to 1, real length of the sequence is passed as the method parameter")
        if sequence_length == 0:
            raise ValueError("sequence_length == 0")
        if not self._fully_connected:
            raise ValueError("product mode is only available for fully connected layers in this backend")
        B, S = int(batch_size), int(sequence_length)
        self._expect(r_input_1, B * S * n_inputs_1, "r_input_1")
        self._expect(r_input_2, B * S * n_inputs_2, "r_input_2")
        self._expect(w_output, B * S * self._n_outputs, "w_output")
        self._expect(r_weights, self.get_weights_dimension(), "r_weights")
        if self._pos_dim > 0:
            if r_positional_embeddings is None:
                raise ValueError("r_positional_embeddings is required when positional_dim > 0")
            self._expect(r_positional_embeddings, (S - 1) * self._n_detectors * self._pos_dim, "r_positional_embeddings")
        cfg = self._cfg(cmp_eps, sliced=sliced_mode)
        self._kept_histogram = None
        with torch.cuda.device(dev):
            ws, ws_bytes = self._product_workspace(cfg, B, S, False, variant, r_weights.device)
            flags = 0
            if keep_histogram and ws is not None:
                L = _native.lib()
                want = L.lutb_product_workspace(ctypes.byref(cfg), B, S, 1)
                if 0 < want <= _LUTDataManager.product_keep_limit:
                    own = torch.empty(want, dtype=torch.uint8, device=r_weights.device)
                    if L.lutb_product_keeps_histogram(ctypes.byref(cfg), B, S, int(n_inputs_1), int(n_inputs_2),
                                                      int(variant), _ptr(own), want):
                        ws, ws_bytes, flags = own, want, _native.PRODUCT_KEEP_HIST
                        self._kept_histogram = (own, self._histogram_key(
                            B, S, r_input_1, r_input_2, r_detector_anchors, r_positional_embeddings, n_inputs_1,
                            n_inputs_2, sliced_mode, cmp_eps, variant))
            rc = _native.lib().lutb_product_forward(
                ctypes.byref(cfg), B, S, _ptr(r_weights), _ptr(r_input_1), _ptr(r_input_2), int(n_inputs_1),
                int(n_inputs_2), _ptr(r_positional_embeddings), _ptr(r_detector_anchors), _ptr(w_output),
                int(variant) | flags, _ptr(ws), ws_bytes, self._stream())
        _native.check(rc)
        self._forward_seen = True

    _kept_histogram = None
    # largest workspace a forward pass may hold on to until its backward pass (per layer)
    product_keep_limit = 2 << 30

    @staticmethod
    def _histogram_key(B, S, x1, x2, anchors, pe, e1, e2, sliced, cmp_eps, variant):
        """What the row histogram depends on: the inputs (storage and version), anchors, embeddings and geometry."""
        def ident(t):
            return None if t is None else (t.data_ptr(), t._version, t.numel())
        return (B, S, ident(x1), ident(x2), ident(anchors), ident(pe), int(e1), int(e2), bool(sliced), float(cmp_eps),
                int(variant))

    def backward_backprop_product(self, r_weights, batch_size, sequence_length, r_input_1, r_input_2,
                                  r_detector_anchors, r_output_gradients, w_input_gradients_1, w_input_gradients_2,
                                  external_lr, n_inputs_1, n_inputs_2, sliced_mode, cmp_eps=0.0,
                                  w_weights_gradients=None, r_positional_embeddings=None,
                                  w_positional_embeddings_gradients=None, r_stream_handles=None,
                                  variant=_native.PRODUCT_AUTO):
        if batch_size == 0:
            raise ValueError("batch_size == 0")
        if not self._forward_seen:
            raise ValueError("no active context")
        self._require_cuda()
        dev = self._device
        for t, name in ((r_weights, "r_weights"), (r_input_1, "r_input_1"), (r_input_2, "r_input_2"),
                        (r_output_gradients, "r_output_gradients"), (w_input_gradients_1, "w_input_gradients_1"),
                        (w_input_gradients_2, "w_input_gradients_2")):
            _check_tensor(t, name, True, dev)
        _check_tensor(r_detector_anchors, "r_detector_anchors", False, dev)
        for t, name in ((w_weights_gradients, "w_weights_gradients"),
                        (r_positional_embeddings, "r_positional_embeddings"),
                        (w_positional_embeddings_gradients, "w_positional_embeddings_gradients")):
            if t is not None:
                _check_tensor(t, name, True, dev)
        if external_lr >= 0.0 and w_weights_gradients is not None:
            raise ValueError("in internal weight gradients mode w_weights_gradients should be nullptr")
        B, S = int(batch_size), int(sequence_length)
        self._expect(r_output_gradients, B * S * self._n_outputs, "r_output_gradients")
        self._expect(w_input_gradients_1, B * S * n_inputs_1, "w_input_gradients_1")
        self._expect(w_input_gradients_2, B * S * n_inputs_2, "w_input_gradients_2")
        cfg = self._cfg(cmp_eps, sliced=sliced_mode)
        kept, self._kept_histogram = self._kept_histogram, None
        with torch.cuda.device(dev):
            ws, ws_bytes = self._product_workspace(cfg, B, S, True, variant, r_weights.device)
            if kept is not None and kept[1] == self._histogram_key(
                    B, S, r_input_1, r_input_2, r_detector_anchors, r_positional_embeddings, n_inputs_1, n_inputs_2,
                    sliced_mode, cmp_eps, variant):
                # the forward pass over these very inputs left its histogram in this workspace
                ws, ws_bytes, variant = kept[0], kept[0].numel(), int(variant) | _native.PRODUCT_REUSE_HIST
            rc = _native.lib().lutb_product_backward(
                ctypes.byref(cfg), B, S, _ptr(r_weights), _ptr(r_input_1), _ptr(r_input_2), int(n_inputs_1),
                int(n_inputs_2), _ptr(r_positional_embeddings), _ptr(r_detector_anchors), _ptr(r_output_gradients),
                _ptr(w_input_gradients_1), _ptr(w_input_gradients_2), _ptr(w_positional_embeddings_gradients),
                _ptr(w_weights_gradients), float(external_lr), int(variant), _ptr(ws), ws_bytes, self._stream())
        _native.check(rc)

    # scratch of the histogram variant of the product kernels: one buffer per device, shared by all layers
    # (a call only uses it between its own launches on the current stream)
    _product_scratch = {}
    product_scratch_limit = 16 << 30

    def _product_workspace(self, cfg, B, S, backward, variant, device):
        """(tensor or None, bytes) handed to the product entry points; None lets AUTO fall back to DIRECT."""
        if variant == _native.PRODUCT_DIRECT or self._INT_MODE or S < 2:
            return None, 0
        rows = 1 << self._n_anchors
        L = _native.lib()
        # the library's own rule for AUTO (include/spiky_b200.h): no workspace is needed when it will pick DIRECT
        quarter = backward or bool(L.lutb_fp32_gemm_available())
        if variant == _native.PRODUCT_AUTO and not ((4 * S >= rows) if quarter else (S >= rows)):
            return None, 0
        one = L.lutb_product_workspace(ctypes.byref(cfg), 1, S, int(backward))
        want = min(L.lutb_product_workspace(ctypes.byref(cfg), B, S, int(backward)),
                   max(one, _LUTDataManager.product_scratch_limit))
        buf = _LUTDataManager._product_scratch.get(device)
        if buf is None or buf.numel() < want:
            _LUTDataManager._product_scratch[device] = None
            buf = torch.empty(want, dtype=torch.uint8, device=device)
            _LUTDataManager._product_scratch[device] = buf
        return buf, buf.numel()

    # ------------------------------------------------------------------ concatenation-mode sequence runtime
    def forward_step_concat(self, r_weights, batch_size, r_input, r_detector_anchors, w_output, w_lookup_indices,
                            cmp_eps=0.0, r_positional_embeddings=None, w_positional_lookup_indices=None,
                            w_min_anchor_deltas=None, w_min_anchor_delta_indices=None,
                            w_positional_min_deltas=None, w_positional_min_delta_indices=None,
                            r_stream_handles=None):
        self._require_cuda()
        dev = self._device
        _check_tensor(r_weights, "r_weights", True, dev)
        _check_tensor(r_input, "r_input", True, dev)
        _check_tensor(r_detector_anchors, "r_detector_anchors", False, dev)
        _check_tensor(w_output, "w_output", True, dev)
        _check_tensor(w_lookup_indices, "w_lookup_indices", False, dev)
        for t, name, real in ((r_positional_embeddings, "r_positional_embeddings", True),
                              (w_positional_lookup_indices, "w_positional_lookup_indices", False),
                              (w_min_anchor_deltas, "w_min_anchor_deltas", True),
                              (w_min_anchor_delta_indices, "w_min_anchor_delta_indices", False),
                              (w_positional_min_deltas, "w_positional_min_deltas", True),
                              (w_positional_min_delta_indices, "w_positional_min_delta_indices", False)):
            if t is not None:
                _check_tensor(t, name, real, dev)
        if batch_size == 0:
            raise ValueError("batch_size == 0")
        if self._seq_len <= 1:
            raise ValueError("forward_step_concat should only be called when sequence_length > 1")
        B, S = int(batch_size), self._seq_len
        self._expect(r_input, B * S * self._n_inputs, "r_input")
        self._expect(w_output, B * S * self._n_outputs, "w_output")
        self._expect(w_lookup_indices, B * S * self._n_detectors, "w_lookup_indices")
        self._expect(r_weights, self.get_weights_dimension(), "r_weights")
        if self._pos_dim > 0 and (r_positional_embeddings is None or w_positional_lookup_indices is None):
            raise ValueError("positional embeddings and their index buffer are required when positional_dim > 0")
        cfg = self._cfg(cmp_eps)
        with torch.cuda.device(dev):
            fn, head = _native.lib().lutb_concat_forward, (ctypes.byref(cfg),)
            if not self._fully_connected:
                if self._sparse is None:
                    raise ValueError("sparse connectivity is not attached")
                sp = self._sparse.c_struct()
                fn, head = _native.lib().lutb_concat_sparse_forward, (ctypes.byref(cfg), ctypes.byref(sp))
            rc = fn(
                *head, B, _ptr(r_weights), _ptr(r_input), _ptr(r_detector_anchors),
                _ptr(r_positional_embeddings), _ptr(w_output), _ptr(w_lookup_indices), _ptr(w_min_anchor_deltas),
                _ptr(w_min_anchor_delta_indices), _ptr(w_positional_lookup_indices), _ptr(w_positional_min_deltas),
                _ptr(w_positional_min_delta_indices), self._stream())
        _native.check(rc)
        self._forward_seen = True

    def backward_backprop_concat(self, r_weights, batch_size, r_output_gradients, r_detector_anchors,
                                 r_lookup_indices, r_min_anchor_deltas, r_min_anchor_delta_indices,
                                 w_input_gradients, external_lr, r_positional_lookup_indices=None,
                                 r_positional_min_deltas=None, r_positional_min_delta_indices=None,
                                 w_positional_embeddings_gradients=None, w_weights_gradients=None,
                                 r_stream_handles=None):
        if batch_size == 0:
            raise ValueError("batch_size == 0")
        if not self._forward_seen:
            raise ValueError("no active context")
        self._require_cuda()
        dev = self._device
        for t, name, real in ((r_weights, "r_weights", True), (r_output_gradients, "r_output_gradients", True),
                              (r_detector_anchors, "r_detector_anchors", False),
                              (r_lookup_indices, "r_lookup_indices", False),
                              (r_min_anchor_deltas, "r_min_anchor_deltas", True),
                              (r_min_anchor_delta_indices, "r_min_anchor_delta_indices", False),
                              (w_input_gradients, "w_input_gradients", True)):
            _check_tensor(t, name, real, dev)
        for t, name, real in ((r_positional_lookup_indices, "r_positional_lookup_indices", False),
                              (r_positional_min_deltas, "r_positional_min_deltas", True),
                              (r_positional_min_delta_indices, "r_positional_min_delta_indices", False),
                              (w_positional_embeddings_gradients, "w_positional_embeddings_gradients", True),
                              (w_weights_gradients, "w_weights_gradients", True)):
            if t is not None:
                _check_tensor(t, name, real, dev)
        if external_lr >= 0.0 and w_weights_gradients is not None:
            raise ValueError("in internal weight gradients mode w_weights_gradients should be nullptr")
        B, S = int(batch_size), self._seq_len
        self._expect(r_output_gradients, B * S * self._n_outputs, "r_output_gradients")
        self._expect(w_input_gradients, B * S * self._n_inputs, "w_input_gradients")
        cfg = self._cfg()
        with torch.cuda.device(dev):
            fn, head = _native.lib().lutb_concat_backward, (ctypes.byref(cfg),)
            if not self._fully_connected:
                if self._sparse is None:
                    raise ValueError("sparse connectivity is not attached")
                sp = self._sparse.c_struct()
                fn, head = _native.lib().lutb_concat_sparse_backward, (ctypes.byref(cfg), ctypes.byref(sp))
            rc = fn(
                *head, B, _ptr(r_weights), _ptr(r_output_gradients), _ptr(r_detector_anchors),
                _ptr(r_lookup_indices), _ptr(r_min_anchor_deltas), _ptr(r_min_anchor_delta_indices),
                _ptr(r_positional_lookup_indices), _ptr(r_positional_min_deltas),
                _ptr(r_positional_min_delta_indices), _ptr(w_input_gradients),
                _ptr(w_positional_embeddings_gradients), _ptr(w_weights_gradients), float(external_lr),
                self._stream())
        _native.check(rc)

    # ------------------------------------------------------------------ stages of the concatenation-mode layer
    # (no counterpart in the reference's data manager, which runs them inside forward_step_concat /
    # backward_backprop_concat; exposed separately for ranks that shard the query positions of a sequence)
    def check_detectors(self, rows, r_input, r_detector_anchors, w_lookup_indices, cmp_eps=0.0,
                        w_min_anchor_deltas=None, w_min_anchor_delta_indices=None):
        """Table indices (and minimum-margin pairs) of ``rows`` input rows."""
        self._require_cuda()
        self._expect(r_input, rows * self._n_inputs, "r_input")
        self._expect(w_lookup_indices, rows * self._n_detectors, "w_lookup_indices")
        cfg = self._cfg(cmp_eps)
        with torch.cuda.device(self._device):
            rc = _native.lib().lutb_check_detectors(ctypes.byref(cfg), int(rows), _ptr(r_input), _ptr(r_detector_anchors),
                                                    _ptr(w_lookup_indices), _ptr(w_min_anchor_deltas),
                                                    _ptr(w_min_anchor_delta_indices), self._stream())
        _native.check(rc)

    def check_positional(self, r_positional_embeddings, w_positional_lookup_indices, cmp_eps=0.0,
                         w_positional_min_deltas=None, w_positional_min_delta_indices=None):
        self._require_cuda()
        cfg = self._cfg(cmp_eps)
        with torch.cuda.device(self._device):
            rc = _native.lib().lutb_check_positional(ctypes.byref(cfg), _ptr(r_positional_embeddings),
                                                     _ptr(w_positional_lookup_indices), _ptr(w_positional_min_deltas),
                                                     _ptr(w_positional_min_delta_indices), self._stream())
        _native.check(rc)

    def concat_pairs_forward(self, r_weights, batch_size, r_lookup_indices, r_positional_lookup_indices, w_output,
                             j_begin, j_end):
        """Outputs of the queries [j_begin, j_end) from the table indices of all tokens."""
        self._require_cuda()
        if not self._fully_connected:
            raise ValueError("query-range stages exist for fully connected concatenation-mode layers only")
        B, S = int(batch_size), self._seq_len
        self._expect(r_lookup_indices, B * S * self._n_detectors, "r_lookup_indices")
        self._expect(w_output, B * S * self._n_outputs, "w_output")
        cfg = self._cfg()
        with torch.cuda.device(self._device):
            rc = _native.lib().lutb_concat_pairs_forward(ctypes.byref(cfg), B, _ptr(r_weights), _ptr(r_lookup_indices),
                                                         _ptr(r_positional_lookup_indices), _ptr(w_output), int(j_begin),
                                                         int(j_end), self._stream())
        _native.check(rc)
        self._forward_seen = True

    def concat_pairs_backward(self, r_weights, batch_size, r_output_gradients, r_detector_anchors, r_lookup_indices,
                              r_min_anchor_deltas, r_min_anchor_delta_indices, w_input_gradients, external_lr,
                              r_positional_lookup_indices, r_positional_min_deltas, r_positional_min_delta_indices,
                              w_positional_embeddings_gradients, w_weights_gradients, j_begin, j_end):
        """Partial gradients from the pairs whose query lies in [j_begin, j_end)."""
        self._require_cuda()
        if not self._fully_connected:
            raise ValueError("query-range stages exist for fully connected concatenation-mode layers only")
        B, S = int(batch_size), self._seq_len
        self._expect(r_output_gradients, B * S * self._n_outputs, "r_output_gradients")
        self._expect(w_input_gradients, B * S * self._n_inputs, "w_input_gradients")
        cfg = self._cfg()
        with torch.cuda.device(self._device):
            rc = _native.lib().lutb_concat_pairs_backward(
                ctypes.byref(cfg), B, _ptr(r_weights), _ptr(r_output_gradients), _ptr(r_detector_anchors),
                _ptr(r_lookup_indices), _ptr(r_min_anchor_deltas), _ptr(r_min_anchor_delta_indices),
                _ptr(r_positional_lookup_indices), _ptr(r_positional_min_deltas), _ptr(r_positional_min_delta_indices),
                _ptr(w_input_gradients), _ptr(w_positional_embeddings_gradients), _ptr(w_weights_gradients),
                float(external_lr), int(j_begin), int(j_end), self._stream())
        _native.check(rc)

    @staticmethod
    def _expect(t, numel, name):
        if t.numel() != numel:
            raise ValueError(f"{name} has {t.numel()} elements, expected {numel}")

    def _sparse_forward(self, L, cfg, B, r_weights, r_input, r_detector_anchors, w_output, w_lookup_indices,
                        w_min_anchor_deltas, w_min_anchor_delta_indices):
        if self._sparse is None:
            raise ValueError("sparse connectivity is not attached")
        sp = self._sparse.c_struct()
        return L.lutb_nonseq_sparse_forward(ctypes.byref(cfg), ctypes.byref(sp), B, _ptr(r_weights), _ptr(r_input),
                                            _ptr(r_detector_anchors), _ptr(w_output), _ptr(w_lookup_indices),
                                            _ptr(w_min_anchor_deltas), _ptr(w_min_anchor_delta_indices),
                                            self._stream())

    def _sparse_backward(self, L, cfg, B, r_weights, r_output_gradients, r_detector_anchors, r_lookup_indices,
                         r_min_anchor_deltas, r_min_anchor_delta_indices, w_input_gradients, external_lr,
                         w_weights_gradients):
        if self._sparse is None:
            raise ValueError("sparse connectivity is not attached")
        sp = self._sparse.c_struct()
        return L.lutb_nonseq_sparse_backward(ctypes.byref(cfg), ctypes.byref(sp), B, _ptr(r_weights),
                                             _ptr(r_output_gradients), _ptr(r_detector_anchors),
                                             _ptr(r_lookup_indices), _ptr(r_min_anchor_deltas),
                                             _ptr(r_min_anchor_delta_indices), _ptr(w_input_gradients),
                                             _ptr(w_weights_gradients), float(external_lr), self._stream())


class LUTDataManagerF(_LUTDataManager):
    """fp32 accumulators (reference: LUTDataManagerF, spiky_cuda/lut/lut.cu:1477-1480)."""

    _INT_MODE = False

    def __init__(self, n_inputs, n_outputs, n_detectors, n_anchors_per_detector, sequence_length, positional_dim,
                 initial_synapse_capacity, forward_group_size, backward_group_size):
        super().__init__(n_inputs, n_outputs, n_detectors, n_anchors_per_detector, sequence_length, positional_dim,
                         initial_synapse_capacity, forward_group_size, backward_group_size, 1.0)


class LUTDataManagerI(_LUTDataManager):
    """int32 fixed-point accumulators, order-independent sums (reference: LUTDataManagerI, lut.cu:1481-1483)."""

    _INT_MODE = True

    def __init__(self, n_inputs, n_outputs, n_detectors, n_anchors_per_detector, sequence_length, positional_dim,
                 initial_synapse_capacity, forward_group_size, backward_group_size, int_rescaler):
        if not int_rescaler > 0:
            raise ValueError("int_rescaler must be positive")
        super().__init__(n_inputs, n_outputs, n_detectors, n_anchors_per_detector, sequence_length, positional_dim,
                         initial_synapse_capacity, forward_group_size, backward_group_size, int_rescaler)
