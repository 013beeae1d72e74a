"""PyTorch layer API of the LUT hot path: same class names, constructor arguments, attributes and
autograd behaviour as the reference's ``spiky.lut.LUTLayer`` module (src/spiky/lut/LUTLayer.py), with
the runtime calls served by the B200 CUDA library through :mod:`spiky_b200.lut_data_manager`.

What stays identical for a user of the reference: ``GradientType`` / ``GradientPolicy`` /
``SynapseMeta`` / ``LUTSharedContext``; ``LUTLayer``, ``Conv2DLUTLayer``, ``ProjectionLUTLayer``
constructors; ``forward`` on ``[B, S, *input_shape]`` float32 contiguous input; ``forward_step*`` /
``backward_step*``; the flat ``_weights`` / ``_positional_embeddings`` parameters and the flat int32
``_detector_anchors``; the three weight-gradient policies.

What differs: kernels run on torch's current stream and nothing synchronises the host; structure
(anchor pairs, sparse connectivity) is derived with torch ops instead of the reference's
synapse-growth engine, so freshly constructed layers draw different random anchors than the reference
does for the same seed (inject ``_explicit_anchors`` or use ``load_structure`` to reproduce a
reference-built layer); anchors are a persistent buffer, so ``state_dict()`` round-trips them.
"""
from dataclasses import dataclass
from enum import Enum
from typing import List

import torch
import torch.nn as nn

from .lut_data_manager import LUTDataManagerF, LUTDataManagerI
from . import structure as _structure
from .structure import PointSamplingPolicy, PointSamplingType  # noqa: F401  (part of the public surface)


class GradientType(Enum):
    """How weight gradients leave the layer (reference: LUTLayer.py:18-22)."""
    Sparse = 0    # torch.sparse_coo gradient holding only touched cells
    Dense = 1     # dense gradient tensor
    Internal = 2  # no gradient: the backward kernel applies -lr * grad to the weights in place


@dataclass(frozen=True)
class GradientPolicy:
    type: GradientType
    normalized: bool = False

    def __post_init__(self):
        if self.normalized and self.type == GradientType.Internal:
            raise ValueError("normalized cannot be combined with Internal gradient policy")


@dataclass(frozen=True, order=True)
class SynapseMeta:
    learning_rate: float = 1.0
    min_weight: float = 0.0
    max_weight: float = 1.0
    initial_noise_level: float = 0.0
    initial_weight: float = 0.0

    def __post_init__(self):
        assert 0.0 <= self.learning_rate <= 1.0
        assert self.min_weight <= self.initial_weight <= self.max_weight


class LUTSharedContext(object):
    """Scratch buffers shared by the layers of one model (reference: LUTLayer.py:49-194).

    Holds the reusable dense gradient buffer of the Sparse policy and the comparison dead band
    ``_cmp_eps``.  The reference also keeps three CUDA streams per ``multi_id`` here; this backend
    launches on the current stream, so ``get_cuda_streams`` returns None.
    """

    def __init__(self, do_asserts=False, _cmp_eps=0.0):
        self._grad_buffers = {}
        self._device = None
        self._do_asserts = do_asserts
        self._cmp_eps = _cmp_eps

    def to_device(self, device):
        dev = device if isinstance(device, torch.device) else torch.device(device)
        if dev.type == "cuda" and dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        self._device = dev
        self._grad_buffers = {k: v.to(dev) for k, v in self._grad_buffers.items()}
        return self

    def get_weight_gradients_buffer(self, numel, device, multi_id=0):
        if self._device is None:
            raise RuntimeError("LUTSharedContext device is None, call to_device(...) first")
        if self._device != device:
            raise RuntimeError(f"LUTSharedContext is on {self._device}, but trying to get buffer on {device}")
        buf = self._grad_buffers.get(multi_id)
        if buf is None or buf.numel() < numel:
            buf = torch.zeros(numel, dtype=torch.float32, device=device)
            self._grad_buffers[multi_id] = buf
        if self._do_asserts:
            assert torch.count_nonzero(buf) == 0
        return buf[:numel]

    def get_dense_to_sparse_converter(self, multi_id=0):
        """One reusable converter per multi_id (reference: LUTLayer.py:88-94)."""
        from .torch_utils import DenseToSparseConverter
        convs = self.__dict__.setdefault("_dense_to_sparse_converters", {})
        if multi_id not in convs:
            convs[multi_id] = DenseToSparseConverter()
        return convs[multi_id]

    def get_cuda_streams(self, device, multi_id=0):
        return None

    def get_cuda_stream(self, device, multi_id=0, stream_index=0):
        return None


def _normalise_device(device):
    dev = device if isinstance(device, torch.device) else torch.device(device)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    return dev


class _LUTFunction(torch.autograd.Function):
    """Autograd bridge (reference: LUTLayerBasic.LUTForwardFN, LUTLayer.py:1117-1181)."""

    @staticmethod
    def forward(ctx, x, weights, pos_embeddings, layer):
        if not layer.training:
            if layer._sequence_length == 1:
                return layer.forward_step(x)
            if layer._concatenation_product:
                return layer.forward_step_concat(x, pos_embeddings)
            return layer.forward_step_product(x, pos_embeddings)
        ctx.layer = layer
        if layer._sequence_length == 1:
            out, idx, md, mk = layer.forward_step(x)
            ctx.save_for_backward(x, idx, md, mk)
            ctx.mode = "nonseq"
            fwd_hook = getattr(layer, "_table_forward_hook", None)
            if fwd_hook is not None:
                # data-parallel sharded table update: the table indices can travel to the other ranks right away,
                # while the rest of the forward pass and the backward pass above this layer still run
                fwd_hook(layer, idx.reshape(-1), x.shape[0])
        elif layer._concatenation_product:
            out, *saved = layer.forward_step_concat(x, pos_embeddings)
            ctx.has_pe = saved[3] is not None
            ctx.save_for_backward(x, *[s for s in saved if s is not None])
            ctx.mode = "concat"
        else:
            out = layer.forward_step_product(x, pos_embeddings)
            if pos_embeddings is None:
                ctx.save_for_backward(x)
            else:
                ctx.save_for_backward(x, pos_embeddings)
            ctx.mode = "product"
        return out

    @staticmethod
    def backward(ctx, grad_output):
        layer = ctx.layer
        if ctx.mode == "nonseq":
            x, idx, md, mk = ctx.saved_tensors
            dx, dw = layer.backward_step(x, grad_output, idx, md, mk, need_input_grad=ctx.needs_input_grad[0])
            return dx, dw, None, None
        if ctx.mode == "concat":
            saved = list(ctx.saved_tensors)
            x, idx, md, mk = saved[:4]
            pe_state = saved[4:7] if ctx.has_pe else (None, None, None)
            dx, dw, dpe = layer.backward_step_concat(x, grad_output, idx, md, mk, *pe_state)
            return dx, dw, dpe, None
        saved = ctx.saved_tensors
        x = saved[0]
        pe = saved[1] if len(saved) > 1 else None
        dx, dw, dpe = layer.backward_step_product(x, pe, grad_output)
        return dx, dw, dpe, None


class LUTLayerBasic(nn.Module):
    """Common machinery of all LUT layers (reference: LUTLayerBasic, LUTLayer.py:197-1242)."""

    # kept under the reference's name for code that reaches for it
    LUTForwardFN = _LUTFunction

    @staticmethod
    def n_lut_channels(n_anchors_per_detector, sequence_length, concatentation_product=True):
        if concatentation_product:
            return 1 << (n_anchors_per_detector * (2 if sequence_length > 1 else 1))
        return 1 << n_anchors_per_detector

    def __init__(self, n_inputs, n_outputs, n_detectors, n_anchors_per_detector, is_fully_connected, sequence_length,
                 synapse_metas: List[SynapseMeta], concatenation_product=True, sliced_product_mode=False,
                 positional_dim=None, unified_pe=False, weights_gradient_policy: GradientPolicy = None,
                 shared_context: LUTSharedContext = None, summation_dtype=torch.float32, _int_rescaler=0.001,
                 _initial_synapse_capacity=None, _forward_group_size: int = 32, _backward_group_size: int = 32,
                 random_seed=None):
        super().__init__()
        assert len(synapse_metas) > 0
        assert sequence_length > 0
        if sequence_length == 1 and not concatenation_product:
            raise ValueError("concatenation_product == False doesn't make sense with sequence_length == 1")
        if sliced_product_mode and concatenation_product:
            raise ValueError("sliced_product_mode == True doesn't make sense in concatenation product mode")
        if sliced_product_mode and n_inputs != positional_dim:
            raise ValueError("if sliced_product_mode == True then n_inputs and positional_dim should be equal")
        if sequence_length > 1:
            assert positional_dim is not None, "positional_dim must be provided when sequence_length > 1"
        else:
            assert positional_dim is None, "positional_dim must be None when sequence_length == 1"
        if weights_gradient_policy is None:
            weights_gradient_policy = GradientPolicy(GradientType.Dense)
        if summation_dtype == torch.int32 and weights_gradient_policy.type == GradientType.Internal:
            raise ValueError("summation dtype torch.int32 can't be combined with GradientType.Internal")
        if is_fully_connected:
            assert len(synapse_metas) == 1, "fully connected mode is not compatible with multiple synapse metas"

        self.device = torch.device("cpu")
        self._n_inputs = n_inputs
        self._n_outputs = n_outputs
        self._n_detectors = n_detectors
        self._n_anchors_per_detector = n_anchors_per_detector
        self._is_fully_connected = is_fully_connected
        self._forward_group_size = _forward_group_size
        self._backward_group_size = _backward_group_size
        self._sequence_length = sequence_length
        self._multi_id = 0
        self._concatenation_product = concatenation_product
        self._sliced_product_mode = sliced_product_mode
        self._unified_positional_embeddings = unified_pe
        self._positional_dim = positional_dim
        self._weights_gradient_policy = weights_gradient_policy
        self._external_lr_hook = None
        self._lookup_indices_callback = None
        self._synapse_metas = synapse_metas
        self._dw_variant = 0

        self._own_shared_context = shared_context is None
        if shared_context is None:
            shared_context = LUTSharedContext().to_device(self.device)
        self._shared_context = shared_context

        # learnable positional embeddings of sequence layers, uniform in [-1, 1]
        if sequence_length > 1 and positional_dim > 0:
            gen = None
            if random_seed is not None:
                gen = torch.Generator(device="cpu")
                gen.manual_seed(random_seed)
            n_pe = (sequence_length - 1) * (1 if unified_pe else n_detectors) * positional_dim
            pe = torch.empty(n_pe, dtype=torch.float32).uniform_(-1.0, 1.0, generator=gen)
            self._positional_embeddings = nn.Parameter(pe)
        else:
            self._positional_embeddings = None

        # the native manager sees the virtual input vector [x_i | x_j | pe] in product mode
        dm_inputs = n_inputs if concatenation_product else 2 * n_inputs + positional_dim
        dm_seq = sequence_length if concatenation_product else 1
        dm_args = (dm_inputs, n_outputs, n_detectors, n_anchors_per_detector, dm_seq,
                   positional_dim if positional_dim is not None else 0,
                   0 if _initial_synapse_capacity is None else _initial_synapse_capacity,
                   _forward_group_size, _backward_group_size)
        if summation_dtype == torch.float32:
            self._lut_dm = LUTDataManagerF(*dm_args)
        else:
            self._lut_dm = LUTDataManagerI(*dm_args, _int_rescaler)
        self._n_lookup_neurons = self._lut_dm.get_number_of_lookup_neurons()
        for i, sm in enumerate(synapse_metas):
            m_id = self._lut_dm.register_synapse_meta(
                learning_rate=sm.learning_rate, min_synaptic_weight=sm.min_weight, max_synaptic_weight=sm.max_weight,
                initial_noise_level=sm.initial_noise_level, initial_weight=sm.initial_weight)
            assert m_id == i
        self._lut_dm.initialize_neurons(is_fully_connected)

        self._weights = None
        self.register_buffer("_detector_anchors", None, persistent=True)

    # ------------------------------------------------------------------ getters
    def _virtual_inputs(self):
        return self._n_inputs if self._concatenation_product else 2 * self._n_inputs + self._positional_dim

    def get_input_neuron_ids(self):
        return torch.arange(0, self._virtual_inputs(), dtype=torch.int32, device=self.device)

    def get_detector_neuron_ids(self):
        n = self._virtual_inputs()
        return torch.arange(n, n + self._n_detectors, dtype=torch.int32, device=self.device)

    def get_lookup_neuron_ids(self):
        return torch.arange(0, self._n_lookup_neurons, dtype=torch.int32, device=self.device)

    def get_output_neuron_ids(self):
        return torch.arange(self._n_lookup_neurons, self._n_lookup_neurons + self._n_outputs, dtype=torch.int32,
                            device=self.device)

    def n_inputs(self):
        return self._n_inputs

    def n_lookup_neurons(self):
        return self._n_lookup_neurons

    def n_outputs(self):
        return self._n_outputs

    def n_detectors(self):
        return self._n_detectors

    def n_anchors_per_detector(self):
        return self._n_anchors_per_detector

    def sequence_length(self):
        return self._sequence_length

    def n_synapses(self):
        if self._is_fully_connected:
            return self._n_lookup_neurons * self._n_outputs
        return self._lut_dm.get_number_of_synapses()

    def input_shape(self):
        return (self._n_inputs,)

    def output_shape(self):
        return (self._n_outputs,)

    def __repr__(self):
        return (f"LUTLayerBasic({self.n_inputs()} inputs, {self.n_detectors()} detectors, "
                f"{self.n_anchors_per_detector()} anchors per detector, {self.n_outputs()} outputs, "
                f"{self.n_synapses()} synapses, {self._lut_dm})")

    def get_smallest_distinguishable_fraction(self) -> float:
        return self._lut_dm.get_smallest_distinguishable_fraction()

    def get_epsilon(self) -> float:
        return self._lut_dm.get_epsilon()

    def get_summation_type(self) -> torch.dtype:
        return torch.int32 if self._lut_dm.get_summations_data_type() == "int32" else torch.float32

    def get_memory_stats(self) -> str:
        return self._lut_dm.get_memory_stats()

    def get_profiling_stats(self) -> str:
        return self._lut_dm.get_profiling_stats()

    def reset_profiler(self):
        self._lut_dm.reset_profiler()

    def set_external_learning_rate_hook(self, hook_fn):
        """hook_fn(weights) -> float learning rate, queried on every backward of the Internal policy."""
        if self._weights_gradient_policy.type != GradientType.Internal:
            raise ValueError("external_learning_rate_hook can only be used with GradientPolicy.Internal")
        if hook_fn is None:
            raise ValueError("external_learning_rate_hook cannot be None when using GradientPolicy.Internal")
        self._external_lr_hook = hook_fn

    def _reset_shared_context(self, new_context):
        self._shared_context = new_context
        self._own_shared_context = False

    def _set_lookup_indices_callback(self, cb):
        assert self._sequence_length == 1
        self._lookup_indices_callback = cb

    def _export_anchors(self):
        if self._detector_anchors is None:
            raise RuntimeError("Detectors are not initialized, call initialize_detectors() first")
        return self._detector_anchors.view(self._n_detectors, self._n_anchors_per_detector, 2)

    def _count_synapses(self, neuron_ids):
        if self._is_fully_connected:
            return self._n_lookup_neurons * self._n_outputs
        return self._lut_dm.count_synapses(neuron_ids)

    def _export_synapses(self, neuron_ids, source_ids, weights, target_ids, synapse_metas=None):
        """One entry per synapse of the given lookup neurons into the caller's tensors: lookup neuron id, weight,
        output neuron id (outputs are numbered after the lookup neurons) (reference: LUTLayer.py:1206-1230)."""
        if self._is_fully_connected:
            source_ids[:] = neuron_ids.view(neuron_ids.numel(), -1).repeat(1, self._n_outputs).flatten()
            weights[:] = self._weights.detach().view(self._n_lookup_neurons, self._n_outputs)[neuron_ids.long()].flatten()
            target_ids[:] = torch.arange(self._n_outputs, device=self.device, dtype=torch.int32).repeat(
                neuron_ids.numel())
            target_ids += self._n_lookup_neurons
            if synapse_metas is not None:
                synapse_metas[:] = 0.0
        else:
            self._lut_dm.export_synapses(self._weights, neuron_ids, source_ids, weights, target_ids, synapse_metas)

    def _export_all_synapses(self):
        n = self.n_synapses()
        source_ids = torch.zeros([n], dtype=torch.int32, device=self.device)
        target_ids = torch.zeros([n], dtype=torch.int32, device=self.device)
        weights = torch.zeros([n], dtype=torch.float32, device=self.device)
        self._export_synapses(self.get_lookup_neuron_ids(), source_ids, weights, target_ids)
        return weights, source_ids, target_ids

    # ------------------------------------------------------------------ structure
    def _set_anchors(self, anchors):
        anchors = anchors.to(dtype=torch.int32, device=self.device).reshape(-1).contiguous()
        assert anchors.numel() == self._n_detectors * self._n_anchors_per_detector * 2
        self._detector_anchors = anchors

    def _init_fc_weights(self, do_normalise_weights=False):
        sm = self._synapse_metas[0]
        n_weights = self._lut_dm.get_weights_dimension()
        with torch.no_grad():
            w = torch.rand(n_weights, dtype=torch.float32, device=self.device)
            w.mul_(sm.initial_noise_level).add_(sm.initial_weight).clip_(sm.min_weight, sm.max_weight)
            if do_normalise_weights:
                w = w.view(self._n_lookup_neurons, self._n_outputs)
                w /= w.norm(dim=-1, keepdim=True)
                w = w.T.flatten()
        self._weights = nn.Parameter(w)

    def to(self, *args, **kwargs):
        device = kwargs.get("device", args[0] if args else None)
        super().to(*args, **kwargs)
        if device is None or isinstance(device, torch.dtype):
            return self
        dev = _normalise_device(device)
        self.device = dev
        self._lut_dm.to_device(dev.index if dev.type == "cuda" else -1)
        if self._own_shared_context:
            self._shared_context.to_device(dev)
        return self

    # ------------------------------------------------------------------ runtime: non-sequence
    def _check_input(self, x, seq_len):
        want = tuple(self.input_shape())
        if not (x.dim() == len(want) + 2 and tuple(x.shape[2:]) == want):
            raise ValueError(f"Input x has invalid shape {tuple(x.shape)}; expected (B, {seq_len}, {', '.join(map(str, want))})")
        assert x.device == self.device, f"input on {x.device}, layer on {self.device}"
        assert x.shape[1] == seq_len, f"Input sequence_length {x.shape[1]} does not match constructor sequence_length {seq_len}"
        if x.dtype != torch.float32:
            raise RuntimeError("tensor r_input must have dtype float32")
        return x.contiguous()

    def forward_step(self, x, output=None):
        assert self._sequence_length == 1
        x = self._check_input(x, 1)
        B = x.shape[0]
        dev = self.device
        external = output is not None
        if not external:
            output = torch.zeros(B * self._n_outputs, dtype=torch.float32, device=dev)
        idx = torch.empty(B * self._n_detectors, dtype=torch.int32, device=dev)
        md = mk = None
        if self.training:
            md = torch.empty(B * self._n_detectors, dtype=torch.float32, device=dev)
            mk = torch.empty(B * self._n_detectors, dtype=torch.int32, device=dev)
        self._lut_dm.forward_step(self._weights.detach(), B, x.view(-1), self._detector_anchors, output, idx,
                                  self._shared_context._cmp_eps, None, md, mk)
        if not external and self.training and self._lookup_indices_callback is not None:
            self._lookup_indices_callback(idx, md, mk)
        out_view = None if external else output.view((B, 1) + tuple(self.output_shape()))
        if self.training:
            shape = (B, 1, self._n_detectors)
            extra = (idx.view(shape), md.view(shape), mk.view(shape))
            return extra if external else (out_view,) + extra
        return out_view

    def _weight_grad_target(self):
        policy = self._weights_gradient_policy.type
        if policy == GradientType.Internal:
            return None
        if policy == GradientType.Sparse:
            numel = ((self._weights.numel() + 3) // 4) * 4
            return self._shared_context.get_weight_gradients_buffer(numel, self.device, self._multi_id)
        return torch.zeros_like(self._weights, requires_grad=False)

    def _external_lr(self):
        if self._weights_gradient_policy.type != GradientType.Internal:
            return -1.0
        if self._external_lr_hook is None:
            raise ValueError("external_learning_rate_hook must be set when using GradientPolicy.Internal")
        return float(self._external_lr_hook(self._weights))

    # Sparse gradient policy of fully connected non-sequence layers: the (cell, value) lists come straight from
    # the table-gradient pass (rows the batch touched) instead of a dense gradient that is compacted afterwards;
    # set to False to take the reference's dense-then-compact route
    _sparse_rows_direct = True

    def _backward_step_sparse_rows(self, x, grad_output, lookup_indices, min_anchor_deltas, min_anchor_delta_indices,
                                   x_grad, batch_size):
        """Input gradient by the usual kernels, table gradient as a list of touched rows; the result is the sparse
        tensor ``_process_gradients`` builds from the dense gradient: cell indices ascending, zero cells dropped."""
        from ._native import SKIP_TABLE_GRADIENT
        dm = self._lut_dm
        grad_flat = grad_output.contiguous().view(-1)
        idx_flat = lookup_indices.reshape(-1)
        if x_grad is not None:
            dm.backward_backprop(self._weights.detach(), batch_size, grad_flat, self._detector_anchors, idx_flat,
                                 min_anchor_deltas.reshape(-1), min_anchor_delta_indices.reshape(-1), x_grad.view(-1),
                                 SKIP_TABLE_GRADIENT, None, None)
        dx = None if x_grad is None else x_grad.view(x.shape)
        rows, values = dm.table_gradient_rows(batch_size, grad_flat, idx_flat)
        if rows.numel() == 0:
            return dx, None
        O = values.shape[1]
        # zero cells (an output gradient that is exactly zero or below the threshold) are not part of the list
        flat = values.reshape(-1)
        pad = (-flat.numel()) % 4
        if pad:
            flat = torch.cat([flat, flat.new_zeros(pad)])
        nz, vals = self._shared_context.get_dense_to_sparse_converter(self._multi_id).dense_to_sparse_32(flat)
        if nz is None:
            return dx, None
        cells = rows[nz // O] * O + nz % O
        if self._weights_gradient_policy.normalized:
            vals /= vals.abs().max().clip(1e-16)
        return dx, torch.sparse_coo_tensor(cells.unsqueeze(0), vals, size=self._weights.shape, device=self.device,
                                           check_invariants=False, is_coalesced=True)

    def _process_gradients(self, w_grad, batch_size):
        """Apply the gradient policy to the dense table gradient (reference: LUTLayer.py:567-609)."""
        policy = self._weights_gradient_policy
        if w_grad is None:
            return None
        if policy.type == GradientType.Sparse:
            # compaction kernel (sorted, deterministic); erases the shared buffer so the next layer gets it clean
            nz, values = self._shared_context.get_dense_to_sparse_converter(self._multi_id).dense_to_sparse_32(
                w_grad, erase_input=True)
            if nz is None:
                return None
            if policy.normalized:
                values /= values.abs().max().clip(1e-16)
            return torch.sparse_coo_tensor(nz.unsqueeze(0), values, size=self._weights.shape, device=self.device,
                                           check_invariants=False, is_coalesced=True)
        if policy.normalized:
            w_grad /= w_grad.abs().max().clip(1e-16)
        return w_grad

    def backward_step(self, x, grad_output, lookup_indices, min_anchor_deltas, min_anchor_delta_indices, x_grad=None,
                      need_input_grad=True):
        """need_input_grad=False (not in the reference, which always computes it): the input-gradient kernels are
        skipped and None is returned in its place; autograd asks for this when the layer's input needs no gradient
        (the first layer of a network fed with data)."""
        assert self._sequence_length == 1
        x = self._check_input(x, 1)
        B = x.shape[0]
        shape = (B, 1, self._n_detectors)
        assert lookup_indices.shape == shape and min_anchor_deltas.shape == shape
        assert min_anchor_delta_indices.shape == shape
        assert grad_output.shape == (B, 1) + tuple(self.output_shape())
        external = x_grad is not None
        if not external and need_input_grad:
            x_grad = torch.zeros(x.numel(), dtype=torch.float32, device=self.device)
        if (not external and self._weights_gradient_policy.type == GradientType.Sparse and self._is_fully_connected
                and self._lut_dm.get_summations_data_type() == "float32" and self._sparse_rows_direct):
            return self._backward_step_sparse_rows(x, grad_output, lookup_indices, min_anchor_deltas,
                                                   min_anchor_delta_indices, x_grad, B)
        hook = getattr(self, "_table_update_hook", None)
        if hook is not None and not external:
            # data-parallel sharded table update: only the input gradient is computed here; the hook gathers the
            # (index, output gradient) pairs of all ranks and updates this rank's share of the tables in place
            from ._native import SKIP_TABLE_GRADIENT
            grad_flat = grad_output.contiguous().view(-1)
            if x_grad is not None:
                self._lut_dm.backward_backprop(
                    self._weights.detach(), B, grad_flat, self._detector_anchors, lookup_indices.reshape(-1),
                    min_anchor_deltas.reshape(-1), min_anchor_delta_indices.reshape(-1), x_grad.view(-1),
                    SKIP_TABLE_GRADIENT, None, None)
            hook(self, lookup_indices.reshape(-1), grad_flat, B)
            return (None if x_grad is None else x_grad.view(x.shape)), None
        sink = None if external else getattr(self, "_table_gradient_sink", None)
        # data-parallel update over peer memory: the dense table gradient goes into the sink's shared buffer and the
        # sink reduces it over the ranks and updates the tables; the parameter gets no .grad
        w_grad = self._weight_grad_target() if sink is None else sink.gradient_buffer(self)
        self._lut_dm.backward_backprop(
            self._weights.detach(), B, grad_output.contiguous().view(-1), self._detector_anchors,
            lookup_indices.reshape(-1), min_anchor_deltas.reshape(-1), min_anchor_delta_indices.reshape(-1),
            None if x_grad is None else x_grad.view(-1), self._external_lr(), w_grad, None, dw_variant=self._dw_variant)
        if sink is not None:
            sink.gradient_ready(self)
            return (None if x_grad is None else x_grad.view(x.shape)), None
        if not external:
            w_grad = self._process_gradients(w_grad, B)
            return (None if x_grad is None else x_grad.view(x.shape)), w_grad
        return (w_grad,)

    # ------------------------------------------------------------------ runtime: sequence layers
    def _prepare_positional_embeddings(self):
        if self._positional_embeddings is None:
            return None
        if self._unified_positional_embeddings:
            return self._positional_embeddings.reshape(self._sequence_length - 1, 1, self._positional_dim).repeat(
                1, self._n_detectors, 1).flatten().contiguous()
        return self._positional_embeddings

    def forward_step_concat(self, x, pos_embeddings, output=None):
        assert self._concatenation_product
        x = self._check_input(x, self._sequence_length)
        B, S, Nt, dev = x.shape[0], x.shape[1], self._n_detectors, self.device
        external = output is not None
        if not external:
            output = torch.zeros(B * S * self._n_outputs, dtype=torch.float32, device=dev)
        train = self.training
        idx = torch.empty(B * S * Nt, dtype=torch.int32, device=dev)
        md = torch.empty(B * S * Nt, dtype=torch.float32, device=dev) if train else None
        mk = torch.empty(B * S * Nt, dtype=torch.int32, device=dev) if train else None
        pidx = pmd = pmk = pe = None
        if self._positional_dim > 0:
            pe = pos_embeddings.detach().contiguous().view(-1)
            pidx = torch.empty((S - 1) * Nt, dtype=torch.int32, device=dev)
            if train:
                pmd = torch.empty((S - 1) * Nt, dtype=torch.float32, device=dev)
                pmk = torch.empty((S - 1) * Nt, dtype=torch.int32, device=dev)
        self._lut_dm.forward_step_concat(self._weights.detach(), B, x.view(-1), self._detector_anchors, output, idx,
                                         self._shared_context._cmp_eps, pe, pidx, md, mk, pmd, pmk, None)
        result = () if external else (output.view((B, S) + tuple(self.output_shape())),)
        if not train:
            return None if external else result[0]
        tok = (B, S, Nt)
        state = (idx.view(tok), md.view(tok), mk.view(tok))
        if self._positional_dim > 0:
            state += (pidx.view(S - 1, Nt), pmd.view(S - 1, Nt), pmk.view(S - 1, Nt))
        else:
            state += (None, None, None)
        return result + state

    def backward_step_concat(self, x, grad_output, lookup_indices, min_anchor_deltas, min_anchor_delta_indices,
                             positional_lookup_indices, positional_min_deltas, positional_min_delta_indices,
                             x_grad=None):
        assert self._concatenation_product
        x = self._check_input(x, self._sequence_length)
        B, S, Nt = x.shape[0], x.shape[1], self._n_detectors
        assert lookup_indices.shape == (B, S, Nt)
        assert grad_output.shape == (B, S) + tuple(self.output_shape())
        if self._positional_dim > 0:
            assert positional_lookup_indices.shape == (S - 1, Nt)
        else:
            assert positional_lookup_indices is None and positional_min_deltas is None
        external = x_grad is not None
        if not external:
            x_grad = torch.zeros(x.numel(), dtype=torch.float32, device=self.device)
        w_grad = self._weight_grad_target()
        pe_grad = None
        if self._positional_dim > 0:
            pe_grad = torch.zeros((S - 1) * Nt * self._positional_dim, dtype=torch.float32, device=self.device)

        def flat(t):
            return None if t is None else t.reshape(-1)

        self._lut_dm.backward_backprop_concat(
            self._weights.detach(), B, grad_output.contiguous().view(-1), self._detector_anchors,
            flat(lookup_indices), flat(min_anchor_deltas), flat(min_anchor_delta_indices), x_grad.view(-1),
            self._external_lr(), flat(positional_lookup_indices), flat(positional_min_deltas),
            flat(positional_min_delta_indices), pe_grad, w_grad, None)
        if not external:
            w_grad = self._process_gradients(w_grad, B)
        if pe_grad is not None and self._weights_gradient_policy.normalized:
            pe_grad /= pe_grad.abs().max().clip(1e-16)
        if external:
            return w_grad, pe_grad
        return x_grad.view(x.shape), w_grad, pe_grad

    def forward_step_product(self, x, pos_embeddings, output=None):
        assert not self._concatenation_product
        x = self._check_input(x, self._sequence_length)
        B, S = x.shape[0], x.shape[1]
        external = output is not None
        if not external:
            output = torch.zeros(B * S * self._n_outputs, dtype=torch.float32, device=self.device)
        xf = x.view(-1)
        pe = None if pos_embeddings is None else pos_embeddings.detach().contiguous().view(-1)
        self._lut_dm.forward_step_product(self._weights.detach(), B, S, xf, xf, self._detector_anchors, output,
                                          self._n_inputs, self._n_inputs, self._sliced_product_mode,
                                          self._shared_context._cmp_eps, pe, None,
                                          variant=getattr(self, "_product_variant", 0),
                                          keep_histogram=self.training)
        return None if external else output.view((B, S) + tuple(self.output_shape()))

    def backward_step_product(self, x, pos_embeddings, grad_output, x_grad=None):
        assert not self._concatenation_product
        x = self._check_input(x, self._sequence_length)
        B, S = x.shape[0], x.shape[1]
        assert grad_output.shape == (B, S) + tuple(self.output_shape())
        external = x_grad is not None
        if not external:
            x_grad = torch.zeros(x.numel(), dtype=torch.float32, device=self.device)
        w_grad = self._weight_grad_target()
        pe = pe_grad = None
        if self._positional_dim > 0:
            pe = pos_embeddings.detach().contiguous().view(-1)
            pe_grad = torch.zeros_like(pe)
        xf, gf = x.view(-1), x_grad.view(-1)
        self._lut_dm.backward_backprop_product(
            self._weights.detach(), B, S, xf, xf, self._detector_anchors, grad_output.contiguous().view(-1), gf, gf,
            self._external_lr(), self._n_inputs, self._n_inputs, self._sliced_product_mode,
            self._shared_context._cmp_eps, w_grad, pe, pe_grad, None, variant=getattr(self, "_product_variant", 0))
        if not external:
            w_grad = self._process_gradients(w_grad, B)
        if pe_grad is not None and self._weights_gradient_policy.normalized:
            pe_grad /= pe_grad.abs().max().clip(1e-16)
        if external:
            return w_grad, pe_grad
        return x_grad.view(x.shape), w_grad, pe_grad

    def load_structure(self, anchors, source_ids, weight_slots, target_ids, n_weights):
        """Adopt the structure of a reference-built layer: its anchor pairs and its synapse export (per
        synapse: lookup neuron id, slot in the flat weight array, output index).  Weights of that layer
        can then be copied into ``_weights`` verbatim."""
        self._set_anchors(torch.as_tensor(anchors))
        index = _structure.SparseIndex.from_export(
            source_ids, weight_slots, target_ids, self._n_detectors, self._n_lookup_neurons // self._n_detectors,
            self._forward_group_size, self._n_outputs, n_weights)
        self._lut_dm.set_sparse_index(index)
        self._weights = nn.Parameter(torch.zeros(n_weights, dtype=torch.float32, device=self.device))
        self._lut_dm.to_device(self.device.index if self.device.type == "cuda" else -1)
        return self

    def forward(self, x):
        if self._sequence_length == 1:
            return _LUTFunction.apply(x, self._weights, None, self)
        return _LUTFunction.apply(x, self._weights, self._prepare_positional_embeddings(), self)


class Conv2DLUTLayer(LUTLayerBasic):
    """Detectors on sliding receptive fields of a 2-D input, outputs fully connected or through a second
    sliding window over the detector grid (reference: Conv2DLUTLayer, LUTLayer.py:1245-1437)."""

    def __init__(self, input_shape, n_anchors_per_detector, detectors_shape, output_kernel_shape, sequence_length=1,
                 receptive_field_shape=None, receptive_field_stride_shape=None, lut_receptive_field_shape=None,
                 lut_receptive_field_stride_shape=None, synapse_meta=SynapseMeta(), concatenation_product=True,
                 sliced_product_mode=False, positional_dim=None, unified_pe=False, do_normalise_weights=False,
                 weights_gradient_policy: GradientPolicy = None, shared_context: LUTSharedContext = None,
                 summation_dtype=torch.float32, _explicit_anchors=None, _int_rescaler=0.001, _forward_group_size=32,
                 _backward_group_size=32, _max_groups_in_growth_buffer=2 ** 20, random_seed=None, device=None):
        # the detectors see the virtual input [x_i | x_j | pe] in product mode
        if concatenation_product:
            virt_shape = tuple(input_shape)
        elif sliced_product_mode:
            virt_shape = (input_shape[0], input_shape[1] * 3)
        else:
            virt_shape = (input_shape[0], input_shape[1] * 2 + (positional_dim or 0))
        if receptive_field_shape is None:
            assert receptive_field_stride_shape is None
            rf, rf_stride = virt_shape, virt_shape
        elif concatenation_product:
            rf, rf_stride = tuple(receptive_field_shape), tuple(receptive_field_stride_shape)
        elif sliced_product_mode:
            rf = (receptive_field_shape[0], receptive_field_shape[1] * 3)
            rf_stride = (receptive_field_stride_shape[0], receptive_field_stride_shape[1] * 3)
        else:
            raise AssertionError("receptive fields are not supported in plain product mode")
        det_geo = _structure.SlidingWindows(virt_shape, rf, rf_stride, tuple(detectors_shape))
        lut_shape = det_geo.out_shape
        n_lut_channels = LUTLayerBasic.n_lut_channels(n_anchors_per_detector, sequence_length)
        n_inputs = input_shape[0] * input_shape[1]
        n_detectors = lut_shape[0] * lut_shape[1]
        if lut_receptive_field_shape is not None:
            out_geo = _structure.SlidingWindows(lut_shape, tuple(lut_receptive_field_shape),
                                                tuple(lut_receptive_field_stride_shape), tuple(output_kernel_shape))
            n_outputs = out_geo.out_shape[0] * out_geo.out_shape[1]
            self._lut_receptive_field_shape = tuple(lut_receptive_field_shape) + (n_lut_channels,)
            self._output_shape = out_geo.out_shape
        else:
            assert lut_receptive_field_stride_shape is None
            out_geo = None
            n_outputs = output_kernel_shape[0] * output_kernel_shape[1]
            self._lut_receptive_field_shape = lut_shape + (n_lut_channels,)
            self._output_shape = tuple(output_kernel_shape)
        self._input_shape = tuple(input_shape)
        self._lut_shape = lut_shape + (n_lut_channels,)
        self._detectors_shape = tuple(detectors_shape)

        super().__init__(
            n_inputs=n_inputs, n_outputs=n_outputs, n_detectors=n_detectors,
            n_anchors_per_detector=n_anchors_per_detector, is_fully_connected=out_geo is None,
            sequence_length=sequence_length, synapse_metas=[synapse_meta],
            concatenation_product=concatenation_product, sliced_product_mode=sliced_product_mode,
            positional_dim=positional_dim, unified_pe=unified_pe, weights_gradient_policy=weights_gradient_policy,
            shared_context=shared_context, summation_dtype=summation_dtype, _int_rescaler=_int_rescaler,
            _initial_synapse_capacity=0, _forward_group_size=_forward_group_size,
            _backward_group_size=_backward_group_size, random_seed=random_seed)

        if _explicit_anchors is None:
            pools, counts = det_geo.input_pools()
            anchors = _structure.sample_anchor_pairs(pools, counts, n_anchors_per_detector, random_seed)
        else:
            anchors = _explicit_anchors
        self._set_anchors(anchors)
        if out_geo is None:
            self._init_fc_weights(do_normalise_weights)
        else:
            assert not do_normalise_weights, "weights normalisation is currently supported in fully connected mode only"
            targets, tcounts = out_geo.output_targets()
            self._attach_sparse(targets, tcounts, synapse_meta, random_seed)
        if device is not None:
            self.to(device=device)

    def _attach_sparse(self, targets, counts, synapse_meta, random_seed):
        index = _structure.SparseIndex.from_detector_targets(
            targets, counts, rows_per_detector=self._n_lookup_neurons // self._n_detectors,
            group_size=self._forward_group_size, n_outputs=self._n_outputs)
        self._lut_dm.set_sparse_index(index)
        self._weights = nn.Parameter(index.initial_weights(synapse_meta, random_seed))

    def input_shape(self):
        return self._input_shape

    def output_shape(self):
        return self._output_shape

    def lut_shape(self):
        return self._lut_shape

    def detectors_shape(self):
        return self._detectors_shape

    def lut_receptive_field_shape(self):
        return self._lut_receptive_field_shape

    def export_weights(self, inverse_order=True):
        """Weights ordered by (output, lookup neuron) and shaped output_shape + lut_receptive_field_shape, or the
        other way round (reference: LUTLayer.py:1417-1437)."""
        weights, source_ids, target_ids = self._export_all_synapses()
        if inverse_order:
            order = torch.argsort(source_ids, stable=True)
            order = order[torch.argsort(target_ids[order], stable=True)]
            return weights[order].view(tuple(self.output_shape()) + tuple(self.lut_receptive_field_shape()))
        order = torch.argsort(target_ids, stable=True)
        order = order[torch.argsort(source_ids[order], stable=True)]
        return weights[order].view(tuple(self.lut_receptive_field_shape()) + tuple(self.output_shape()))

    def __repr__(self):
        return (f"Conv2DLUTLayer(input_shape={self.input_shape()}, output_shape={self.output_shape()}, "
                f"detectors_shape={self.detectors_shape()}, n_anchors_per_detector={self.n_anchors_per_detector()})")


class LUTLayer(Conv2DLUTLayer):
    """Fully connected LUT layer on a flat input (reference: LUTLayer, LUTLayer.py:1440-1508)."""

    def __init__(self, n_inputs, n_anchors_per_detector, n_detectors, n_outputs, sequence_length=1,
                 synapse_meta=SynapseMeta(), concatenation_product=True, sliced_product_mode=False,
                 positional_dim=None, unified_pe=False, do_normalise_weights=False,
                 weights_gradient_policy: GradientPolicy = None, shared_context: LUTSharedContext = None,
                 summation_dtype=torch.float32, _explicit_anchors=None, _int_rescaler=0.001, _forward_group_size=32,
                 _backward_group_size=32, _max_groups_in_growth_buffer=2 ** 20, random_seed=None, device=None):
        super().__init__(
            input_shape=(1, n_inputs), n_anchors_per_detector=n_anchors_per_detector,
            detectors_shape=(1, n_detectors), output_kernel_shape=(1, n_outputs), sequence_length=sequence_length,
            synapse_meta=synapse_meta, concatenation_product=concatenation_product,
            sliced_product_mode=sliced_product_mode, positional_dim=positional_dim, unified_pe=unified_pe,
            do_normalise_weights=do_normalise_weights, weights_gradient_policy=weights_gradient_policy,
            shared_context=shared_context, summation_dtype=summation_dtype, _explicit_anchors=_explicit_anchors,
            _int_rescaler=_int_rescaler, _forward_group_size=_forward_group_size,
            _backward_group_size=_backward_group_size, _max_groups_in_growth_buffer=_max_groups_in_growth_buffer,
            random_seed=random_seed, device=device)

    def input_shape(self):
        return self._input_shape[1:]

    def output_shape(self):
        return self._output_shape[1:]

    def detectors_shape(self):
        return self._detectors_shape[1:]

    def lut_shape(self):
        return self._lut_shape[1:]

    def lut_receptive_field_shape(self):
        return self._lut_receptive_field_shape[1:]

    def __repr__(self):
        return (f"LUTLayer({self.n_inputs()} inputs, {self.n_detectors()} detectors, {self.n_outputs()} outputs, "
                f"{self.n_anchors_per_detector()} anchors per detector)")


class ProjectionLUTLayer(LUTLayerBasic):
    """Groups of detectors on rectangles of a 2-D input; every table row of a group projects onto a small
    rectangle of the 2-D output around the group's (rescaled) centre
    (reference: ProjectionLUTLayer, LUTLayer.py:1511-1648)."""

    def __init__(self, input_shape, output_shape, n_anchors_per_detector, n_detector_groups, n_detectors_in_group,
                 receptive_shape, projection_shape, synapse_meta=SynapseMeta(), projection_prob=1.0,
                 detectors_sampling_policy: PointSamplingPolicy = PointSamplingPolicy(PointSamplingType.RandomUniform),
                 input_sparsity_mask=None, output_sparsity_mask=None, weights_gradient_policy: GradientPolicy = None,
                 shared_context: LUTSharedContext = None, summation_dtype=torch.float32, _int_rescaler=0.001,
                 _forward_group_size=32, _backward_group_size=32, _max_groups_in_growth_buffer=2 ** 20,
                 random_seed=None, device=None):
        assert n_detector_groups >= 1 and n_detectors_in_group >= 1
        assert 0.0 < projection_prob <= 1.0
        self._n_detector_groups = n_detector_groups
        self._n_detectors_in_group = n_detectors_in_group
        self._input_shape = tuple(input_shape)
        self._output_shape = tuple(output_shape)
        h, w = input_shape
        oh, ow = output_shape
        super().__init__(
            n_inputs=h * w, n_outputs=oh * ow, n_detectors=n_detector_groups * n_detectors_in_group,
            n_anchors_per_detector=n_anchors_per_detector, is_fully_connected=False, sequence_length=1,
            synapse_metas=[synapse_meta], weights_gradient_policy=weights_gradient_policy,
            shared_context=shared_context, summation_dtype=summation_dtype, _int_rescaler=_int_rescaler,
            _forward_group_size=_forward_group_size, _backward_group_size=_backward_group_size,
            random_seed=random_seed)

        centers = _structure.sample_centers(detectors_sampling_policy, n_detector_groups, h, w, random_seed)
        self._group_centers = centers
        # detector inputs: grid points within (r-1)/2 of the centre
        pools, counts = _structure.rectangle_members(centers, (receptive_shape[0] - 1) / 2 + 1e-4,
                                                     (receptive_shape[1] - 1) / 2 + 1e-4, h, w, input_sparsity_mask)
        pools = pools.repeat_interleave(n_detectors_in_group, dim=0)
        counts = counts.repeat_interleave(n_detectors_in_group)
        self._set_anchors(_structure.sample_anchor_pairs(pools, counts, n_anchors_per_detector, random_seed))
        # lookup -> output: output cells within r/2 of the centre rescaled to output coordinates
        scaled = centers.clone()
        scaled[:, 0] *= ow / w
        scaled[:, 1] *= oh / h
        targets, tcounts = _structure.rectangle_members(scaled, projection_shape[0] / 2 + 1e-4,
                                                        projection_shape[1] / 2 + 1e-4, oh, ow, output_sparsity_mask)
        if projection_prob < 1.0:
            gen = torch.Generator(device="cpu")
            if random_seed is not None:
                gen.manual_seed(int(random_seed) + 1)
            keep = (torch.rand(targets.shape, generator=gen) < projection_prob) & (targets >= 0)
            order = torch.argsort((~keep).to(torch.int8), dim=1, stable=True)
            targets = torch.where(torch.gather(keep, 1, order), torch.gather(targets, 1, order),
                                  torch.full_like(targets, -1))
            tcounts = keep.sum(dim=1)
        targets = targets.repeat_interleave(n_detectors_in_group, dim=0)
        tcounts = tcounts.repeat_interleave(n_detectors_in_group)
        index = _structure.SparseIndex.from_detector_targets(
            targets, tcounts, rows_per_detector=1 << n_anchors_per_detector, group_size=_forward_group_size,
            n_outputs=oh * ow)
        self._lut_dm.set_sparse_index(index)
        self._weights = nn.Parameter(index.initial_weights(synapse_meta, random_seed))
        if device is not None:
            self.to(device=device)

    def input_shape(self):
        return self._input_shape

    def output_shape(self):
        return self._output_shape

    def detectors_shape(self):
        return (self._n_detector_groups, self._n_detectors_in_group)

    def export_weights(self):
        """(weights, lookup neuron ids, output neuron ids) ordered by output, then lookup neuron
        (reference: LUTLayer.py:1629-1645)."""
        weights, source_ids, target_ids = self._export_all_synapses()
        order = torch.argsort(source_ids, stable=True)
        order = order[torch.argsort(target_ids[order], stable=True)]
        return weights[order], source_ids[order], target_ids[order]

    def __repr__(self):
        return (f"ProjectionLUTLayer(input_shape={self.input_shape()}, output_shape={self.output_shape()}, "
                f"n_detectors={self._n_detectors}, n_anchors_per_detector={self.n_anchors_per_detector()})")
