"""Forward-only inference for large fully connected LUT layers: int8 tables and detector sharding.

Neither exists in the reference (it has no quantised tables and is single-device).  Definitions:

* int8 tables: ``q int8 [Nt, T, O]`` with one fp32 scale per table.  Outputs are the reference's int32
  fixed-point forward (``LUTDataManagerI``) evaluated on the de-quantised table: ``dequant='f32'`` takes the
  entries as the fp32 numbers ``f32(scale[t] * q)`` (exactly what the reference would be handed, so the
  fixed-point oracle pins the arithmetic bit for bit), ``dequant='exact'`` (default, about four times faster) as
  the exact reals ``scale[t] * q``; the two differ by one fp32 rounding per entry before the block truncation.
* detector sharding: rank r owns detectors ``[r * Nt / G, (r + 1) * Nt / G)`` with their anchors and tables,
  the input batch is replicated, every rank produces partial sums for all outputs and one all-reduce
  combines them (int32 accumulators for int8 tables: exact, order independent; fp32 for fp32 tables).
"""
import ctypes

import torch
import torch.distributed as dist

from . import _native
from ._native import LayerCfg


def quantize_tables(weights, n_detectors, rows, n_outputs):
    """fp32 [Nt * T * O] -> (q int8 [Nt * T * O], scale fp32 [Nt]); symmetric, scale = max|W_t| / 127."""
    w = weights.detach().reshape(n_detectors, rows * n_outputs).to(torch.float32)
    scale = (w.abs().amax(dim=1) / 127.0).clamp_min(1e-30)
    q = torch.round(w / scale[:, None]).clamp_(-127, 127).to(torch.int8)
    return q.reshape(-1).contiguous(), scale.contiguous()


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


class LUTInference:
    """Eval-mode forward of a fully connected non-sequence LUT layer (or of one detector shard of it).

    tables: fp32 [Nt*T*O] (``dtype='fp32'``) or int8 with ``scales`` (``dtype='int8'``).  ``group`` selects the
    process group whose ranks hold the other shards; None or a single rank means the layer is not sharded.
    """

    def __init__(self, n_inputs, n_outputs, n_detectors, n_anchors, anchors, tables, scales=None, cmp_eps=0.0,
                 backward_group_size=32, int_rescaler=0.001, group=None, device="cuda:0", dequant="exact"):
        self.device = torch.device(device)
        self.dequant = {"f32": _native.INT8_DEQUANT_F32, "exact": _native.INT8_DEQUANT_EXACT}[dequant]
        self.I, self.O, self.Nt, self.Nc = n_inputs, n_outputs, n_detectors, n_anchors
        self.anchors = anchors.to(self.device, torch.int32).reshape(-1).contiguous()
        self.int8 = tables.dtype == torch.int8
        self.tables = tables.to(self.device).reshape(-1).contiguous()
        self.scales = None if scales is None else scales.to(self.device, torch.float32).contiguous()
        if self.int8:
            assert self.scales is not None and self.scales.numel() == n_detectors
            assert n_outputs % 4 == 0, "int8 tables need n_outputs to be a multiple of 4"
        assert self.tables.numel() == n_detectors * (1 << n_anchors) * n_outputs
        self.group = group
        self.cfg = LayerCfg(n_inputs=n_inputs, n_outputs=n_outputs, n_detectors=n_detectors, n_anchors=n_anchors,
                            seq_len=1, pos_dim=0, forward_group=32, backward_group=backward_group_size,
                            int_mode=0, sliced_product=0, cmp_eps=float(cmp_eps), reserved0=0.0,
                            int_rescaler=float(int_rescaler), lr_meta=1.0)

    @classmethod
    def shard_of(cls, rank, world, n_inputs, n_outputs, n_detectors, n_anchors, anchors, tables, scales=None,
                 backward_group_size=32, **kw):
        """The shard of rank ``rank``: detectors are split evenly; shard boundaries must be multiples of the
        detector block so that fixed-point block sums are the same as in the unsharded layer."""
        assert n_detectors % world == 0, "n_detectors must be divisible by the number of shards"
        per = n_detectors // world
        assert per % backward_group_size == 0 or world == 1, "a shard must hold whole detector blocks"
        T = 1 << n_anchors
        a = anchors.reshape(n_detectors, -1)[rank * per:(rank + 1) * per]
        t = tables.reshape(n_detectors, T * n_outputs)[rank * per:(rank + 1) * per]
        s = None if scales is None else scales[rank * per:(rank + 1) * per]
        return cls(n_inputs, n_outputs, per, n_anchors, a, t, s, backward_group_size=backward_group_size, **kw)

    def partial(self, x):
        """Partial sums of this shard: int32 [B, O] fixed-point accumulators (int8 tables) or fp32 [B, O]."""
        assert x.device == self.device and x.dtype == torch.float32
        x = x.contiguous()
        B = x.shape[0]
        L = _native.lib()
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        idx = torch.empty(B * self.Nt, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            if self.int8:
                acc = torch.zeros(B * self.O, dtype=torch.int32, device=self.device)
                rc = L.lutb_infer_int8_accumulate(ctypes.byref(self.cfg), B, _ptr(self.tables), _ptr(self.scales),
                                                  _ptr(x.view(-1)), _ptr(self.anchors), _ptr(acc), _ptr(idx), self.dequant,
                                                  stream)
            else:
                acc = torch.zeros(B * self.O, dtype=torch.float32, device=self.device)
                rc = L.lutb_nonseq_fc_forward(ctypes.byref(self.cfg), B, _ptr(self.tables), _ptr(x.view(-1)),
                                              _ptr(self.anchors), _ptr(acc), _ptr(idx), None, None, stream)
        _native.check(rc)
        self.last_indices = idx.view(B, self.Nt)
        return acc.view(B, self.O)

    def finish(self, acc):
        """int32 accumulators -> fp32 outputs (in place reinterpretation); fp32 partial sums pass through."""
        if not self.int8:
            return acc
        out = acc.view(torch.float32)
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        with torch.cuda.device(self.device):
            _native.check(_native.lib().lutb_fixed_to_float(_ptr(out), out.numel(), self.cfg.int_rescaler, stream))
        return out

    def __call__(self, x):
        acc = self.partial(x)
        if self.group is not None and dist.get_world_size(self.group) > 1:
            dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=self.group)
        return self.finish(acc)
