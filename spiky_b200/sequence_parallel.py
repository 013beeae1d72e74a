"""Query-sharded execution of a concatenation-mode attention LUT layer over the ranks of a process group.

The reference is single-process.  Its concatenation-mode layer (src/spiky/lut/LUTLayer.py:677-777; kernels
fill_outputs_fully_connected_seq_logic, spiky_cuda/lut/lut_runtime_kernels_logic.proto:1807-1905, and
propagate_through_detectors_seq_fc_logic / gather_w_gradients_seq_fc_cpu_logic, :3629-4044) sums, for every query
token j, the table rows selected by the pairs (i, j) with i < j; a row is addressed by the table index of token j, the
table index of token i and the positional index of the distance.  The per-token indices depend on one token each, the
pair work grows with the square of the context: so the tokens are split over the ranks,

    rank r owns the tokens [r * S / G, (r + 1) * S / G) of every sequence,

each rank computes the indices of its own tokens, ONE all-gather makes the indices (int32 [B, S, Nt], plus the
minimum-margin deltas and pairs in training) known everywhere, and each rank runs the pair stage for its own QUERY
tokens only.  Outputs are disjoint per query, so the forward needs no reduction.  Backward: a pair (i, j) sends
gradient to token j and to token i < j, which may live on another rank, and to the table row and the positional
embedding it used: the partial input gradients are reduce-scattered back to the owners of the tokens, the partial
table and positional gradients are summed over the ranks (all-reduce).  The arithmetic is the unsharded layer's up to
fp32 summation order; fixed-point (int32) layers are not supported (the range backward needs fp32 accumulators).

Causal pairs make the late ranks' share larger (rank r holds the queries with about (r + 1/2) * S / G keys each); a
balanced assignment would interleave blocks of queries.  Contiguous blocks are kept because they match how a long
sequence is naturally split.
"""
import torch
import torch.distributed as dist


def _world(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def _gather_tokens(local, group, world):
    """[B, S_local, ...] on every rank -> [B, world * S_local, ...] (token blocks in rank order)."""
    if world == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=1).contiguous()


def _reduce_scatter_tokens(full, group, world, rank, s_local):
    """Sum of [B, S, ...] over the ranks, each rank keeping its own token block [B, S_local, ...]."""
    if world == 1:
        return full
    parts = [full[:, r * s_local:(r + 1) * s_local].contiguous() for r in range(world)]
    out = torch.empty_like(parts[rank])
    if dist.get_backend(group) == "nccl":
        dist.reduce_scatter(out, parts, op=dist.ReduceOp.SUM, group=group)
    else:
        # gloo has no reduce_scatter: reduce every block to its owner
        for r, p in enumerate(parts):
            dist.reduce(p, dst=dist.get_global_rank(group, r) if group is not None else r, op=dist.ReduceOp.SUM,
                        group=group)
        out = parts[rank]
    return out


class _QueryShardedConcatFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, weights, pos_embeddings, wrapper):
        layer, group = wrapper.layer, wrapper.group
        world, rank = _world(group)
        dm = layer._lut_dm
        B, s_local = x_local.shape[0], x_local.shape[1]
        S, Nt, dev = layer._sequence_length, layer._n_detectors, x_local.device
        assert s_local * world == S, "every rank holds S / world tokens of each sequence"
        train = layer.training
        cmp_eps = layer._shared_context._cmp_eps
        rows = B * s_local
        idx = torch.empty(rows * Nt, dtype=torch.int32, device=dev)
        md = torch.empty(rows * Nt, dtype=torch.float32, device=dev) if train else None
        mk = torch.empty(rows * Nt, dtype=torch.int32, device=dev) if train else None
        dm.check_detectors(rows, x_local.contiguous().view(-1), layer._detector_anchors, idx, cmp_eps, md, mk)
        idx = _gather_tokens(idx.view(B, s_local, Nt), group, world)
        if train:
            md = _gather_tokens(md.view(B, s_local, Nt), group, world)
            mk = _gather_tokens(mk.view(B, s_local, Nt), group, world)
        pidx = pmd = pmk = None
        if layer._positional_dim > 0:
            pe = pos_embeddings.detach().contiguous().view(-1)
            pidx = torch.empty((S - 1) * Nt, dtype=torch.int32, device=dev)
            if train:
                pmd = torch.empty((S - 1) * Nt, dtype=torch.float32, device=dev)
                pmk = torch.empty((S - 1) * Nt, dtype=torch.int32, device=dev)
            dm.check_positional(pe, pidx, cmp_eps, pmd, pmk)
        j0, j1 = rank * s_local, (rank + 1) * s_local
        y = torch.zeros(B * S * layer._n_outputs, dtype=torch.float32, device=dev)
        dm.concat_pairs_forward(weights.detach(), B, idx.view(-1), pidx, y, j0, j1)
        ctx.wrapper = wrapper
        ctx.range = (j0, j1, world, rank)
        ctx.shape = (B, S, s_local)
        ctx.state = (idx, md, mk, pidx, pmd, pmk)
        ctx.pe_shape = None if pos_embeddings is None else pos_embeddings.shape
        ctx.save_for_backward(weights)
        return y.view((B, S) + tuple(layer.output_shape()))[:, j0:j1].contiguous()

    @staticmethod
    def backward(ctx, grad_local):
        wrapper = ctx.wrapper
        layer, group = wrapper.layer, wrapper.group
        (weights,) = ctx.saved_tensors
        j0, j1, world, rank = ctx.range
        B, S, s_local = ctx.shape
        idx, md, mk, pidx, pmd, pmk = ctx.state
        dev, Nt, npe = grad_local.device, layer._n_detectors, layer._positional_dim
        dm = layer._lut_dm
        dY = torch.zeros((B, S) + tuple(grad_local.shape[2:]), dtype=torch.float32, device=dev)
        dY[:, j0:j1] = grad_local
        dX = torch.zeros(B * S * layer._n_inputs, dtype=torch.float32, device=dev)
        dW = torch.zeros_like(weights)
        dPE = torch.zeros((S - 1) * Nt * npe, dtype=torch.float32, device=dev) if npe > 0 else None
        dm.concat_pairs_backward(weights.detach(), B, dY.view(-1), layer._detector_anchors, idx.view(-1), md.view(-1),
                                 mk.view(-1), dX, -1.0, pidx, pmd, pmk, dPE, dW, j0, j1)
        dX = _reduce_scatter_tokens(dX.view(B, S, layer._n_inputs), group, world, rank, s_local)
        if world > 1:
            dist.all_reduce(dW, op=dist.ReduceOp.SUM, group=group)
            if dPE is not None:
                dist.all_reduce(dPE, op=dist.ReduceOp.SUM, group=group)
        if dPE is not None:
            dPE = dPE.view(ctx.pe_shape)
        return dX.view((B, s_local) + tuple(layer.input_shape())), dW, dPE, None


class QueryShardedConcatAttention(torch.nn.Module):
    """Wraps a concatenation-mode, fully connected sequence ``LUTLayer``: ``forward(x_local)`` takes this rank's token
    block ``[B, S / G, n_inputs]`` and returns the layer's output for the same tokens ``[B, S / G, n_outputs]``.
    The wrapped layer's parameters (tables, positional embeddings) receive complete gradients on every rank, so the
    replicas stay identical under any optimiser; Dense gradient policy only."""

    def __init__(self, layer, group=None):
        super().__init__()
        from .lut_layer import GradientType

        if not layer._concatenation_product or layer._sequence_length <= 1 or not layer._is_fully_connected:
            raise ValueError("query sharding is built for fully connected concatenation-mode sequence layers")
        if layer._lut_dm.get_summations_data_type() != "float32":
            raise ValueError("query sharding needs fp32 accumulators")
        if layer._weights_gradient_policy.type != GradientType.Dense or layer._weights_gradient_policy.normalized:
            raise ValueError("query sharding returns plain dense table gradients (GradientType.Dense, not normalized)")
        self.layer = layer
        self.group = group

    def forward(self, x_local):
        layer = self.layer
        pos = layer._prepare_positional_embeddings() if layer._positional_dim > 0 else None
        return _QueryShardedConcatFn.apply(x_local, layer._weights, pos, self)
