"""Data-parallel glue for LUT models: one process per GPU, identical replicas, batch split per rank.

The reference is single-process; this module adds the one exchange step data parallelism needs: table
gradients (and positional-embedding gradients) are sums over the batch, so after every backward the ranks
all-reduce them (NCCL over NVLink on GPUs; any torch.distributed backend works, gloo is used by the CPU
tests).  Forward outputs and input gradients are per-sample and need no communication.

Replicas must be built from the same seeds: anchors are structure, not parameters, and are never
synchronised afterwards; ``broadcast_structure`` copies rank 0's anchors and parameters once at start-up.
"""
import torch
import torch.distributed as dist


def _buckets(tensors, bucket_bytes):
    bucket, size = [], 0
    for t in tensors:
        nbytes = t.numel() * t.element_size()
        if bucket and size + nbytes > bucket_bytes:
            yield bucket
            bucket, size = [], 0
        bucket.append(t)
        size += nbytes
    if bucket:
        yield bucket


def allreduce_gradients(params, group=None, average=False, bucket_bytes=256 << 20):
    """Sum (or average) the dense ``.grad`` of every parameter over the ranks, in place.

    Large gradients (a table's dW is as large as the table) are reduced in place one by one; small ones are
    packed into flat buckets first so that the collective's launch latency is paid once per bucket.
    Sparse gradients are densified per parameter before the reduction.
    """
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    world = dist.get_world_size(group)
    grads = []
    for p in params:
        if p.grad is None:
            continue
        if p.grad.is_sparse:
            p.grad = p.grad.to_dense()
        grads.append(p.grad)
    small_limit = 4 << 20
    large = [g for g in grads if g.numel() * g.element_size() >= small_limit]
    small = [g for g in grads if g.numel() * g.element_size() < small_limit]
    for g in large:
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)
        if average:
            g.div_(world)
    for bucket in _buckets(small, bucket_bytes):
        flat = torch.cat([g.reshape(-1) for g in bucket])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat.div_(world)
        offset = 0
        for g in bucket:
            g.copy_(flat[offset:offset + g.numel()].view_as(g))
            offset += g.numel()


def broadcast_structure(module, src=0, group=None):
    """Make every rank's replica identical to rank ``src``'s: parameters and buffers (anchors included)."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    for t in list(module.parameters()) + list(module.buffers()):
        dist.broadcast(t.data, src=src, group=group)


def shard_batch(n, rank, world):
    """[begin, end) of the contiguous slice of an ``n``-sample batch owned by ``rank``."""
    per = (n + world - 1) // world
    return min(n, rank * per), min(n, (rank + 1) * per)


class OverlappedGradientSync:
    """All-reduces each parameter's gradient as soon as autograd has produced it, on the collective's own
    stream, so that the exchange of the last layers' table gradients overlaps the backward pass of the earlier
    layers (the tables of the last layer finish first).  Call ``wait()`` before the optimiser step.

    Only dense gradients are handled; parameters whose layer uses the Internal policy have no gradient and are
    skipped (their update happens inside the backward kernel and would need reduce-then-apply instead).
    """

    def __init__(self, params, group=None, average=True):
        self.average = average
        self.handles = []
        self.enabled = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if self.enabled else 1
        self._hooks = []
        self._nccl = self.enabled and dist.get_backend(group) == "nccl"
        if self._nccl and group is None:
            # The backward kernels keep every SM busy; on a high-priority stream the collective's blocks are
            # scheduled as soon as any block of the running kernel retires instead of after its last one.
            opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
            group = dist.new_group(backend="nccl", pg_options=opts)
        self.group = group
        if self.enabled:
            for p in params:
                if p.requires_grad:
                    self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))

    def _on_grad(self, p):
        g = p.grad
        if g is None:
            return
        if g.is_sparse:
            p.grad = g = g.to_dense()
        op = dist.ReduceOp.SUM
        if self.average:
            if self._nccl:
                op = dist.ReduceOp.AVG  # averaged inside the collective: no extra pass over the gradient
            else:
                g.div_(self.world)
        self.handles.append((p, dist.all_reduce(g, op=op, group=self.group, async_op=True)))

    def wait(self):
        for _, h in self.handles:
            h.wait()
        self.handles = []

    def wait_each(self):
        """Yields the parameters in the order their gradients were produced, each once its exchange has finished:
        an update applied per parameter overlaps the exchanges that are still in flight."""
        handles, self.handles = self.handles, []
        for p, h in handles:
            h.wait()
            yield p

    def remove(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []


def exchange_sparse_gradients(params, group=None, average=False):
    """Exchange of ``GradientType.Sparse`` table gradients: every rank contributes the (cell, value) lists of the
    cells its shard of the batch touched and receives everybody's, so the payload is the touched cells instead of
    the whole table (a concatenation-mode table has 2^(2Nc+Npe) rows of which a step touches a few).

    One all-gather of the list lengths for all parameters, then per parameter one all-gather of the cell numbers and
    one of the values, padded to the longest list.  The received lists are concatenated into an uncoalesced sparse
    gradient: cells touched by several ranks appear once per rank and are summed when the optimiser coalesces (or
    densifies) the gradient, which is the same sum a dense all-reduce would have produced.  Parameters whose
    gradient is dense or missing on every rank are left alone.
    """
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    world = dist.get_world_size(group)
    params = list(params)
    if not params:
        return
    device = params[0].device
    # Every rank must issue the same collectives.  A rank whose shard touched nothing has no gradient at all for a
    # table, so the list lengths are exchanged for every parameter first: -1 = no gradient here, -2 = dense gradient
    # here; a parameter takes part when any rank holds a sparse gradient for it, ranks without one send an empty list.
    grads, lengths = [], []
    for p in params:
        g = p.grad
        if g is None:
            lengths.append(-1)
        elif not g.is_sparse:
            lengths.append(-2)
        else:
            g = g if g.is_coalesced() else g.coalesce()
            lengths.append(g._nnz())
        grads.append(g)
    counts = torch.tensor(lengths, dtype=torch.int64, device=device)
    all_counts = [torch.empty_like(counts) for _ in range(world)]
    dist.all_gather(all_counts, counts, group=group)
    all_counts = torch.stack(all_counts).cpu()  # [world][n_params]
    for n, (p, g) in enumerate(zip(params, grads)):
        column = all_counts[:, n]
        if int(column.max()) < 0:
            continue  # nobody holds a sparse gradient for this parameter
        if int((column == -2).sum()) > 0:
            raise ValueError(f"parameter {n}: dense gradient on one rank, sparse on another")
        longest = int(column.max())
        if longest == 0:
            continue
        mine = 0 if g is None else g._nnz()
        dtype = p.dtype if g is None else g.dtype
        cells = torch.zeros(longest, dtype=torch.int64, device=device)
        values = torch.zeros(longest, dtype=dtype, device=device)
        if mine:
            cells[:mine] = g.indices()[0]
            values[:mine] = g.values()
        got_cells = [torch.empty_like(cells) for _ in range(world)]
        got_values = [torch.empty_like(values) for _ in range(world)]
        dist.all_gather(got_cells, cells, group=group)
        dist.all_gather(got_values, values, group=group)
        keep = [max(int(column[r]), 0) for r in range(world)]
        cells = torch.cat([c[:k] for c, k in zip(got_cells, keep)])
        values = torch.cat([v[:k] for v, k in zip(got_values, keep)])
        if average:
            values = values / world
        p.grad = torch.sparse_coo_tensor(cells.unsqueeze(0), values, size=p.shape, device=device,
                                         check_invariants=False, is_coalesced=False)


def average_internal_policy_weights(module, group=None):
    """Data parallelism for tables trained with ``GradientType.Internal``: the backward kernel has already applied
    ``W_r = W - lr * dW_r`` on every rank with that rank's shard gradient, so averaging the tables over the ranks
    gives ``W - lr * mean_r(dW_r)``, the update a reduce-then-apply with the averaged gradient would have made
    (equal up to fp32 rounding of the per-rank updates).  Call once per step, after backward; positional embeddings
    of such layers are ordinary parameters with ordinary gradients and are not touched here.
    """
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return 0
    from .lut_layer import GradientType, LUTLayerBasic

    world = dist.get_world_size(group)
    nccl = dist.get_backend(group) == "nccl"
    done = 0
    for layer in module.modules():
        if isinstance(layer, LUTLayerBasic) and layer._weights_gradient_policy.type == GradientType.Internal:
            w = layer._weights.data
            if nccl:
                dist.all_reduce(w, op=dist.ReduceOp.AVG, group=group)
            else:
                dist.all_reduce(w, op=dist.ReduceOp.SUM, group=group)
                w.div_(world)
            done += 1
    return done
