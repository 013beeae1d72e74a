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
        self.paused = False   # True: gradients stay local (used to time a step without its exchange)
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
        if self.paused:
            self.handles.append((p, None))
            return
        op = dist.ReduceOp.SUM
        if self.average:
            if self._nccl:
                op = dist.ReduceOp.AVG  # averaged inside the collective: no extra pass over the gradient
            else:
                g.div_(self.world)
        self.handles.append((p, dist.all_reduce(g, op=op, group=self.group, async_op=True)))

    def wait(self):
        for _, h in self.handles:
            if h is not None:
                h.wait()
        self.handles = []

    def wait_each(self):
        """Yields the parameters in the order their gradients were produced, each once its exchange has finished:
        an update applied per parameter overlaps the exchanges that are still in flight."""
        handles, self.handles = self.handles, []
        for p, h in handles:
            if h is not None:
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


def _all_gather_uneven(views, rank, group):
    """All-gather where ``views[r]`` (rank r's contribution, already in place on rank r) differ in size."""
    if dist.get_backend(group) == "nccl":
        # unequal sizes: torch issues one grouped broadcast per rank
        return [dist.all_gather(list(views), views[rank], group=group, async_op=True)]
    works = []
    for r, v in enumerate(views):
        if v.numel():
            works.append(dist.broadcast(v, src=dist.get_global_rank(group, r) if group is not None else r, group=group,
                                        async_op=True))
    return works


class ShardedTableUpdate:
    """Data-parallel SGD for sparse non-sequence LUT layers without exchanging dense table gradients.

    The table gradient of such a layer is a function of the table indices and the output gradients alone:
    ``dW[row(t, idx[b, t]) + p] += dY[b, target(p)]``.  Per step and layer every rank therefore all-gathers its
    ``idx`` (as uint8 / int16 when the tables have at most 256 / 65536 rows) and ``dY`` - for the three layers of the
    sparse conv-net configuration 12 MB per rank against 382 MB of dense gradients - applies the SGD update of the
    *whole* batch to its own share of the detectors in place (``lutb_nonseq_sparse_table_grad`` over a chunk range),
    and all-gathers the updated shares.  Bytes received per rank and step: ``(G-1) * (idx + dY)`` plus ``(G-1)/G`` of
    the tables, against ``2 * (G-1)/G`` of the tables for a ring all-reduce of the gradients; the optimiser pass
    and the dense gradient buffers disappear.  The result is plain SGD with the gradient summed (``average=False``)
    or averaged (default) over the global batch: what all-reduce + ``torch.optim.SGD`` computes, up to fp32
    summation order.

    Use: ``sync = ShardedTableUpdate(layers, lr)`` once; run forward / backward as usual (each layer's backward calls
    back into this object; the layer's ``_weights`` gets no ``.grad``); call ``sync.wait()`` before the next forward.
    The exchange and the update of a layer run on a side stream and overlap the backward pass of the layers below.
    """

    def __init__(self, layers, lr, group=None, average=True, weight_gather="padded"):
        from .lut_layer import GradientType, LUTLayerBasic

        # how the updated shares travel: "padded" = one equal-size all-gather through a staging buffer (shares are
        # padded to the largest), "uneven" = all-gather on views of the tables (grouped broadcasts under NCCL)
        assert weight_gather in ("padded", "uneven")
        self.weight_gather = weight_gather
        self.group = group
        self.lr = lr
        self.enabled = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if self.enabled else 1
        self.rank = dist.get_rank(group) if self.enabled else 0
        self.scale_div = self.world if average else 1
        self.layers = list(layers)
        self._pending = []
        self._side = None
        self._plans = {}
        self._bufs = {}
        for layer in self.layers:
            if not isinstance(layer, LUTLayerBasic) or layer._is_fully_connected or layer._sequence_length != 1:
                raise ValueError("ShardedTableUpdate handles non-sequence layers with sparse lookup connectivity")
            if layer._lut_dm.get_summations_data_type() != "float32":
                raise ValueError("ShardedTableUpdate needs fp32 accumulators")
            if layer._weights_gradient_policy.type == GradientType.Internal:
                raise ValueError("the layer already updates its tables in place (Internal policy)")
            index = layer._lut_dm._sparse
            if index.max_count > 32:
                raise ValueError("rows longer than 32 synapses are not supported by the ranged table-gradient pass")
            cuts = index.shard_chunks(self.world)
            bounds = index.chunk_weight_bounds()
            rows = index.rows_per_detector
            self._plans[id(layer)] = dict(
                cuts=cuts, wcuts=[int(bounds[c]) for c in cuts],
                idx_dtype=torch.uint8 if rows <= 256 else (torch.int16 if rows <= 65536 else torch.int32))
            layer._table_update_hook = self._on_backward

    def _learning_rate(self):
        return float(self.lr() if callable(self.lr) else self.lr)

    # the arithmetic of one share; replaced by the CPU tests, which have no kernels to run
    def _apply(self, layer, batch, dY_all, idx_all, scale, c0, c1):
        layer._lut_dm.table_gradient(batch, dY_all, idx_all, layer._weights.detach(), scale, c0, c1)

    def _on_backward(self, layer, idx, dY, batch):
        plan = self._plans[id(layer)]
        W, G = self.world, self.group
        if W == 1:
            # nothing to exchange: in-place SGD on all chunks, on the current stream
            self._apply(layer, batch, dY, idx, -self._learning_rate() / self.scale_div, 0, plan["cuts"][1])
            return
        on_gpu = idx.is_cuda
        if on_gpu and self._side is None:
            self._side = torch.cuda.Stream(device=idx.device)
        main = torch.cuda.current_stream(idx.device) if on_gpu else None
        if on_gpu:
            self._side.wait_stream(main)  # input gradient of this layer (it reads the tables) and dY are ordered before
        ctx = torch.cuda.stream(self._side) if on_gpu else _NullContext()
        with ctx:
            buf = self._buffers(layer, plan, idx, dY)
            small, idx_all, dY_all = buf["small"], buf["idx_all"], buf["dY_all"]
            small.copy_(idx)   # narrowing copy: the indices travel as uint8 / int16 when the table allows it
            w1 = dist.all_gather_into_tensor(idx_all, small, group=G, async_op=True)
            w2 = dist.all_gather_into_tensor(dY_all, dY.contiguous(), group=G, async_op=True)
            w1.wait()  # orders the update below (same stream) after the collectives; the host does not block
            w2.wait()
            if on_gpu:
                # tensors made on the main stream, used on the side stream
                idx.record_stream(self._side)
                dY.record_stream(self._side)
            c0, c1 = plan["cuts"][self.rank], plan["cuts"][self.rank + 1]
            self._apply(layer, W * batch, dY_all, idx_all, -self._learning_rate() / self.scale_div, c0, c1)
            w = layer._weights.detach()
            views = [w[plan["wcuts"][r]:plan["wcuts"][r + 1]] for r in range(W)]
            if self.weight_gather == "uneven":
                self._pending.extend(_all_gather_uneven(views, self.rank, G))
            else:
                longest = max(v.numel() for v in views)
                lo = plan["wcuts"][self.rank]
                if lo + longest <= w.numel():
                    # the share is sent in place, padded with whatever follows it in the table (the receivers keep
                    # only the share's own length)
                    send = w[lo:lo + longest]
                else:
                    send = buf["send"]
                    send[:views[self.rank].numel()] = views[self.rank]
                recv = buf["recv"]
                work = dist.all_gather_into_tensor(recv, send, group=G, async_op=True)
                work.wait()  # orders the copies below (same stream) after the collective; the host does not block
                for r, v in enumerate(views):
                    if r != self.rank and v.numel():
                        v.copy_(recv[r * longest:r * longest + v.numel()])

    def _buffers(self, layer, plan, idx, dY):
        """Exchange buffers of a layer, allocated once per batch size (on the stream that uses them)."""
        key = (id(layer), idx.numel(), dY.numel())
        buf = self._bufs.get(key)
        if buf is None:
            W = self.world
            w = layer._weights
            longest = max(plan["wcuts"][r + 1] - plan["wcuts"][r] for r in range(W))
            buf = dict(small=torch.empty(idx.numel(), dtype=plan["idx_dtype"], device=idx.device),
                       idx_all=torch.empty(W * idx.numel(), dtype=plan["idx_dtype"], device=idx.device),
                       dY_all=torch.empty(W * dY.numel(), dtype=dY.dtype, device=dY.device))
            if self.weight_gather != "uneven":
                buf["send"] = torch.empty(longest, dtype=w.dtype, device=w.device)
                buf["recv"] = torch.empty(W * longest, dtype=w.dtype, device=w.device)
            self._bufs[key] = buf
        return buf

    def wait(self):
        """Makes the current stream (and, for CPU process groups, the host) wait for every outstanding exchange."""
        for w in self._pending:
            w.wait()
        self._pending = []
        if self._side is not None:
            torch.cuda.current_stream(self._side.device).wait_stream(self._side)

    def remove(self):
        for layer in self.layers:
            if getattr(layer, "_table_update_hook", None) is not None:
                del layer._table_update_hook


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False
