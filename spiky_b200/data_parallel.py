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

    ``transport="peer"`` (one node, CUDA, ``batch_size`` given): nothing goes through collectives.  The tables and the
    gathered arrays live in buffers every rank has mapped; the indices of a layer leave for the other ranks right
    after its forward pass, its output gradients after its backward pass (``lutb_peer_broadcast``: plain stores into
    the other ranks' memory), the ranks meet through flags in peer memory (``lutb_peer_barrier``), each updates its
    share and stores it into every rank's tables.  Every layer has its own stream and barrier channel; the next
    forward pass of a layer waits for that layer's exchange only (``wait()`` is then optional).  The launches carry no
    per-step arguments, so the whole step, exchange included, can be captured into a CUDA graph and replayed.
    """

    def __init__(self, layers, lr, group=None, average=True, weight_gather="padded", transport="collectives",
                 batch_size=None, barrier="flags", share_copies="stores"):
        from .lut_layer import GradientType, LUTLayerBasic

        # how the updated shares travel: "padded" = one equal-size all-gather through a staging buffer (shares are
        # padded to the largest), "uneven" = all-gather on views of the tables (grouped broadcasts under NCCL)
        assert weight_gather in ("padded", "uneven")
        self.weight_gather = weight_gather
        # transport "collectives": all-gathers of the process group.  "peer" (one node, CUDA): the tables and the
        # gathered (index, output gradient) arrays live in buffers every rank has mapped; a rank stores its pairs into
        # every rank's arrays and, after its update, its share of the tables into every rank's tables
        # (lutb_peer_broadcast: plain posted stores over NVLink, no staging, no collective kernels), with
        # lutb_peer_barrier between the phases.  Needs the per-rank batch size up front (the arrays are allocated
        # once, collectively).
        assert transport in ("collectives", "peer") and barrier in ("flags", "collective")
        self.transport = transport
        self.barrier = barrier
        # peer transport, how the updated shares travel: "stores" = lutb_peer_broadcast (one kernel stores into all
        # ranks), "engine" = one asynchronous copy per rank on the copy engines (no SM used; measured no faster: 0.98
        # against 0.96 ms per step at two GPUs)
        assert share_copies in ("stores", "engine")
        self.share_copies = share_copies
        self.batch_size = batch_size
        self._space = None
        self._dirty = False
        # True: the pairs and the table shares still travel but the update itself is skipped (tables unchanged); for
        # timing the exchange alone
        self.exchange_only = False
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
        if self.transport == "peer" and self.world > 1:
            self._setup_peer()

    def _setup_peer(self):
        if not self.batch_size:
            raise ValueError("transport='peer' needs batch_size (samples per rank and step)")
        device = self.layers[0]._weights.device
        if device.type != "cuda":
            raise ValueError("transport='peer' needs the tables on a CUDA device")
        W, B = self.world, int(self.batch_size)
        sizes = {}
        for li, layer in enumerate(self.layers):
            plan = self._plans[id(layer)]
            item = torch.empty(0, dtype=plan["idx_dtype"]).element_size()
            sizes[f"w{li}"] = 4 * ((layer._weights.numel() + 3) // 4 * 4)
            sizes[f"i{li}"] = W * B * layer.n_detectors() * item
            sizes[f"d{li}"] = W * B * layer.n_outputs() * 4
        self._space = _PeerSpace(sizes, device, self.group, "ShardedTableUpdate", channels=len(self.layers))
        for li, layer in enumerate(self.layers):
            plan = self._plans[id(layer)]
            shared = self._space.tensor(f"w{li}", torch.float32, layer._weights.numel())
            shared.copy_(layer._weights.detach())
            layer._weights.data = shared
            plan["li"] = li
            plan["idx_all"] = self._space.tensor(f"i{li}", plan["idx_dtype"])
            plan["dY_all"] = self._space.tensor(f"d{li}", torch.float32)
            # The exchange of a layer runs on the layer's own stream and ends with its own barrier and event: the
            # next forward pass of THAT layer waits for the event (forward pre-hook), nothing else does.  The upper
            # layers' exchanges, which start first and move most bytes, so overlap the rest of the backward pass and
            # the next step's forward pass of the layers below them; only the bottom layer's exchange is exposed.
            plan["stream"] = torch.cuda.Stream(device=device)
            plan["done"] = None
            plan["hook"] = layer.register_forward_pre_hook(lambda module, inputs: self.wait_layer(module))
            # the indices of a layer are known after its forward pass: they leave for the other ranks then (four fifths
            # of the pair bytes), off the path between the layer's backward pass and its update
            plan["idx_sent"] = False
            layer._table_forward_hook = self._on_forward_peer
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)  # every rank's tables are in place before anyone stores into them

    def _send_indices(self, layer, idx, stream):
        """Narrows this rank's table indices into its slot of the gathered array and stores the slot into every other
        rank's array (on `stream`, inside the caller's stream context)."""
        from . import _native
        plan, space = self._plans[id(layer)], self._space
        li, n_i = plan["li"], idx.numel()
        own = plan["idx_all"][self.rank * n_i:(self.rank + 1) * n_i]
        own.copy_(idx)   # narrowing copy: the indices travel as uint8 / int16 when the table allows it
        _native.peer_broadcast(space.others(f"i{li}"), self.rank * n_i * own.element_size(), own.data_ptr(),
                               n_i * own.element_size(), stream.cuda_stream)

    def _on_forward_peer(self, layer, idx, batch):
        plan = self._plans[id(layer)]
        if batch != self.batch_size:
            raise ValueError(f"transport='peer' was set up for {self.batch_size} samples per rank, got {batch}")
        # (the layer's forward pre-hook has waited for the previous step's exchange of this layer: every rank is done
        # reading the gathered indices of that step)
        stream = plan["stream"]
        stream.wait_stream(torch.cuda.current_stream(idx.device))
        with torch.cuda.stream(stream):
            self._send_indices(layer, idx, stream)
        plan["idx_sent"] = True
        plan["idx_ref"] = idx   # referenced until the layer's stream has read it (its backward pass comes later)

    def _on_backward_peer(self, layer, idx, dY, batch):
        from . import _native
        plan, space = self._plans[id(layer)], self._space
        W, li = self.world, plan["li"]
        if batch != self.batch_size:
            raise ValueError(f"transport='peer' was set up for {self.batch_size} samples per rank, got {batch}")
        main = torch.cuda.current_stream(idx.device)
        stream = plan["stream"]
        stream.wait_stream(main)  # the input gradient of this layer (it reads the tables) and dY are ordered before
        with torch.cuda.stream(stream):
            side = stream.cuda_stream
            idx_all, dY_all = plan["idx_all"], plan["dY_all"]
            n_d = dY.numel()
            if not plan["idx_sent"]:   # (a backward pass whose forward pass ran without the hook, e.g. exchange timing)
                self._send_indices(layer, idx, stream)
            plan["idx_sent"] = False
            dYc = dY.contiguous()
            _native.peer_broadcast(space.ptrs[f"d{li}"], self.rank * n_d * 4, dYc.data_ptr(), n_d * 4, side)
            # the layer's stream reads these after the main stream has moved on: they stay referenced until the next
            # backward pass of the layer (by then its forward pass has waited for this exchange)
            plan["last"] = (idx, dYc)
            # every rank's pairs have landed everywhere, and no rank still reads these tables
            space.barrier(stream, self.barrier, li)
            c0, c1 = plan["cuts"][self.rank], plan["cuts"][self.rank + 1]
            if not self.exchange_only:
                self._apply(layer, W * batch, dY_all, idx_all, -self._learning_rate() / self.scale_div, c0, c1)
            lo, hi = plan["wcuts"][self.rank], plan["wcuts"][self.rank + 1]
            if hi > lo and self.share_copies == "engine":
                # one copy per peer on the copy engines: no SM is taken from the kernels beside it
                for r in range(W):
                    if r != self.rank:
                        _native.peer_copy(space.ptrs[f"w{li}"][r] + lo * 4, space.ptrs[f"w{li}"][self.rank] + lo * 4,
                                          (hi - lo) * 4, side)
            elif hi > lo:
                _native.peer_broadcast(space.others(f"w{li}"), lo * 4, space.ptrs[f"w{li}"][self.rank] + lo * 4,
                                       (hi - lo) * 4, side)
            # every rank's share of this layer has landed in this rank's tables, nobody still reads the gathered pairs
            space.barrier(stream, self.barrier, li)
            plan["done"] = torch.cuda.Event()
            plan["done"].record(stream)

    def wait_layer(self, layer):
        """Makes the current stream wait for the outstanding exchange of one layer (peer transport)."""
        plan = self._plans.get(id(layer))
        if plan is not None and plan.get("done") is not None:
            torch.cuda.current_stream(layer._weights.device).wait_event(plan["done"])
            plan["done"] = None

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
        if self._space is not None:
            return self._on_backward_peer(layer, idx, dY, batch)
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
        if self._space is not None:
            for layer in self.layers:
                self.wait_layer(layer)
        if self._side is not None:
            torch.cuda.current_stream(self._side.device).wait_stream(self._side)

    def remove(self):
        """Detaches from the layers; with the peer transport also moves the tables back into ordinary device memory
        and releases the shared buffers (collective)."""
        if self._space is not None:
            self.wait()
        for layer in self.layers:
            if getattr(layer, "_table_update_hook", None) is not None:
                del layer._table_update_hook
        if self._space is not None:
            device = self._space.device
            for layer in self.layers:
                layer._weights.data = layer._weights.data.clone()
            for plan in self._plans.values():
                plan.pop("idx_all", None)
                plan.pop("dY_all", None)
                plan.pop("last", None)
                plan.pop("idx_ref", None)
                plan.pop("hook").remove()
            for layer in self.layers:
                if getattr(layer, "_table_forward_hook", None) is not None:
                    del layer._table_forward_hook
            torch.cuda.synchronize(device)
            dist.barrier(group=self.group)  # nobody still reads a buffer that is about to go
            self._space.release()
            self._space = None


class _DeviceSpan:
    """A span of device memory as an object ``torch.as_tensor`` can wrap without copying."""

    def __init__(self, ptr, numel):
        self.__cuda_array_interface__ = {"shape": (int(numel),), "typestr": "<f4", "data": (int(ptr), False),
                                         "strides": None, "version": 2}


class _PeerSpace:
    """Named device buffers of this rank that every other rank of the group (same node) has mapped, plus the flags of
    the stream-ordered barrier between them.  ``sizes``: ``{name: bytes}``, the same on every rank.  Construction and
    ``release`` are collective.  A rank that fails to allocate or to map tells the others through the same
    collectives, so that all ranks raise ``RuntimeError`` together instead of one leaving the others waiting."""

    def __init__(self, sizes, device, group=None, what="peer memory", channels=1):
        from . import _native

        self._native = _native
        self.group = group
        self.device = device
        self.what = what
        enabled = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if enabled else 1
        self.rank = dist.get_rank(group) if enabled else 0
        if self.world > _native.MAX_PEER_RANKS:
            raise ValueError(f"{what} supports up to {_native.MAX_PEER_RANKS} ranks")
        self.names = list(sizes)
        self.sizes = dict(sizes)
        self._owned, self._mapped = [], []
        # barrier channels: barriers issued on different streams must not share flags (a rank may run them in another
        # order than its peers); every channel has its own flag array and epoch counter
        self.channels = int(channels)
        self._token = None
        own, handles, error = {}, {}, None
        try:
            with torch.cuda.device(device):
                # the barrier's flags: one 64-bit slot per rank, zero before the first epoch
                # per channel: one 64-bit flag per rank, then this rank's own barrier count
                own["_flags"], handles["_flags"] = _native.peer_alloc(16 * _native.MAX_PEER_RANKS * self.channels)
                self._owned.append(own["_flags"])
                torch.as_tensor(_DeviceSpan(own["_flags"], 4 * _native.MAX_PEER_RANKS * self.channels),
                                device=device).zero_()
                for name in self.names:
                    own[name], handles[name] = _native.peer_alloc(max(16, (int(sizes[name]) + 15) // 16 * 16))
                    self._owned.append(own[name])
        except RuntimeError as e:
            error = str(e)
        everyone = self._agree((error, handles), "allocating shareable device memory")
        # ptrs[name][r]: rank r's buffer as this process addresses it
        self.ptrs = {name: [None] * self.world for name in ["_flags"] + self.names}
        error = None
        try:
            with torch.cuda.device(device):
                for r in range(self.world):
                    for name in self.ptrs:
                        if r == self.rank:
                            self.ptrs[name][r] = own[name]
                        else:
                            self.ptrs[name][r] = _native.peer_open(everyone[r][1][name])
                            self._mapped.append(self.ptrs[name][r])
        except RuntimeError as e:
            error = str(e)
        self._agree((error, None), "mapping the other ranks' buffers")   # also: every rank has mapped every buffer
        torch.cuda.synchronize(device)

    def _agree(self, mine, doing):
        everyone = [mine]
        if self.world > 1:
            everyone = [None] * self.world
            dist.all_gather_object(everyone, mine, group=self.group)
        errors = [f"rank {r}: {e[0]}" for r, e in enumerate(everyone) if e[0]]
        if errors:
            self.release()
            raise RuntimeError(f"{self.what}: {doing} failed ({errors[0]})")
        return everyone

    def tensor(self, name, dtype=torch.float32, numel=None):
        """This rank's buffer ``name`` as a flat tensor (no copy)."""
        item = torch.empty(0, dtype=dtype).element_size()
        n = self.sizes[name] // item if numel is None else int(numel)
        assert n * item <= max(16, (self.sizes[name] + 15) // 16 * 16)
        if dtype == torch.float32:
            t = torch.as_tensor(_DeviceSpan(self.ptrs[name][self.rank], n), device=self.device)
        else:
            t = torch.as_tensor(_DeviceSpan(self.ptrs[name][self.rank], (n * item + 3) // 4), device=self.device)
            t = t.view(torch.uint8)[:n * item].view(dtype)
        assert t.data_ptr() == self.ptrs[name][self.rank]
        return t

    def others(self, name):
        """The other ranks' buffers ``name`` (mapped pointers)."""
        return [p for r, p in enumerate(self.ptrs[name]) if r != self.rank]

    def barrier(self, stream, kind="flags", channel=0):
        """Barrier over the ranks on ``stream`` (the host does not block): "flags" = lutb_peer_barrier, a one-warp
        kernel over flags in peer memory whose wait is bounded (a rank that is seconds late is counted by
        lutb_device_wait_errors and not waited for); "collective" = a one-element all-reduce of the process group.
        Every rank issues the barriers of a channel in the same order; channels are independent of each other."""
        if self.world == 1:
            return
        if kind == "flags":
            # epoch 0: the kernel counts the barriers of the channel itself (the launch can be replayed from a graph)
            off = channel * 16 * self._native.MAX_PEER_RANKS
            self._native.peer_barrier(self.rank, [p + off for p in self.ptrs["_flags"]], 0, stream.cuda_stream)
        else:
            if self._token is None:
                self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
            with torch.cuda.stream(stream):
                dist.all_reduce(self._token, group=self.group, async_op=True).wait()

    def release(self):
        """Unmaps the other ranks' buffers, then frees this rank's (collective when there are several ranks)."""
        with torch.cuda.device(self.device):
            for p in self._mapped:
                self._native.peer_close(p)
            if self.world > 1:
                dist.barrier(group=self.group)  # all mappings closed before the owners free
            for p in self._owned:
                self._native.peer_free(p)
        self._mapped, self._owned = [], []


class PeerTableUpdate:
    """Data-parallel SGD for non-sequence LUT layers on one node: gradient reduction, table update and the broadcast
    of the updated tables in ONE kernel over peer memory (``lutb_peer_sgd_update``), instead of an all-reduce of the
    dense gradients followed by an optimiser pass.

    Every rank's tables and dense table gradients live in buffers the other ranks have mapped (CUDA IPC over NVLink).
    The layer's backward writes its table gradient into the rank's buffer; then rank r reads slice r of every rank's
    gradient, applies ``w -= lr / G * sum`` (``average=False``: ``lr * sum``) and stores the new slice into every
    rank's tables.  Per rank ``(G-1)/G`` of the tables cross the links in each direction, at the same time; the
    optimiser pass, the gradient ``.grad`` tensors and NCCL's staging disappear, and because each element is computed
    by one rank the replicas stay bit-identical.  The kernel itself never waits on another rank: a one-element
    all-reduce of the process group before it (every rank's gradient of this layer is complete) and one after the last
    layer (every rank's stores have landed) order it, on a side stream, so the exchange of a layer overlaps the
    backward pass of the layers below it.

    Use: ``sync = PeerTableUpdate(layers, lr)`` once, after the layers are on their device (their ``_weights`` move
    into the shared buffers; ``remove()`` moves them back); run forward / backward as usual (the layers' ``_weights``
    get no ``.grad``); call ``sync.wait()`` before the next forward.  fp32 tables, dense gradient policy, one
    process per GPU, all ranks on one node.
    """

    def __init__(self, layers, lr, group=None, average=True, barrier="flags"):
        from . import _native
        from .lut_layer import GradientType, LUTLayerBasic

        # how the ranks meet before and after the update kernels: "flags" = a one-warp kernel over flags in peer memory
        # (lutb_peer_barrier: a few microseconds; its wait is bounded, a rank that is seconds late is counted by
        # lutb_device_wait_errors and not waited for), "collective" = a one-element all-reduce of the process group
        assert barrier in ("flags", "collective")
        self.barrier = barrier
        self._native = _native
        self.group = group
        self.lr = lr
        self.enabled = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if self.enabled else 1
        self.rank = dist.get_rank(group) if self.enabled else 0
        if self.world > _native.MAX_PEER_RANKS:
            raise ValueError(f"PeerTableUpdate supports up to {_native.MAX_PEER_RANKS} ranks")
        self.scale_div = self.world if average else 1
        self.layers = list(layers)
        self._side = None
        self._dirty = False
        # True: every rank applies its own gradient to its own copy (the replicas drift apart); for measuring what
        # the exchange costs
        self.paused = False
        self._state = {}
        for layer in self.layers:
            if not isinstance(layer, LUTLayerBasic) or layer._sequence_length != 1:
                raise ValueError("PeerTableUpdate handles non-sequence LUT layers")
            if layer._weights_gradient_policy.type != GradientType.Dense:
                raise ValueError("PeerTableUpdate needs the dense gradient policy")
            if not layer._weights.is_cuda or layer._weights.dtype != torch.float32:
                raise ValueError("PeerTableUpdate needs fp32 tables on a CUDA device")
        device = self.layers[0]._weights.device
        sizes = {}
        for li, layer in enumerate(self.layers):
            nbytes = 4 * ((layer._weights.numel() + 3) // 4 * 4)
            sizes[f"g{li}"] = nbytes
            sizes[f"w{li}"] = nbytes
        self._space = _PeerSpace(sizes, device, group, "PeerTableUpdate")
        if self.world > 1:
            self._side = torch.cuda.Stream(device=device)
        for li, layer in enumerate(self.layers):
            n = layer._weights.numel()
            grad = self._space.tensor(f"g{li}", torch.float32, n)
            shared = self._space.tensor(f"w{li}", torch.float32, n)
            grad.zero_()
            shared.copy_(layer._weights.detach())
            layer._weights.data = shared
            # slice r of the tables belongs to rank r; cuts on 16-byte boundaries
            cuts = [(n * r // self.world) // 4 * 4 for r in range(self.world)] + [n]
            self._state[id(layer)] = dict(grad=grad, cuts=cuts, g_ptrs=self._space.ptrs[f"g{li}"],
                                          w_ptrs=self._space.ptrs[f"w{li}"])
            layer._table_gradient_sink = self
        torch.cuda.synchronize(device)
        if self.world > 1:
            dist.barrier(group=group)  # every rank's tables are in place before anyone's kernel may store into them

    def _learning_rate(self):
        return float(self.lr() if callable(self.lr) else self.lr)

    def _rendezvous(self):
        """Barrier over the ranks on the side stream (the host does not block)."""
        self._space.barrier(self._side, self.barrier)

    # called by the layer's backward
    def gradient_buffer(self, layer):
        """The zeroed buffer the layer's backward accumulates its dense table gradient into."""
        grad = self._state[id(layer)]["grad"]
        grad.zero_()
        return grad

    def gradient_ready(self, layer):
        """The layer's table gradient has been launched on the current stream: reduce, update, distribute."""
        st = self._state[id(layer)]
        scale = self._learning_rate() / self.scale_div
        lo, hi = st["cuts"][self.rank], st["cuts"][self.rank + 1]
        device = layer._weights.device
        if self.world == 1 or self.paused:
            # no exchange: this rank's gradient alone updates this rank's copy of the whole table set
            own_g, own_w = [st["g_ptrs"][self.rank]], [st["w_ptrs"][self.rank]]
            self._native.peer_sgd_update(0, own_g, own_w, 0, st["cuts"][-1], scale,
                                         torch.cuda.current_stream(device).cuda_stream)
            return
        self._side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(self._side):
            self._rendezvous()  # every rank's gradient of this layer is complete and no rank still reads these tables
            self._native.peer_sgd_update(self.rank, st["g_ptrs"], st["w_ptrs"], lo, hi, scale, self._side.cuda_stream)
        self._dirty = True

    def wait(self):
        """Makes the current stream wait until every rank's update of this step has landed in this rank's tables."""
        if self._side is None or not self._dirty:
            return
        with torch.cuda.stream(self._side):
            self._rendezvous()
        torch.cuda.current_stream(self._side.device).wait_stream(self._side)
        self._dirty = False

    def remove(self):
        """Moves the tables back into ordinary device memory and releases the shared buffers (collective)."""
        if not self.layers:
            return
        self.wait()
        device = self.layers[0]._weights.device
        for layer in self.layers:
            layer._weights.data = layer._weights.data.clone()
            if getattr(layer, "_table_gradient_sink", None) is self:
                del layer._table_gradient_sink
        self._state = {}
        torch.cuda.synchronize(device)
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody still reads a buffer that is about to go
        self._space.release()
        self.layers = []


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False
