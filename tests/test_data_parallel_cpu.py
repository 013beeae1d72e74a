"""Data-parallel exchange on CPU ranks (gloo, world size 2): the all-reduced per-shard table gradients equal
the full-batch gradient, and a rank that fails before the collective is reported on the host (no GPU involved)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, result_dir, fail_rank):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import datetime
    import synth
    from oracle import lut_oracle as orc
    from spiky_b200.data_parallel import allreduce_gradients, shard_batch

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        B, I, Nt, Nc, O = 24, 40, 6, 4, 8
        x = synth.uniform(1, (B, I))
        anchors = synth.anchor_pairs(2, Nt, Nc, I)
        W = synth.normal(3, (Nt * (1 << Nc) * O,), 0.0, 0.02)
        dY = synth.normal(4, (B, O))
        b0, b1 = shard_batch(B, rank, world)
        if rank == fail_rank:
            raise RuntimeError("injected failure before the collective")
        _, idx, md, mk = orc.nonseq_fc_forward(W, x[b0:b1], anchors, Nt, Nc, O)
        _, dW = orc.nonseq_fc_backward(W, dY[b0:b1], anchors, idx, md, mk, I, Nc)
        p = torch.nn.Parameter(torch.from_numpy(W.copy()))
        p.grad = torch.from_numpy(dW)
        small = torch.nn.Parameter(torch.zeros(5))
        small.grad = torch.full((5,), float(rank + 1))
        allreduce_gradients([p, small])
        if rank == 0:
            _, idx, md, mk = orc.nonseq_fc_forward(W, x, anchors, Nt, Nc, O)
            _, full = orc.nonseq_fc_backward(W, dY, anchors, idx, md, mk, I, Nc)
            err = float(np.abs(p.grad.numpy() - full).max() / np.abs(full).max())
            ok = err < 1e-6 and torch.equal(small.grad, torch.full((5,), float(sum(range(1, world + 1)))))
            open(os.path.join(result_dir, "ok"), "w").write(f"{ok} {err}")
    finally:
        dist.destroy_process_group()


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_allreduce_of_shard_gradients_equals_full_batch(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), -1), nprocs=2, join=True)
    ok, err = open(tmp_path / "ok").read().split()
    assert ok == "True", f"relative error {err}"


def test_failed_rank_is_reported_on_the_host(tmp_path):
    """A rank that raises before the collective: the job ends with an error on the host instead of hanging
    (the surviving rank's collective is bounded by the process-group timeout)."""
    with pytest.raises(Exception):
        mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), 1), nprocs=2, join=True)
    assert not (tmp_path / "ok").exists()


def _overlap_worker(rank, world, port, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import datetime
    import synth
    from oracle import lut_oracle as orc
    from spiky_b200.data_parallel import OverlappedGradientSync

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        # (1) hook-driven exchange: every parameter's gradient is averaged over the ranks as soon as autograd has
        # produced it; wait_each yields the parameters in production order
        a = torch.nn.Parameter(torch.arange(6, dtype=torch.float32))
        b = torch.nn.Parameter(torch.ones(4))
        sync = OverlappedGradientSync([a, b], average=True)
        loss = ((rank + 1) * a).sum() + ((rank + 1) ** 2 * b * b).sum()
        loss.backward()
        order = [id(p) for p in sync.wait_each()]
        mean1 = sum(r + 1 for r in range(world)) / world
        mean2 = sum(2 * (r + 1) ** 2 for r in range(world)) / world
        ok = set(order) == {id(a), id(b)} and torch.allclose(a.grad, torch.full((6,), mean1)) and \
            torch.allclose(b.grad, torch.full((4,), mean2)) and sync.handles == []
        sync.remove()
        # (2) detector sharding: integer partial accumulators of the shards add up to the unsharded result exactly
        B, I, Nt, Nc, O = 10, 64, 128, 5, 8
        x = synth.normal(11, (B, I))
        anchors = synth.anchor_pairs(12, Nt, Nc, I)
        q = synth.integers(13, (Nt * (1 << Nc) * O,), -127, 128).astype(np.int8)
        s = (0.02 / 127 * synth.uniform(14, (Nt,), 0.5, 1.5)).astype(np.float32)
        per = Nt // world
        T = 1 << Nc
        part, _ = orc.infer_int8(q.reshape(Nt, -1)[rank * per:(rank + 1) * per].reshape(-1), s[rank * per:(rank + 1) * per],
                                 x, anchors.reshape(Nt, -1)[rank * per:(rank + 1) * per].reshape(per, Nc, 2), per, Nc, O,
                                 int_rescaler=0.05)
        acc = torch.from_numpy(part.copy())
        dist.all_reduce(acc, op=dist.ReduceOp.SUM)
        full, _ = orc.infer_int8(q, s, x, anchors, Nt, Nc, O, int_rescaler=0.05)
        ok = ok and np.array_equal(acc.numpy(), full)
        if rank == 0:
            open(os.path.join(result_dir, "ok2"), "w").write(str(bool(ok)))
    finally:
        dist.destroy_process_group()


def test_overlapped_gradient_sync_and_sharded_accumulators(tmp_path):
    mp.spawn(_overlap_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "ok2").read() == "True"


def _sparse_worker(rank, world, port, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import datetime
    import synth
    from oracle import lut_oracle as orc
    from spiky_b200.data_parallel import average_internal_policy_weights, exchange_sparse_gradients, shard_batch
    from spiky_b200.lut_layer import GradientPolicy, GradientType, LUTLayer, SynapseMeta

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        # (1) sparse exchange: each rank holds the touched cells of its shard's table gradient; after the exchange
        # the (summed) sparse gradient equals the full-batch dense gradient
        B, I, Nt, Nc, O = 12, 40, 6, 5, 8
        x = synth.uniform(1, (B, I))
        anchors = synth.anchor_pairs(2, Nt, Nc, I)
        W = synth.normal(3, (Nt * (1 << Nc) * O,), 0.0, 0.02)
        dY = synth.normal(4, (B, O))
        b0, b1 = shard_batch(B, rank, world)
        _, idx, md, mk = orc.nonseq_fc_forward(W, x[b0:b1], anchors, Nt, Nc, O)
        _, dW = orc.nonseq_fc_backward(W, dY[b0:b1], anchors, idx, md, mk, I, Nc)
        p = torch.nn.Parameter(torch.from_numpy(W.copy()))
        cells = torch.from_numpy(np.flatnonzero(dW))
        p.grad = torch.sparse_coo_tensor(cells.unsqueeze(0), torch.from_numpy(dW)[cells], size=p.shape)
        untouched = torch.nn.Parameter(torch.zeros(7))          # no gradient on any rank
        lonely = torch.nn.Parameter(torch.zeros(9))             # gradient on rank 1 only
        if rank == 1:
            lonely.grad = torch.sparse_coo_tensor(torch.tensor([[2, 5]]), torch.tensor([1.5, -2.0]), size=(9,))
        dense = torch.nn.Parameter(torch.zeros(3))              # dense everywhere: left alone
        dense.grad = torch.full((3,), float(rank))
        exchange_sparse_gradients([p, untouched, lonely, dense])
        _, idx, md, mk = orc.nonseq_fc_forward(W, x, anchors, Nt, Nc, O)
        _, full = orc.nonseq_fc_backward(W, dY, anchors, idx, md, mk, I, Nc)
        got = p.grad.to_dense().numpy()
        ok = p.grad.is_sparse and float(np.abs(got - full).max()) <= 1e-6 * float(np.abs(full).max())
        ok = ok and p.grad._nnz() < p.numel() and untouched.grad is None
        expect = torch.zeros(9)
        expect[2], expect[5] = 1.5, -2.0
        ok = ok and torch.equal(lonely.grad.to_dense(), expect)
        ok = ok and torch.equal(dense.grad, torch.full((3,), float(rank)))
        # (2) Internal policy: tables that took their rank's in-place update are averaged over the ranks
        layer = LUTLayer(n_inputs=16, n_anchors_per_detector=3, n_detectors=4, n_outputs=5,
                         synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
                         weights_gradient_policy=GradientPolicy(GradientType.Internal), random_seed=5, device=None)
        other = LUTLayer(n_inputs=16, n_anchors_per_detector=3, n_detectors=4, n_outputs=5,
                         synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0), random_seed=5, device=None)
        model = torch.nn.ModuleList([layer, other])
        start = layer._weights.detach().clone()
        step = torch.arange(start.numel(), dtype=torch.float32) * 1e-3
        with torch.no_grad():
            layer._weights -= (rank + 1) * step      # stands for -lr * dW_r
            other._weights += rank                   # not an Internal-policy layer: must stay as it is
        kept = other._weights.detach().clone()
        n = average_internal_policy_weights(model)
        mean = sum(r + 1 for r in range(world)) / world
        ok = ok and n == 1 and torch.allclose(layer._weights.detach(), start - mean * step, atol=1e-6)
        ok = ok and torch.equal(other._weights.detach(), kept)
        flags = [torch.zeros(1) for _ in range(world)]
        dist.all_gather(flags, torch.tensor([1.0 if ok else 0.0]))
        if rank == 0:
            open(os.path.join(result_dir, "ok3"), "w").write(str(all(float(f) == 1.0 for f in flags)))
    finally:
        dist.destroy_process_group()


def test_sparse_gradient_exchange_and_internal_policy_average(tmp_path):
    mp.spawn(_sparse_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "ok3").read() == "True"


def _sharded_worker(rank, world, port, result_dir, weight_gather):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import datetime
    import synth
    from oracle import lut_oracle as orc
    from spiky_b200.data_parallel import ShardedTableUpdate, shard_batch
    from spiky_b200.lut_layer import ProjectionLUTLayer, SynapseMeta

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    try:
        meta = SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.2, initial_weight=-0.1)
        layer = ProjectionLUTLayer((16, 16), (12, 12), 4, 10, 4, (5, 5), (3, 3), synapse_meta=meta, random_seed=2,
                                   device=None)
        index = layer._lut_dm._sparse
        sp = dict(index.numpy(), group_size=index.group_size)
        anchors = layer._detector_anchors.numpy()
        W0 = layer._weights.detach().numpy().copy()
        B, I, O, Nc, lr = 10, 256, 144, 4, 0.05
        x = synth.sparse_images(41, (B, I))
        dY = synth.normal(42, (B, O))
        _, idx, md, mk = orc.nonseq_sparse_forward(W0, x, anchors, sp, Nc, O)
        _, dW_global = orc.nonseq_sparse_backward(W0, dY, anchors, idx, md, mk, sp, I, Nc)

        sync = ShardedTableUpdate([layer], lr, weight_gather=weight_gather)
        plan = sync._plans[id(layer)]
        calls = []

        def apply_with_oracle(layer_, batch, dY_all, idx_all, scale, c0, c1):
            # the kernel's arithmetic on the gathered batch, restricted to this rank's share of the weight slots
            assert idx_all.dtype == torch.uint8 and batch == B
            idx_np = idx_all.numpy().astype(np.int32).reshape(batch, -1)
            dY_np = dY_all.numpy().reshape(batch, O)
            w = layer_._weights.detach().numpy()
            zeros = np.zeros_like(idx_np)
            _, dW = orc.nonseq_sparse_backward(w, dY_np, anchors, idx_np, zeros.astype(np.float32) + 1.0, zeros, sp, I, Nc)
            lo, hi = plan["wcuts"][plan["cuts"].index(c0)], plan["wcuts"][plan["cuts"].index(c0) + 1]
            calls.append((c0, c1, lo, hi))
            with torch.no_grad():
                layer_._weights[lo:hi] += scale * torch.from_numpy(dW[lo:hi])

        sync._apply = apply_with_oracle
        b0, b1 = shard_batch(B, rank, world)
        sync._on_backward(layer, torch.from_numpy(idx[b0:b1].reshape(-1).copy()),
                          torch.from_numpy(dY[b0:b1].reshape(-1).copy()), b1 - b0)
        sync.wait()
        got = layer._weights.detach().numpy()
        want = W0 - (lr / world) * dW_global
        err = float(np.abs(got - want).max())
        ok = err <= 1e-6 * max(float(np.abs(want).max()), 1e-30) and len(calls) == 1
        ok = ok and calls[0][:2] == (plan["cuts"][rank], plan["cuts"][rank + 1]) and plan["cuts"][0] == 0
        ok = ok and plan["wcuts"][-1] == index.n_weights and float(np.abs(got - W0).max()) > 0
        flags = [torch.zeros(1) for _ in range(world)]
        dist.all_gather(flags, torch.tensor([1.0 if ok else 0.0]))
        if rank == 0:
            open(os.path.join(result_dir, "ok4"), "w").write(f"{all(float(f) == 1.0 for f in flags)} {err}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("weight_gather", ["padded", "uneven"])
def test_sharded_table_update_equals_global_batch_sgd(tmp_path, weight_gather):
    mp.spawn(_sharded_worker, args=(2, _free_port(), str(tmp_path), weight_gather), nprocs=2, join=True)
    ok, err = open(tmp_path / "ok4").read().split()
    assert ok == "True", f"max abs error {err}"


def _sharded_model_worker(rank, world, port, result_dir):
    """Two sparse layers and a fully connected readout trained for two steps: ranks with half the batch each and the
    sharded table update must end with the tables a single process gets from SGD on the whole batch."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import datetime
    import synth
    from oracle_backend import use_oracle_backend
    from spiky_b200.data_parallel import ShardedTableUpdate, allreduce_gradients, shard_batch
    from spiky_b200.lut_layer import LUTLayer, ProjectionLUTLayer, SynapseMeta

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        meta = SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.3, initial_weight=-0.15)

        def build():
            torch.manual_seed(123)  # the initial noise comes from the global generator
            layers = torch.nn.ModuleList([
                ProjectionLUTLayer((12, 12), (10, 10), 4, 6, 5, (5, 5), (3, 3), synapse_meta=meta, random_seed=2, device=None),
                ProjectionLUTLayer((10, 10), (8, 8), 4, 5, 6, (5, 5), (3, 3), synapse_meta=meta, random_seed=3, device=None),
                LUTLayer(64, 4, 6, 5, synapse_meta=meta, random_seed=4, device=None)])
            use_oracle_backend(layers)
            layers.train()
            return layers

        def run(layers, x, labels):
            z = x
            for layer in layers[:-1]:
                z = layer(z)
            logits = layers[-1](z.reshape(z.shape[0], 1, -1)).reshape(z.shape[0], -1)
            return torch.nn.functional.cross_entropy(logits, labels)

        B, lr, steps = 8, 0.1, 2
        xs = [torch.from_numpy(synth.sparse_images(60 + s, (B, 144))).view(B, 1, 12, 12) for s in range(steps)]
        ys = [torch.from_numpy(synth.integers(70 + s, (B,), 0, 5).astype(np.int64)) for s in range(steps)]
        # (a) single process, whole batch, dense gradients + SGD
        full = build()
        opt = torch.optim.SGD([l._weights for l in full], lr=lr)
        for s in range(steps):
            opt.zero_grad()
            run(full, xs[s], ys[s]).backward()
            opt.step()
        # (b) this rank's half of the batch, sharded in-place update of the sparse layers, all-reduce for the readout
        mine = build()
        sync = ShardedTableUpdate(list(mine[:-1]), lr)
        opt = torch.optim.SGD([mine[-1]._weights], lr=lr)
        b0, b1 = shard_batch(B, rank, world)
        for s in range(steps):
            sync.wait()
            opt.zero_grad()
            run(mine, xs[s][b0:b1], ys[s][b0:b1]).backward()
            assert mine[0]._weights.grad is None and mine[1]._weights.grad is None
            allreduce_gradients([mine[-1]._weights], average=True)
            opt.step()
        sync.wait()
        ok = True
        worst = 0.0
        for a, b in zip(full, mine):
            err = float((a._weights - b._weights).abs().max())
            worst = max(worst, err)
            ok = ok and err <= 2e-6
        flags = [torch.zeros(1) for _ in range(world)]
        dist.all_gather(flags, torch.tensor([1.0 if ok else 0.0]))
        if rank == 0:
            open(os.path.join(result_dir, "ok5"), "w").write(f"{all(float(f) == 1.0 for f in flags)} {worst}")
    finally:
        dist.destroy_process_group()


def test_sharded_table_update_trains_like_one_process(tmp_path):
    mp.spawn(_sharded_model_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    ok, err = open(tmp_path / "ok5").read().split()
    assert ok == "True", f"max abs difference of the tables {err}"
