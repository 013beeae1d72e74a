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
