"""Query-sharded concatenation-mode attention on two CPU ranks (gloo), the layers' runtime served by the oracle:
every rank's output block, input-gradient block and the full table / positional gradients equal the unsharded
layer's, and one process running the two query ranges one after the other gives the same sums."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _layer(unified_pe=False):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_backend import use_oracle_backend
    from spiky_b200.lut_layer import LUTLayer, SynapseMeta

    S, E, Nt, Nc, Npe, O = 8, 10, 3, 2, 2, 6
    layer = LUTLayer(E, Nc, Nt, O, sequence_length=S, synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
                     concatenation_product=True, positional_dim=Npe, unified_pe=unified_pe, random_seed=5)
    with torch.no_grad():
        g = torch.Generator().manual_seed(1)
        layer._weights.copy_(torch.empty(layer._weights.shape).normal_(0.0, 0.05, generator=g))
    use_oracle_backend(layer)
    layer.train()
    g = torch.Generator().manual_seed(2)
    x = torch.rand(3, S, E, generator=g) * 2 - 1
    dy = torch.randn(3, S, O, generator=g)
    return layer, x, dy


def _reference(unified_pe):
    layer, x, dy = _layer(unified_pe)
    xr = x.clone().requires_grad_(True)
    y = layer(xr)
    y.backward(dy)
    return (y.detach(), xr.grad.clone(), layer._weights.grad.clone(), layer._positional_embeddings.grad.clone())


def _worker(rank, world, port, result_dir, unified_pe):
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        y_ref, dx_ref, dw_ref, dpe_ref = _reference(unified_pe)
        layer, x, dy = _layer(unified_pe)
        from spiky_b200.sequence_parallel import QueryShardedConcatAttention

        sharded = QueryShardedConcatAttention(layer)
        s_local = x.shape[1] // world
        sl = slice(rank * s_local, (rank + 1) * s_local)
        xl = x[:, sl].clone().requires_grad_(True)
        y = sharded(xl)
        y.backward(dy[:, sl].contiguous())
        checks = {
            "y": torch.allclose(y.detach(), y_ref[:, sl], rtol=1e-5, atol=1e-6),
            "dx": torch.allclose(xl.grad, dx_ref[:, sl], rtol=1e-5, atol=1e-6),
            "dw": torch.allclose(layer._weights.grad, dw_ref, rtol=1e-5, atol=1e-6),
            "dpe": torch.allclose(layer._positional_embeddings.grad, dpe_ref, rtol=1e-5, atol=1e-6),
            "nonzero": bool(dw_ref.abs().sum() > 0 and dx_ref.abs().sum() > 0 and dpe_ref.abs().sum() > 0),
        }
        open(os.path.join(result_dir, f"rank{rank}"), "w").write(repr(checks))
    finally:
        dist.destroy_process_group()


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(tmp_path, unified_pe):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), unified_pe), nprocs=2, join=True)
    for rank in range(2):
        checks = eval(open(tmp_path / f"rank{rank}").read())
        assert all(checks.values()), (rank, checks)


def test_query_sharded_concat_layer_matches_unsharded_layer(tmp_path):
    _run(tmp_path, False)


def test_query_sharded_concat_layer_with_unified_positional_embeddings(tmp_path):
    _run(tmp_path, True)


def test_one_process_is_the_unsharded_layer():
    """Without a process group the wrapper runs the pair stages over the whole sequence."""
    y_ref, dx_ref, dw_ref, dpe_ref = _reference(False)
    layer, x, dy = _layer(False)
    from spiky_b200.sequence_parallel import QueryShardedConcatAttention

    xr = x.clone().requires_grad_(True)
    y = QueryShardedConcatAttention(layer)(xr)
    y.backward(dy)
    assert torch.allclose(y.detach(), y_ref, rtol=1e-5, atol=1e-6)
    assert torch.allclose(xr.grad, dx_ref, rtol=1e-5, atol=1e-6)
    assert torch.allclose(layer._weights.grad, dw_ref, rtol=1e-5, atol=1e-6)
    assert torch.allclose(layer._positional_embeddings.grad, dpe_ref, rtol=1e-5, atol=1e-6)
