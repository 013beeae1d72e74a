"""The default bench workload's training step on CPU (layers served by the oracle): the three ways bench.py can make the
SGD update - dense gradients + torch.optim.SGD, the Internal gradient policy, the sharded in-place update - train
the same network to the same tables."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def test_convnet_step_variants_agree_on_cpu():
    import bench
    from oracle_backend import use_oracle_backend
    from spiky_b200.data_parallel import ShardedTableUpdate

    B, steps = 3, 2
    results = {}
    start = None
    for variant in ("dense", "internal", "sharded"):
        wl = bench.SparseConvNetWorkload(batch=B, internal=variant == "internal", sharded=variant == "sharded")
        wl.layers = wl.build(None)
        for layer in wl.layers:
            use_oracle_backend(layer)
            layer.train()
        if start is None:
            start = [l._weights.detach().clone() for l in wl.layers]
        params = [l._weights for l in wl.layers]
        if wl.sharded:
            wl.table_sync = ShardedTableUpdate(wl.layers[:-1], wl.LR)
            params = params[-1:]
        wl.opt = None if wl.internal else torch.optim.SGD(params, lr=wl.LR)
        losses = []
        for s in range(steps):
            x, labels = wl.host_inputs(500 + s, B)
            loss = wl._run(torch.from_numpy(x).view(B, 1, 28, 28), torch.from_numpy(labels))
            losses.append(float(loss.detach()))
        assert np.isfinite(losses).all()
        results[variant] = ([l._weights.detach() for l in wl.layers], losses)
    dense_w, dense_losses = results["dense"]
    assert any(not torch.equal(a, b) for a, b in zip(dense_w, start)), "the step changed nothing"
    for variant in ("internal", "sharded"):
        w, losses = results[variant]
        assert np.allclose(losses, dense_losses, rtol=1e-5), variant
        for li, (a, b) in enumerate(zip(w, dense_w)):
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-7), f"{variant}: layer {li}"


def test_both_arms_describe_the_workload_identically():
    """`config` of the JSON line must not depend on whether the workload was set up on a device (our arm) or only
    constructed (the reference arm)."""
    import bench

    for name in ("sparse_convnet", "sparse_convnet_eager", "sparse_convnet_sharded_peer_graph"):
        cfg = bench.workload_config(bench.WORKLOADS[name](None))
        assert cfg["l2"] == "inputs>L2" and cfg["per_gpu_units"] == 512
    assert bench.workload_config(bench.WORKLOADS["sparse_convnet"](None)) == \
        bench.workload_config(bench.WORKLOADS["sparse_convnet_eager"](None))
