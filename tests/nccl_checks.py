"""Multi-GPU correctness checks over NCCL, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 tests/nccl_checks.py

Every rank computes its share through the CUDA library; rank 0 compares the combined result with the same layer run
on ONE GPU over the whole batch (and with the oracle where that is cheap).  Prints one line per check and exits
non-zero when any fails.  tests/test_multi_gpu.py runs it under pytest when at least two GPUs are visible.

  dp_fc_f32 / dp_fc_i32   sum over ranks of the table gradients = gradient of the concatenated batch
                           (1e-5 with fp32 accumulators, bit-exact with int32 accumulators)
  dp_overlapped            OverlappedGradientSync (NCCL AVG on a high-priority stream, per-parameter hooks) on a sparse
                           projection layer = full-batch gradient / world
  dp_sharded_update        ShardedTableUpdate = in-place SGD of the concatenated batch
  dp_sparse_exchange       exchange_sparse_gradients = sum of the ranks' sparse gradients
  shard_int8 / shard_fp32  detector-sharded inference = unsharded layer (int8: bit-exact)
  seq_concat               query-sharded concatenation-mode attention = unsharded layer
  replicas                 three data-parallel training steps of a small conv-net leave identical tables everywhere
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)

import synth  # noqa: E402
from oracle import lut_oracle as orc  # noqa: E402

RESULTS = []


def report(name, ok, detail=""):
    RESULTS.append(bool(ok))
    if dist.get_rank() == 0:
        print(f"{'ok  ' if ok else 'FAIL'} {name} {detail}", flush=True)


def rel_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def check_dp_fc(rank, world, dev, int_mode):
    from spiky_b200.lut_layer import LUTLayer, SynapseMeta

    B, I, Nt, Nc, O = 64 * world, 96, 12, 5, 24
    kw = dict(summation_dtype=torch.int32, _int_rescaler=0.05) if int_mode else {}
    layer = LUTLayer(I, Nc, Nt, O, synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0), random_seed=3, device=dev, **kw)
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(synth.normal(4, (layer._weights.numel(),), 0.0, 0.05)))
    layer.train()
    x = torch.from_numpy(synth.uniform(1, (B, 1, I))).to(dev)
    dy = torch.from_numpy(synth.normal(2, (B, 1, O))).to(dev)
    per = B // world
    sl = slice(rank * per, (rank + 1) * per)
    y, idx, md, mk = layer.forward_step(x[sl].contiguous())
    _, dw = layer.backward_step(x[sl].contiguous(), dy[sl].contiguous(), idx, md, mk)
    if int_mode:
        # fixed-point accumulators add exactly: exchange them as integers
        acc = torch.round(dw.double() * 1048575.0 * 0.05).to(torch.int64)
        dist.all_reduce(acc)
        total = acc
    else:
        total = dw.clone()
        dist.all_reduce(total)
    y, idx, md, mk = layer.forward_step(x)
    _, full = layer.backward_step(x, dy, idx, md, mk)
    if int_mode:
        full_acc = torch.round(full.double() * 1048575.0 * 0.05).to(torch.int64)
        report("dp_fc_i32", torch.equal(total, full_acc), "(fixed-point accumulators, bit-exact)")
    else:
        report("dp_fc_f32", rel_err(total.cpu().numpy(), full.cpu().numpy()) <= 1e-5,
               f"rel {rel_err(total.cpu().numpy(), full.cpu().numpy()):.2e}")


def small_convnet(dev, policy=None):
    from spiky_b200.lut_layer import (GradientPolicy, GradientType, ProjectionLUTLayer, SynapseMeta, PointSamplingPolicy,
                                      PointSamplingType)

    layers = []
    for li, (h, o, g, per) in enumerate([(20, 16, 8, 16), (16, 12, 6, 32)]):
        layer = ProjectionLUTLayer((h, h), (o, o), 6, g * g, per, (5, 5), (4, 4),
                                   synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
                                   detectors_sampling_policy=PointSamplingPolicy(PointSamplingType.Grid, grid_h=g, grid_w=g,
                                                                                 stride_h=2, stride_w=2, pad_h=2, pad_w=2),
                                   weights_gradient_policy=policy or GradientPolicy(GradientType.Dense), random_seed=50 + li)
        with torch.no_grad():
            layer._weights.normal_(0.0, 0.05, generator=torch.Generator().manual_seed(60 + li))
        layer.to(device=dev)
        layer.train()
        layers.append(layer)
    return layers


def check_dp_overlapped(rank, world, dev):
    from spiky_b200.data_parallel import OverlappedGradientSync

    layers = small_convnet(dev)
    B = 32 * world
    x = torch.from_numpy(synth.sparse_images(7, (B, 1, 20, 20))).to(dev)
    params = [l._weights for l in layers]
    sync = OverlappedGradientSync(params, average=True)

    def run(xb):
        for p in params:
            p.grad = None
        z = xb
        for l in layers:
            z = l(z)
        (z ** 2).sum().backward()

    per = B // world
    run(x[rank * per:(rank + 1) * per].contiguous())
    sync.wait()
    got = [p.grad.clone() for p in params]
    sync.remove()
    run(x)
    worst = max(rel_err(g.cpu().numpy(), (p.grad / world).cpu().numpy()) for g, p in zip(got, params))
    report("dp_overlapped", worst <= 1e-5, f"rel {worst:.2e}")


def check_dp_sharded_update(rank, world, dev, transport="collectives"):
    from spiky_b200.data_parallel import ShardedTableUpdate
    from spiky_b200.lut_layer import GradientPolicy, GradientType

    lr = 0.05
    B = 32 * world
    x = torch.from_numpy(synth.sparse_images(8, (B, 1, 20, 20))).to(dev)

    def run(layers, xb):
        z = xb
        for l in layers:
            z = l(z)
        (z ** 2).sum().backward()

    layers = small_convnet(dev)
    per = B // world
    try:
        sync = ShardedTableUpdate(layers, lr, average=False, transport=transport, batch_size=per)
    except RuntimeError as e:
        # all ranks raise together; a node that does not allow the mapping cannot run the peer transport
        report("dp_sharded_update_" + transport, True, "unavailable here: " + str(e)[:160])
        return
    run(layers, x[rank * per:(rank + 1) * per].contiguous())
    sync.wait()
    torch.cuda.synchronize()
    ref = small_convnet(dev, GradientPolicy(GradientType.Internal))
    for l in ref:
        l.set_external_learning_rate_hook(lambda w: lr)
    run(ref, x)
    worst = max(rel_err(a._weights.detach().cpu().numpy(), b._weights.detach().cpu().numpy()) for a, b in zip(layers, ref))
    moved = all(not torch.equal(a._weights, small._weights) for a, small in zip(ref, small_convnet(dev)))
    # a second step reuses the gathered arrays; the replicas must stay bit-identical
    run(layers, x[rank * per:(rank + 1) * per].contiguous())
    sync.wait()
    torch.cuda.synchronize()
    sums = torch.stack([l._weights.detach().double().sum() for l in layers])
    lo, hi = sums.clone(), sums.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    report("dp_sharded_update_" + transport, worst <= 1e-5 and moved and bool((hi == lo).all()),
           f"rel {worst:.2e}, checksum spread {float((hi - lo).abs().max()):.1e}")
    sync.remove()


def check_dp_peer_update(rank, world, dev, barrier="flags"):
    """Gradient reduction + SGD + distribution of the tables in one kernel over peer memory: one step against the
    single-process update of the whole batch, replicas bit-identical after a second one."""
    from spiky_b200.data_parallel import PeerTableUpdate
    from spiky_b200.lut_layer import GradientPolicy, GradientType

    lr = 0.05
    B = 32 * world
    x = torch.from_numpy(synth.sparse_images(8, (B, 1, 20, 20))).to(dev)

    def run(layers, xb):
        z = xb
        for l in layers:
            z = l(z)
        (z ** 2).sum().backward()

    layers = small_convnet(dev, GradientPolicy(GradientType.Dense))
    try:
        sync = PeerTableUpdate(layers, lr, average=False, barrier=barrier)
    except RuntimeError as e:
        # all ranks raise together; a node that does not allow the mapping cannot run this path
        report("dp_peer_update", True, "unavailable here: " + str(e)[:160])
        return
    per = B // world
    run(layers, x[rank * per:(rank + 1) * per].contiguous())
    sync.wait()
    torch.cuda.synchronize()
    ref = small_convnet(dev, GradientPolicy(GradientType.Internal))
    for l in ref:
        l.set_external_learning_rate_hook(lambda w: lr)
    run(ref, x)
    worst = max(rel_err(a._weights.detach().cpu().numpy(), b._weights.detach().cpu().numpy()) for a, b in zip(layers, ref))
    # a second step on the updated tables (gradient buffers reused, exchange of step one long finished)
    run(layers, x[rank * per:(rank + 1) * per].contiguous())
    sync.wait()
    torch.cuda.synchronize()
    sums = torch.stack([l._weights.detach().double().sum() for l in layers])
    lo, hi = sums.clone(), sums.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    no_grads = all(l._weights.grad is None for l in layers)
    report("dp_peer_update_" + barrier, worst <= 1e-5 and bool((hi == lo).all()) and no_grads,
           f"rel {worst:.2e}, checksum spread {float((hi - lo).abs().max()):.1e}")
    sync.remove()
    report("dp_peer_update_removed", all(l._weights.is_cuda and not hasattr(l, "_table_gradient_sink") for l in layers))


def check_dp_sparse_exchange(rank, world, dev):
    from spiky_b200.data_parallel import exchange_sparse_gradients
    from spiky_b200.lut_layer import LUTLayer, SynapseMeta, GradientPolicy, GradientType

    B, I, Nt, Nc, O = 40 * world, 48, 6, 6, 16
    layer = LUTLayer(I, Nc, Nt, O, synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
                     weights_gradient_policy=GradientPolicy(GradientType.Sparse), random_seed=5, device=dev)
    layer.train()
    x = torch.from_numpy(synth.uniform(11, (B, 1, I))).to(dev)
    dy = torch.from_numpy(synth.normal(12, (B, 1, O))).to(dev)
    per = B // world
    sl = slice(rank * per, (rank + 1) * per)
    y, idx, md, mk = layer.forward_step(x[sl].contiguous())
    _, g = layer.backward_step(x[sl].contiguous(), dy[sl].contiguous(), idx, md, mk)
    layer._weights.grad = g
    nnz_local = g._nnz()
    exchange_sparse_gradients([layer._weights])
    total = layer._weights.grad.coalesce().to_dense()
    y, idx, md, mk = layer.forward_step(x)
    _, full = layer.backward_step(x, dy, idx, md, mk)
    err = rel_err(total.cpu().numpy(), full.to_dense().cpu().numpy())
    report("dp_sparse_exchange", err <= 1e-5 and nnz_local < layer._weights.numel() // 2,
           f"rel {err:.2e}, {nnz_local} of {layer._weights.numel()} cells touched on this rank")


def check_sharded_inference(rank, world, dev):
    from spiky_b200.inference import LUTInference

    B, I, Nt, Nc, O = 300, 512, 64 * world, 8, 64
    gen = torch.Generator().manual_seed(5)
    a1 = torch.randint(0, I, (Nt, Nc), generator=gen)
    anchors = torch.stack([a1, (a1 + torch.randint(1, I, (Nt, Nc), generator=gen)) % I], dim=-1).to(torch.int32)
    q = torch.randint(-127, 128, (Nt * (1 << Nc) * O,), generator=gen, dtype=torch.int32).to(torch.int8)
    s = (0.02 / 127) * (0.5 + torch.rand(Nt, generator=gen))
    w = torch.empty(Nt * (1 << Nc) * O).normal_(0.0, 0.02, generator=gen)
    x = torch.empty(B, I).normal_(generator=gen).to(dev)
    for name, tables, scales in (("shard_int8", q, s), ("shard_fp32", w, None)):
        sharded = LUTInference.shard_of(rank, world, I, O, Nt, Nc, anchors, tables, scales, int_rescaler=0.05,
                                        group=dist.group.WORLD, device=dev)
        whole = LUTInference(I, O, Nt, Nc, anchors, tables, scales, int_rescaler=0.05, device=dev)
        got, want = sharded(x), whole(x)
        if scales is not None:
            report(name, torch.equal(got, want), "(int32 accumulators, bit-exact)")
        else:
            report(name, rel_err(got.cpu().numpy(), want.cpu().numpy()) <= 1e-5,
                   f"rel {rel_err(got.cpu().numpy(), want.cpu().numpy()):.2e}")


def check_seq_concat(rank, world, dev):
    from spiky_b200.lut_layer import LUTLayer, SynapseMeta
    from spiky_b200.sequence_parallel import QueryShardedConcatAttention

    B, S, E, Nt, Nc, Npe, O = 2, 8 * world, 24, 6, 4, 3, 16

    def make():
        layer = LUTLayer(E, Nc, Nt, O, sequence_length=S, synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
                         concatenation_product=True, positional_dim=Npe, random_seed=5, device=dev)
        with torch.no_grad():
            layer._weights.copy_(torch.empty(layer._weights.shape).normal_(0.0, 0.05, generator=torch.Generator().manual_seed(1)))
        layer.train()
        return layer

    g = torch.Generator().manual_seed(2)
    x = (torch.rand(B, S, E, generator=g) * 2 - 1).to(dev)
    dy = torch.randn(B, S, O, generator=g).to(dev)
    ref = make()
    xr = x.clone().requires_grad_(True)
    ref(xr).backward(dy)
    layer = make()
    s_local = S // world
    sl = slice(rank * s_local, (rank + 1) * s_local)
    xl = x[:, sl].clone().requires_grad_(True)
    y = QueryShardedConcatAttention(layer)(xl)
    y.backward(dy[:, sl].contiguous())
    errs = dict(y=rel_err(y.detach().cpu().numpy(), ref(x).detach()[:, sl].cpu().numpy()),
                dx=rel_err(xl.grad.cpu().numpy(), xr.grad[:, sl].cpu().numpy()),
                dw=rel_err(layer._weights.grad.cpu().numpy(), ref._weights.grad.cpu().numpy()),
                dpe=rel_err(layer._positional_embeddings.grad.cpu().numpy(), ref._positional_embeddings.grad.cpu().numpy()))
    worst = torch.tensor([max(errs.values())], device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    report("seq_concat", float(worst) <= 1e-5, f"worst rel over ranks {float(worst):.2e}")


def check_replicas(rank, world, dev):
    from spiky_b200.data_parallel import OverlappedGradientSync

    layers = small_convnet(dev)
    params = [l._weights for l in layers]
    sync = OverlappedGradientSync(params, average=True)
    for step in range(3):
        x = torch.from_numpy(synth.sparse_images(100 + 10 * step + rank, (32, 1, 20, 20))).to(dev)
        for p in params:
            p.grad = None
        z = x
        for l in layers:
            z = l(z)
        (z ** 2).sum().backward()
        with torch.no_grad():
            for p in sync.wait_each():
                p.add_(p.grad, alpha=-0.05)
    sums = torch.stack([p.detach().double().sum() for p in params])
    lo, hi = sums.clone(), sums.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    report("replicas", bool((hi == lo).all()), f"checksum spread {float((hi - lo).abs().max()):.1e}")
    sync.remove()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    try:
        check_dp_fc(rank, world, dev, False)
        check_dp_fc(rank, world, dev, True)
        check_dp_overlapped(rank, world, dev)
        check_dp_sharded_update(rank, world, dev)
        check_dp_sharded_update(rank, world, dev, "peer")
        check_dp_peer_update(rank, world, dev, "flags")
        check_dp_peer_update(rank, world, dev, "collective")
        check_dp_sparse_exchange(rank, world, dev)
        check_sharded_inference(rank, world, dev)
        check_seq_concat(rank, world, dev)
        check_replicas(rank, world, dev)
        from spiky_b200 import _native
        report("device_waits", _native.device_wait_errors() == 0)
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()
    if not all(RESULTS):
        sys.exit(1)


if __name__ == "__main__":
    main()
