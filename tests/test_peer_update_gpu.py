"""Data-parallel SGD over peer memory (lutb_peer_sgd_update, spiky_b200.data_parallel.PeerTableUpdate) on one GPU:
the kernel with the ranks' buffers emulated as separate allocations of the same device (one launch per rank, nothing
waits), bit for bit against the oracle's statement of the arithmetic; and the layer-level update at world size 1 against
torch's SGD on the dense gradients."""
import numpy as np
import pytest
import torch

import synth
from oracle import lut_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_ranks,n", [(1, 1000), (2, 4099), (3, 37), (4, 65536 + 5), (8, 300001), (11, 2050), (16, 70001)])
def test_kernel_matches_the_oracle_bit_for_bit(n_ranks, n):
    from spiky_b200 import _native

    scale = 0.0125
    w0 = synth.normal(10 + n_ranks, (n,), 0.0, 0.05)
    grads = [synth.normal(20 + r, (n,), 0.0, 1.0) for r in range(n_ranks)]
    want = orc.peer_sgd_update(w0, grads, scale)
    g_dev = [torch.from_numpy(g).cuda() for g in grads]
    # every emulated rank starts from the same tables; guard cells around them must stay untouched
    w_dev = [torch.full((n + 8,), 7.0, device="cuda") for _ in range(n_ranks)]
    for w in w_dev:
        w[4:4 + n] = torch.from_numpy(w0).cuda()
    # slices on arbitrary (also unaligned) cuts
    cuts = sorted({0, n} | {int(c) for c in np.random.default_rng(n).integers(0, n + 1, n_ranks - 1)})
    cuts += [n] * (n_ranks + 1 - len(cuts))
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(n_ranks):
        _native.peer_sgd_update(r, [g.data_ptr() for g in g_dev], [w.data_ptr() + 16 for w in w_dev], cuts[r],
                                cuts[r + 1], scale, stream)
    torch.cuda.synchronize()
    for w in w_dev:
        got = w.cpu().numpy()
        assert np.array_equal(got[4:4 + n], want)
        assert (got[:4] == 7.0).all() and (got[4 + n:] == 7.0).all()


def test_argument_checks():
    from spiky_b200 import _native

    w = torch.zeros(64, device="cuda")
    with pytest.raises(ValueError):
        _native.peer_sgd_update(0, [w.data_ptr() + 4], [w.data_ptr()], 0, 8, 1.0, 0)   # unaligned buffer
    with pytest.raises(ValueError):
        _native.peer_sgd_update(1, [w.data_ptr()], [w.data_ptr()], 0, 8, 1.0, 0)       # rank outside the group
    with pytest.raises(ValueError):
        _native.peer_sgd_update(0, [w.data_ptr()], [w.data_ptr()], 8, 4, 1.0, 0)       # reversed slice


def test_shareable_buffer_round_trip():
    """Allocation and handle export work on this device (mapping needs a second process: the two-GPU check)."""
    from spiky_b200 import _native
    from spiky_b200.data_parallel import _DeviceSpan

    ptr, handle = _native.peer_alloc(4096)
    try:
        assert ptr % 256 == 0 and len(handle) == _native.PEER_HANDLE_BYTES
        t = torch.as_tensor(_DeviceSpan(ptr, 1024), device="cuda:0")
        assert t.data_ptr() == ptr and t.dtype == torch.float32
        t.fill_(3.0)
        assert float(t.sum()) == 3072.0
        del t
        torch.cuda.synchronize()
    finally:
        _native.peer_free(ptr)


def _net(seed):
    from spiky_b200.lut_layer import (GradientPolicy, GradientType, LUTLayer, ProjectionLUTLayer, SynapseMeta,
                                      PointSamplingPolicy, PointSamplingType)
    meta = SynapseMeta(min_weight=-1.0, max_weight=1.0)
    policy = GradientPolicy(GradientType.Dense)
    proj = ProjectionLUTLayer((12, 12), (8, 8), 6, 16, 8, (5, 5), (4, 4), synapse_meta=meta,
                              detectors_sampling_policy=PointSamplingPolicy(PointSamplingType.Grid, grid_h=4, grid_w=4,
                                                                            stride_h=2, stride_w=2, pad_h=2, pad_w=2),
                              weights_gradient_policy=policy, random_seed=seed)
    fc = LUTLayer(64, 6, 12, 10, synapse_meta=meta, weights_gradient_policy=policy, random_seed=seed + 1)
    for i, l in enumerate((proj, fc)):
        with torch.no_grad():
            l._weights.normal_(0.0, 0.05, generator=torch.Generator().manual_seed(seed + 10 + i))
        l.to(device="cuda:0")
        l.train()
    return [proj, fc]


def _step(layers, x, labels):
    z = layers[0](x)
    logits = layers[1](z.reshape(z.shape[0], 1, -1)).reshape(z.shape[0], -1)
    loss = torch.nn.functional.cross_entropy(logits, labels)
    loss.backward()
    return float(loss.detach())


def test_layer_update_equals_sgd_on_dense_gradients():
    """World size 1: the fused update is plain SGD; the tables follow torch.optim.SGD step for step."""
    from spiky_b200.data_parallel import PeerTableUpdate

    lr = 0.05
    x = torch.from_numpy(synth.uniform(5, (32, 1, 12, 12))).cuda()
    labels = torch.from_numpy(synth.integers(6, (32,), 0, 10)).cuda()
    ref = _net(300)
    opt = torch.optim.SGD([l._weights for l in ref], lr=lr)
    ours = _net(300)
    sync = PeerTableUpdate(ours, lr)
    for step in range(3):
        opt.zero_grad(set_to_none=True)
        loss_ref = _step(ref, x, labels)
        opt.step()
        sync.wait()
        loss = _step(ours, x, labels)
        assert all(l._weights.grad is None for l in ours)
        assert abs(loss - loss_ref) <= 1e-5 * abs(loss_ref)
        for a, b in zip(ours, ref):
            torch.testing.assert_close(a._weights.detach(), b._weights.detach(), rtol=0, atol=1e-7)
    moved = ours[0]._weights.detach().clone()
    sync.remove()
    assert torch.equal(ours[0]._weights.detach(), moved)   # the tables survive the move back to ordinary memory
    assert not hasattr(ours[0], "_table_gradient_sink")


def test_barrier_passes_when_every_flag_holds_the_epoch():
    """Two emulated ranks on one device: rank 1's arrival is written by the host, then rank 0's barrier kernel must
    publish its own arrival in both flag arrays and return at once."""
    from spiky_b200 import _native

    flags = [torch.zeros(16, dtype=torch.int64, device="cuda") for _ in range(2)]
    flags[0][1] = 3                      # "rank 1 has arrived at epoch 3", in rank 0's array
    before = _native.device_wait_errors()
    _native.peer_barrier(0, [f.data_ptr() for f in flags], 3, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert _native.device_wait_errors() == before
    assert flags[0].tolist()[:2] == [3, 3] and flags[1].tolist()[:2] == [3, 0]
    # a later epoch of the other rank also satisfies the wait (flags only grow)
    flags[0][1] = 9
    _native.peer_barrier(0, [f.data_ptr() for f in flags], 4, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert _native.device_wait_errors() == before and int(flags[1][0]) == 4


def test_barrier_wait_is_bounded():
    """A flag nothing sets: the kernel gives up after its bound (about two seconds), counts the wait and returns; the
    context stays usable.  Runs in a child process, the counter is per process."""
    import subprocess
    import sys
    import os

    code = (
        "import time, torch\n"
        "from spiky_b200 import _native\n"
        "flags = [torch.zeros(16, dtype=torch.int64, device='cuda') for _ in range(2)]\n"
        "assert _native.device_wait_errors() == 0\n"
        "t0 = time.time()\n"
        "_native.peer_barrier(0, [f.data_ptr() for f in flags], 1, torch.cuda.current_stream().cuda_stream)\n"
        "torch.cuda.synchronize()\n"
        "dt = time.time() - t0\n"
        "assert _native.device_wait_errors() == 1, _native.device_wait_errors()\n"
        "assert 0.5 < dt < 20, dt\n"
        "x = torch.ones(8, device='cuda') * 2\n"
        "assert float(x.sum()) == 16.0\n"
        "print('bounded', round(dt, 2))\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "bounded" in out.stdout


@pytest.mark.parametrize("nbytes,src_shift,dst_offset", [(4096, 0, 0), (100003, 0, 32), (1 << 20, 16, 4096), (77, 5, 5),
                                                         (3000, 3, 16), (9, 0, 0)])
def test_broadcast_copies_bytes_into_every_buffer(nbytes, src_shift, dst_offset):
    """Three emulated ranks on one device: the byte range lands at the offset in every buffer and nowhere else; source
    and destinations aligned alike (fast path) or not (byte path)."""
    from spiky_b200 import _native

    rng = np.random.default_rng(nbytes)
    payload = rng.integers(0, 256, nbytes, dtype=np.uint8)
    src = torch.zeros(nbytes + 64, dtype=torch.uint8, device="cuda")
    src[src_shift:src_shift + nbytes] = torch.from_numpy(payload).cuda()
    dst = [torch.full((dst_offset + nbytes + 64,), 0xAB, dtype=torch.uint8, device="cuda") for _ in range(3)]
    _native.peer_broadcast([d.data_ptr() for d in dst], dst_offset, src.data_ptr() + src_shift, nbytes,
                           torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    for d in dst:
        got = d.cpu().numpy()
        assert np.array_equal(got[dst_offset:dst_offset + nbytes], payload)
        assert (got[:dst_offset] == 0xAB).all() and (got[dst_offset + nbytes:] == 0xAB).all()


def test_barrier_counts_its_own_epochs():
    """Epoch 0: the kernel keeps the count in device memory behind the rank slots, so the identical launch can be
    repeated (CUDA-graph replay); one rank, three barriers."""
    from spiky_b200 import _native

    flags = torch.zeros(2 * _native.MAX_PEER_RANKS, dtype=torch.int64, device="cuda")
    before = _native.device_wait_errors()
    for _ in range(3):
        _native.peer_barrier(0, [flags.data_ptr()], 0, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert _native.device_wait_errors() == before
    assert int(flags[0]) == 3 and int(flags[_native.MAX_PEER_RANKS]) == 3
