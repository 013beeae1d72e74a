"""CUDA path of sparse (projection) LUT layers against the reference's golden vectors and the oracle."""
import numpy as np
import pytest
import torch

import golden_util
import synth
from cases import projection_inputs
from oracle import lut_oracle as orc

pytestmark = pytest.mark.gpu
REL = 1e-5


def run_layer(layer, x, dY, cfg_like, internal_lr=None):
    """forward_step (eval + train) and backward_step of a sparse layer on the GPU; numpy results."""
    B = x.shape[0]
    I, O, Nt = layer.n_inputs(), layer.n_outputs(), layer.n_detectors()
    xt = torch.from_numpy(x).view((B, 1) + tuple(layer.input_shape())).cuda()
    out = {}
    layer.eval()
    out["y_eval"] = layer.forward_step(xt).cpu().numpy().reshape(B, O)
    layer.train()
    y, idx, md, mk = layer.forward_step(xt)
    if internal_lr is not None:
        layer.set_external_learning_rate_hook(lambda w: internal_lr)
    dx, dw = layer.backward_step(xt, torch.from_numpy(dY).view((B, 1) + tuple(layer.output_shape())).cuda(), idx, md, mk)
    torch.cuda.synchronize()
    out.update(y=y.cpu().numpy().reshape(B, O), idx=idx.cpu().numpy().reshape(B, Nt),
               min_delta=md.cpu().numpy().reshape(B, Nt), min_k=mk.cpu().numpy().reshape(B, Nt),
               dX=dx.cpu().numpy().reshape(B, I))
    if internal_lr is not None:
        out["W_after"] = layer._weights.detach().cpu().numpy()
    else:
        out["dW"] = dw.cpu().numpy()
    return out


def compare(got, ref, int_mode):
    assert np.array_equal(got["idx"], ref["idx"]) and np.array_equal(got["min_k"], ref["min_k"])
    assert np.array_equal(got["min_delta"].view(np.int32), ref["min_delta"].view(np.int32))
    for k in ["y", "y_eval", "dX"] + (["W_after"] if "W_after" in ref else ["dW"]):
        if int_mode:
            assert np.array_equal(got[k], ref[k]), f"{k}: fixed-point results must be bit-exact"
        else:
            golden_util.assert_close(got[k], ref[k], REL, k)


@pytest.mark.parametrize("name", golden_util.names("proj_"))
def test_projection_layer_matches_reference_golden(name):
    from spiky_b200.lut_layer import ProjectionLUTLayer, SynapseMeta, GradientPolicy, GradientType

    cfg, ref = golden_util.load(name)
    internal = cfg.get("policy") == "internal"
    layer = ProjectionLUTLayer(
        cfg["in_shape"], cfg["out_shape"], cfg["Nc"], cfg["groups"], cfg["per_group"], cfg["receptive"],
        cfg["projection"], synapse_meta=SynapseMeta(learning_rate=cfg.get("lr_meta", 1.0), min_weight=-1.0, max_weight=1.0),
        weights_gradient_policy=GradientPolicy(GradientType.Internal if internal else GradientType.Dense),
        summation_dtype=torch.int32 if cfg.get("int_mode") else torch.float32,
        _int_rescaler=cfg.get("int_rescaler", 0.001), _forward_group_size=cfg.get("G", 32), random_seed=1, device="cuda:0")
    # adopt the reference-built structure, then its weights verbatim
    layer.load_structure(ref["anchors"], ref["syn_source"], ref["syn_slot"], ref["syn_target"], cfg["n_weights"])
    x, W, dY = projection_inputs(cfg, cfg["n_weights"])
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
    got = run_layer(layer, x, dY, cfg, cfg["ext_lr"] if internal else None)
    compare(got, ref, cfg.get("int_mode", False))


@pytest.mark.parametrize("int_mode", [False, True])
def test_own_projection_layer_matches_oracle(int_mode):
    """A layer shaped like the first layer of the sparse conv-net configuration (28x28 -> 24x24, 5x5 receptive
    fields on a stride-2 grid, 4x4 projections, 256-row tables), built without the reference."""
    from spiky_b200.lut_layer import ProjectionLUTLayer, SynapseMeta, PointSamplingPolicy, PointSamplingType

    layer = ProjectionLUTLayer(
        (28, 28), (24, 24), 8, 144, 8, (5, 5), (4, 4),
        synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.1, initial_weight=-0.05),
        detectors_sampling_policy=PointSamplingPolicy(PointSamplingType.Grid, grid_h=12, grid_w=12, stride_h=2,
                                                      stride_w=2, pad_h=2, pad_w=2),
        summation_dtype=torch.int32 if int_mode else torch.float32, _int_rescaler=0.01, random_seed=3, device="cuda:0")
    B = 24
    x = synth.sparse_images(5, (B, 28 * 28))
    dY = synth.normal(6, (B, 24 * 24))
    got = run_layer(layer, x, dY, None)
    index = layer._lut_dm._sparse
    sp = dict(index.numpy(), group_size=index.group_size)
    W = layer._weights.detach().cpu().numpy()
    anchors = layer._detector_anchors.cpu().numpy()
    kw = dict(int_mode=int_mode, int_rescaler=0.01)
    y, idx, md, mk = orc.nonseq_sparse_forward(W, x, anchors, sp, 8, 24 * 24, **kw)
    dX, dW = orc.nonseq_sparse_backward(W, dY, anchors, idx, md, mk, sp, 28 * 28, 8, **kw)
    compare(got, dict(y=y, y_eval=y, idx=idx, min_delta=md, min_k=mk, dX=dX, dW=dW), int_mode)
    # header holes of the flat weight array never receive gradient
    assert not got["dW"][~index.slot_mask().cpu().numpy()].any()


def test_projection_autograd_and_sgd_step():
    from spiky_b200.lut_layer import ProjectionLUTLayer, SynapseMeta

    layer = ProjectionLUTLayer((16, 16), (12, 12), 4, 10, 4, (5, 5), (3, 3),
                               synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.2,
                                                        initial_weight=-0.1), random_seed=2, device="cuda:0")
    opt = torch.optim.SGD(layer.parameters(), lr=0.1)
    x = torch.rand(8, 1, 16, 16, device="cuda:0", requires_grad=True)
    y = layer(x)
    assert y.shape == (8, 1, 12, 12)
    loss = (y ** 2).sum()
    loss.backward()
    assert x.grad is not None and layer._weights.grad is not None
    before = layer._weights.detach().clone()
    opt.step()
    assert not torch.equal(before, layer._weights.detach())


@pytest.mark.parametrize("per_group,projection,batch", [(40, (3, 3), 9), (1, (4, 4), 130), (33, (2, 2), 7), (5, (6, 6), 6)])
def test_chunk_shapes_match_oracle(per_group, projection, batch):
    """Detector groups that do not fill a 32-detector chunk, spill into a second chunk, or hold a single detector;
    batches that are not a multiple of the per-warp sample run; rows of 4 to 36 synapses."""
    from spiky_b200.lut_layer import ProjectionLUTLayer, SynapseMeta

    layer = ProjectionLUTLayer(
        (14, 14), (12, 12), 5, 6, per_group, (5, 5), projection,
        synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.1, initial_weight=0.02),
        random_seed=7, device="cuda:0")
    x = synth.sparse_images(15, (batch, 14 * 14))
    dY = synth.normal(16, (batch, 12 * 12))
    got = run_layer(layer, x, dY, None)
    index = layer._lut_dm._sparse
    sp = dict(index.numpy(), group_size=index.group_size)
    W = layer._weights.detach().cpu().numpy()
    anchors = layer._detector_anchors.cpu().numpy()
    y, idx, md, mk = orc.nonseq_sparse_forward(W, x, anchors, sp, 5, 12 * 12)
    dX, dW = orc.nonseq_sparse_backward(W, dY, anchors, idx, md, mk, sp, 14 * 14, 5)
    compare(got, dict(y=y, y_eval=y, idx=idx, min_delta=md, min_k=mk, dX=dX, dW=dW), False)


@pytest.mark.parametrize("kind", ["sparse", "fc", "sparse_int"])
def test_input_gradient_is_skipped_when_not_needed(kind):
    """A layer whose input needs no gradient (first layer of a network) skips the input-gradient kernels: the table
    gradient is unchanged, autograd returns no gradient for the input."""
    from spiky_b200.lut_layer import LUTLayer, ProjectionLUTLayer, SynapseMeta

    meta = SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.2, initial_weight=-0.1)
    if kind == "fc":
        layer = LUTLayer(64, 5, 12, 16, synapse_meta=meta, random_seed=2, device="cuda:0")
        x = torch.rand(9, 1, 64, device="cuda:0")
    else:
        layer = ProjectionLUTLayer((16, 16), (12, 12), 4, 10, 4, (5, 5), (3, 3), synapse_meta=meta, random_seed=2,
                                   summation_dtype=torch.int32 if kind == "sparse_int" else torch.float32,
                                   _int_rescaler=0.01, device="cuda:0")
        x = torch.rand(9, 1, 16, 16, device="cuda:0")
    layer.train()
    y, idx, md, mk = layer.forward_step(x)
    dY = torch.randn_like(y)
    dx, dw = layer.backward_step(x, dY, idx, md, mk)
    none, dw2 = layer.backward_step(x, dY, idx, md, mk, need_input_grad=False)
    assert none is None and dx is not None and dx.abs().sum() > 0
    if kind == "sparse_int":
        assert torch.equal(dw, dw2)
    else:
        golden_util.assert_close(dw2.cpu().numpy(), dw.cpu().numpy(), 1e-6, "dW")
    # through autograd: input without requires_grad
    layer.zero_grad()
    out = layer(x)
    (out * dY).sum().backward()
    assert x.grad is None
    golden_util.assert_close(layer._weights.grad.cpu().numpy(), dw.cpu().numpy(), 1e-6, "dW via autograd")
    xg = x.clone().requires_grad_(True)
    layer.zero_grad()
    (layer(xg) * dY).sum().backward()
    golden_util.assert_close(xg.grad.cpu().numpy(), dx.cpu().numpy(), 1e-6, "dX via autograd")


@pytest.mark.parametrize("idx_dtype", [torch.uint8, torch.int16, torch.int32])
def test_ranged_table_gradient_matches_backward(idx_dtype):
    """The table-gradient pass alone, run over two chunk ranges and fed with narrow table indices, reproduces the dense
    table gradient of the full backward; the input-gradient-only call leaves the tables' gradient out."""
    from spiky_b200 import _native
    from spiky_b200.lut_layer import ProjectionLUTLayer, SynapseMeta

    meta = SynapseMeta(learning_rate=0.5, min_weight=-1.0, max_weight=1.0, initial_noise_level=0.2, initial_weight=-0.1)
    layer = ProjectionLUTLayer((16, 16), (12, 12), 5, 10, 40, (5, 5), (3, 3), synapse_meta=meta, random_seed=2,
                               device="cuda:0")
    layer.train()
    B = 37
    x = torch.rand(B, 1, 16, 16, device="cuda:0")
    y, idx, md, mk = layer.forward_step(x)
    dY = torch.randn_like(y)
    dx, dw = layer.backward_step(x, dY, idx, md, mk)
    dm, index = layer._lut_dm, layer._lut_dm._sparse
    assert index.n_chunks >= 4
    cut = index.n_chunks // 3
    target = torch.zeros_like(dw)
    narrow = idx.reshape(-1).to(idx_dtype)
    flat = dY.contiguous().view(-1)
    dm.table_gradient(B, flat, narrow, target, 1.0, 0, cut)
    bounds = index.chunk_weight_bounds()
    assert not target[int(bounds[cut]):].any() and target[:int(bounds[cut])].any()
    dm.table_gradient(B, flat, narrow, target, 1.0, cut, index.n_chunks)
    dm.table_gradient(B, flat, narrow, target, 1.0, cut, cut)  # empty range: nothing happens
    golden_util.assert_close(target.cpu().numpy(), dw.cpu().numpy(), 1e-6, "dW from two ranges")
    # input gradient only
    dx2 = torch.zeros(x.numel(), device="cuda:0")
    dm.backward_backprop(layer._weights.detach(), B, flat, layer._detector_anchors, idx.reshape(-1), md.reshape(-1),
                         mk.reshape(-1), dx2, _native.SKIP_TABLE_GRADIENT, None, None)
    golden_util.assert_close(dx2.cpu().numpy(), dx.reshape(-1).cpu().numpy(), 1e-6, "dX alone")
    with pytest.raises(ValueError):
        dm.table_gradient(B, flat, narrow, target, 1.0, 0, index.n_chunks + 1)


def test_sharded_table_update_on_one_rank_equals_in_place_sgd():
    """Without a process group the sharded update degenerates to in-place SGD on all chunks: same tables afterwards
    as the Internal gradient policy, and no gradient on the parameter."""
    from spiky_b200.data_parallel import ShardedTableUpdate
    from spiky_b200.lut_layer import GradientPolicy, GradientType, ProjectionLUTLayer, SynapseMeta

    meta = SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.2, initial_weight=-0.1)
    kw = dict(synapse_meta=meta, random_seed=2, device="cuda:0")
    a = ProjectionLUTLayer((16, 16), (12, 12), 4, 10, 4, (5, 5), (3, 3), **kw)
    b = ProjectionLUTLayer((16, 16), (12, 12), 4, 10, 4, (5, 5), (3, 3),
                           weights_gradient_policy=GradientPolicy(GradientType.Internal), **kw)
    assert torch.equal(a._weights, b._weights) and torch.equal(a._detector_anchors, b._detector_anchors)
    b.set_external_learning_rate_hook(lambda w: 0.05)
    sync = ShardedTableUpdate([a], 0.05)
    x = torch.rand(12, 1, 16, 16, device="cuda:0", requires_grad=True)
    g = torch.randn(12, 1, 12, 12, device="cuda:0")
    grads = []
    for layer in (a, b):
        layer.train()
        xin = x.detach().clone().requires_grad_(True)
        (layer(xin) * g).sum().backward()
        grads.append(xin.grad)
    sync.wait()
    torch.cuda.synchronize()
    assert a._weights.grad is None
    golden_util.assert_close(grads[0].cpu().numpy(), grads[1].cpu().numpy(), 1e-6, "dX")
    golden_util.assert_close(a._weights.detach().cpu().numpy(), b._weights.detach().cpu().numpy(), 1e-6, "tables")
    sync.remove()
    assert not hasattr(a, "_table_update_hook")
