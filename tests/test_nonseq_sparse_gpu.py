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
