"""The Python layer mirror (spiky_b200.lut_layer) on CPU against the reference's fixtures, with the runtime calls served
by the oracle (tests/oracle_backend.py): what the GPU tests check through the CUDA library is checked here for the host
side alone - tensor shapes and views, positional-embedding preparation, gradient policies, in-place SGD plumbing."""
import numpy as np
import pytest
import torch

import golden_util
import test_concat_gpu as concat_t
import test_product_gpu as product_t
from oracle_backend import OracleDataManager, use_oracle_backend


@pytest.mark.parametrize("name", golden_util.names("concat_"))
def test_concat_layer_on_cpu_matches_reference(name):
    cfg, ref = golden_util.load(name)
    x, anchors, W, pe, dY = concat_t.inputs_for(cfg)
    got = concat_t.run_gpu(cfg, x, anchors, W, pe, dY, device=None, prepare=use_oracle_backend)
    concat_t.compare(cfg, got, ref)


@pytest.mark.parametrize("name", golden_util.names("prod_"))
def test_product_layer_on_cpu_matches_reference(name):
    cfg, ref = golden_util.load(name)
    x, anchors, W, pe, dY = product_t.inputs_for(cfg)
    got = product_t.run_gpu(cfg, x, anchors, W, pe, dY, device=None, prepare=use_oracle_backend)
    product_t.compare(cfg, got, ref)


@pytest.mark.parametrize("policy_name", ["Dense", "Sparse", "Internal"])
def test_gradient_policies_through_autograd_on_cpu(policy_name):
    """The three weight-gradient policies of a fully connected layer: Dense and Sparse hand the same gradient to the
    optimiser (Sparse as a coalesced COO tensor of the touched cells), Internal applies it inside the backward call."""
    from spiky_b200.lut_layer import GradientPolicy, GradientType, LUTLayer, LUTSharedContext, SynapseMeta
    from spiky_b200 import torch_utils

    meta = SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.3, initial_weight=-0.15)
    ctx = LUTSharedContext().to_device("cpu")

    def make(policy):
        layer = LUTLayer(20, 4, 5, 6, synapse_meta=meta, weights_gradient_policy=GradientPolicy(policy),
                         shared_context=ctx, random_seed=3, device=None)
        use_oracle_backend(layer)
        layer.train()
        return layer

    dense = make(GradientType.Dense)
    x = torch.rand(7, 1, 20)
    g = torch.randn(7, 1, 6)
    xd = x.clone().requires_grad_(True)
    (dense(xd) * g).sum().backward()
    want = dense._weights.grad.clone()
    assert want.abs().sum() > 0
    if policy_name == "Dense":
        assert isinstance(dense._lut_dm, OracleDataManager) and xd.grad.shape == x.shape
        return
    if policy_name == "Internal":
        layer = make(GradientType.Internal)
        layer.set_external_learning_rate_hook(lambda w: 0.5)
        with torch.no_grad():
            layer._weights.copy_(dense._weights)
        before = layer._weights.detach().clone()
        xi = x.clone().requires_grad_(True)
        (layer(xi) * g).sum().backward()
        assert layer._weights.grad is None
        assert torch.allclose(layer._weights.detach(), before - 0.5 * want, atol=1e-6)
        assert torch.allclose(xi.grad, xd.grad, atol=1e-6)
        return
    # Sparse: the compaction runs in the CUDA library; _HostConverter stands in for it, so that the layer's handling of
    # the converter's result is what is tested
    layer = make(GradientType.Sparse)
    with torch.no_grad():
        layer._weights.copy_(dense._weights)
    ctx.__dict__.setdefault("_dense_to_sparse_converters", {})[layer._multi_id] = _HostConverter()
    xs = x.clone().requires_grad_(True)
    (layer(xs) * g).sum().backward()
    grad = layer._weights.grad
    assert grad.is_sparse and grad._nnz() == int((want != 0).sum())
    assert torch.equal(grad.to_dense(), want)
    assert not ctx.get_weight_gradients_buffer(want.numel(), torch.device("cpu"), layer._multi_id).any()
    assert torch_utils.DenseToSparseConverter is not None


def _run_nonseq_layer(layer, x, dY, internal_lr=None):
    """forward_step (eval + train) and backward_step of a non-sequence layer on CPU tensors; numpy results."""
    B = x.shape[0]
    I, O, Nt = layer.n_inputs(), layer.n_outputs(), layer.n_detectors()
    xt = torch.from_numpy(x).view((B, 1) + tuple(layer.input_shape()))
    out = {}
    layer.eval()
    out["y_eval"] = layer.forward_step(xt).numpy().reshape(B, O)
    layer.train()
    y, idx, md, mk = layer.forward_step(xt)
    if internal_lr is not None:
        layer.set_external_learning_rate_hook(lambda w: internal_lr)
    dx, dw = layer.backward_step(xt, torch.from_numpy(dY).view((B, 1) + tuple(layer.output_shape())), idx, md, mk)
    out.update(y=y.numpy().reshape(B, O), idx=idx.numpy().reshape(B, Nt), min_delta=md.numpy().reshape(B, Nt),
               min_k=mk.numpy().reshape(B, Nt), dX=dx.numpy().reshape(B, I))
    if internal_lr is not None:
        out["W_after"] = layer._weights.detach().numpy()
    else:
        out["dW"] = dw.numpy()
    return out


def _compare_nonseq(got, ref, int_mode):
    assert np.array_equal(got["idx"], ref["idx"]) and np.array_equal(got["min_k"], ref["min_k"])
    assert np.array_equal(got["min_delta"].view(np.int32), ref["min_delta"].view(np.int32))
    for k in ["y", "y_eval", "dX"] + (["W_after"] if "W_after" in ref else ["dW"]):
        if k not in ref:
            continue
        if int_mode:
            assert np.array_equal(got[k], ref[k]), f"{k}: fixed-point results must be bit-exact"
        else:
            golden_util.assert_close(got[k], ref[k], 1e-5, k)


@pytest.mark.parametrize("name", golden_util.names("proj_"))
def test_projection_layer_on_cpu_matches_reference(name):
    from cases import projection_inputs
    from spiky_b200.lut_layer import GradientPolicy, GradientType, ProjectionLUTLayer, SynapseMeta

    cfg, ref = golden_util.load(name)
    internal = cfg.get("policy") == "internal"
    layer = ProjectionLUTLayer(
        cfg["in_shape"], cfg["out_shape"], cfg["Nc"], cfg["groups"], cfg["per_group"], cfg["receptive"],
        cfg["projection"], synapse_meta=SynapseMeta(learning_rate=cfg.get("lr_meta", 1.0), min_weight=-1.0, max_weight=1.0),
        weights_gradient_policy=GradientPolicy(GradientType.Internal if internal else GradientType.Dense),
        summation_dtype=torch.int32 if cfg.get("int_mode") else torch.float32,
        _int_rescaler=cfg.get("int_rescaler", 0.001), _forward_group_size=cfg.get("G", 32), random_seed=1, device=None)
    layer.load_structure(ref["anchors"], ref["syn_source"], ref["syn_slot"], ref["syn_target"], cfg["n_weights"])
    use_oracle_backend(layer)
    x, W, dY = projection_inputs(cfg, cfg["n_weights"])
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
    got = _run_nonseq_layer(layer, x, dY, cfg["ext_lr"] if internal else None)
    _compare_nonseq(got, ref, cfg.get("int_mode", False))


@pytest.mark.parametrize("name", golden_util.names("conv2d_"))
def test_conv2d_layer_on_cpu_matches_reference(name):
    from cases import conv2d_inputs
    from test_conv2d_structure import _cpu_layer

    cfg, ref = golden_util.load(name)
    layer = _cpu_layer(cfg)
    if cfg["lut_rf"] is not None:
        layer.load_structure(ref["anchors"], ref["syn_source"], ref["syn_slot"], ref["syn_target"], cfg["n_weights"])
    else:
        layer._set_anchors(torch.from_numpy(ref["anchors"]))
    use_oracle_backend(layer)
    x, W, dY = conv2d_inputs(cfg, cfg["n_weights"], cfg["O"])
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
    got = _run_nonseq_layer(layer, x, dY)
    _compare_nonseq(got, ref, cfg.get("int_mode", False))


class _HostConverter:
    """Stand-in for the CUDA compaction of the Sparse policy with the same contract: sorted non-zero cells, their
    values, the source buffer erased."""

    def dense_to_sparse_32(self, buf, erase_input=False):
        cells = torch.nonzero(buf.view(torch.int32) != 0).flatten()
        if cells.numel() == 0:
            return None, None
        values = buf[cells].clone()
        if erase_input:
            buf.zero_()
        return cells, values


@pytest.mark.parametrize("concat", [True, False])
def test_training_steps_agree_across_gradient_policies(concat):
    """A small LUTTransformer trained for a few SGD steps ends with the same tables and embeddings whether the table
    gradients leave the layers dense, as sparse COO tensors, or are applied inside the backward call (the matrix the
    reference's test_lut_transformer_small.py runs against its pure-Python model)."""
    from spiky_b200.lut_layer import GradientPolicy, GradientType, LUTSharedContext, SynapseMeta
    from spiky_b200.lut_transformer import LUTTransformer

    lr, steps, V, S = 0.05, 4, 17, 6
    meta = SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.4, initial_weight=-0.2)
    gen = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, V, (steps, 3, S + 1), generator=gen)

    def train(policy):
        ctx = LUTSharedContext().to_device("cpu")
        ctx.__dict__["_dense_to_sparse_converters"] = {0: _HostConverter()}
        model = LUTTransformer(V, 12, S, positional_dim=2, num_layers=2, num_heads=2, n_detectors=2,
                               n_anchors_per_detector=3, concatenation_product=concat, seed=11, device=None,
                               weights_gradient_policy=GradientPolicy(policy), synapse_meta=meta,
                               lut_shared_context=ctx)
        use_oracle_backend(model)
        model.train()
        return model

    models = {p: train(p) for p in (GradientType.Dense, GradientType.Sparse, GradientType.Internal)}
    first = models[GradientType.Dense]
    for m in models.values():  # initial noise comes from the global generator: start from identical parameters
        m.load_state_dict(first.state_dict())
    start = {k: v.clone() for k, v in first.state_dict().items()}
    models[GradientType.Internal].set_external_learning_rate_hook(lambda w: lr)
    for policy, model in models.items():
        params = [p for p in model.parameters() if p.requires_grad]
        opt = torch.optim.SGD(params, lr=lr)
        for step in range(steps):
            opt.zero_grad(set_to_none=True)
            logits = model(tokens[step, :, :-1])
            loss = torch.nn.functional.cross_entropy(logits.reshape(-1, V), tokens[step, :, 1:].reshape(-1))
            loss.backward()
            if policy == GradientType.Sparse:
                assert any(p.grad is not None and p.grad.is_sparse for p in params)
            if policy == GradientType.Internal:
                assert all(layer._weights.grad is None for layer in model._lut_layers())
            opt.step()
    want = first.state_dict()
    assert any("_weights" in k and not torch.equal(v, start[k]) for k, v in want.items()), "training moved nothing"
    for policy in (GradientType.Sparse, GradientType.Internal):
        got = models[policy].state_dict()
        for key, value in want.items():
            if value.dtype.is_floating_point:
                assert torch.allclose(got[key], value, rtol=1e-4, atol=1e-6), f"{policy}: {key}"
            else:
                assert torch.equal(got[key], value), f"{policy}: {key}"
