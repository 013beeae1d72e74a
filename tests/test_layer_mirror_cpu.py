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
    # Sparse: the compaction runs in the CUDA library; stand in for it with the same contract (sorted cells, erased
    # buffer) so that the layer's handling of the converter's result is what is tested
    class HostConverter:
        def dense_to_sparse_32(self, buf, erase_input=True):
            cells = torch.nonzero(buf.view(torch.int32) != 0).flatten()
            if cells.numel() == 0:
                return None, None
            values = buf[cells].clone()
            if erase_input:
                buf.zero_()
            return cells, values

    layer = make(GradientType.Sparse)
    with torch.no_grad():
        layer._weights.copy_(dense._weights)
    ctx.__dict__.setdefault("_dense_to_sparse_converters", {})[layer._multi_id] = HostConverter()
    xs = x.clone().requires_grad_(True)
    (layer(xs) * g).sum().backward()
    grad = layer._weights.grad
    assert grad.is_sparse and grad._nnz() == int((want != 0).sum())
    assert torch.equal(grad.to_dense(), want)
    assert not ctx.get_weight_gradients_buffer(want.numel(), torch.device("cpu"), layer._multi_id).any()
    assert torch_utils.DenseToSparseConverter is not None
