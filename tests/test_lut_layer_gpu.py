"""Layer API (LUTLayer through torch.autograd) on the GPU against the CPU oracle."""
import numpy as np
import pytest
import torch

import golden_util
import synth
from oracle import lut_oracle as orc

pytestmark = pytest.mark.gpu


def build_layer(I, Nc, Nt, O, anchors, W, policy=None, summation_dtype=torch.float32, **kw):
    from spiky_b200.lut_layer import LUTLayer, SynapseMeta

    layer = LUTLayer(I, Nc, Nt, O, synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
                     weights_gradient_policy=policy, summation_dtype=summation_dtype,
                     _explicit_anchors=torch.from_numpy(anchors.reshape(-1)), device="cuda:0", **kw)
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
    return layer


@pytest.mark.parametrize("policy_name", ["dense", "sparse", "internal"])
def test_autograd_matches_oracle(policy_name):
    from spiky_b200.lut_layer import GradientPolicy, GradientType

    B, I, Nt, Nc, O = 37, 100, 24, 5, 16
    x = synth.uniform(1, (B, I))
    anchors = synth.anchor_pairs(2, Nt, Nc, I)
    W = synth.normal(3, (Nt * (1 << Nc) * O,), 0.0, 0.02)
    dY = synth.normal(4, (B, O))
    policy = {"dense": GradientType.Dense, "sparse": GradientType.Sparse, "internal": GradientType.Internal}[policy_name]
    layer = build_layer(I, Nc, Nt, O, anchors, W, GradientPolicy(policy))
    if policy == GradientType.Internal:
        layer.set_external_learning_rate_hook(lambda w: 0.1)
    layer.train()
    xt = torch.from_numpy(x).view(B, 1, I).cuda().requires_grad_(True)
    y = layer(xt)
    y.backward(torch.from_numpy(dY).view(B, 1, O).cuda())
    ry, ridx, rmd, rmk = orc.nonseq_fc_forward(W, x, anchors, Nt, Nc, O)
    Wc = W.copy()
    rdX, rdW = orc.nonseq_fc_backward(Wc, dY, anchors, ridx, rmd, rmk, I, Nc,
                                      external_lr=0.1 if policy == GradientType.Internal else -1.0)
    golden_util.assert_close(y.detach().cpu().numpy().reshape(B, O), ry, 1e-5, "y")
    golden_util.assert_close(xt.grad.cpu().numpy().reshape(B, I), rdX, 1e-5, "dX")
    if policy == GradientType.Internal:
        assert layer._weights.grad is None
        golden_util.assert_close(layer._weights.detach().cpu().numpy(), Wc, 1e-5, "W after internal update")
    else:
        g = layer._weights.grad
        if policy == GradientType.Sparse:
            assert g.is_sparse
            g = g.to_dense()
        golden_util.assert_close(g.cpu().numpy(), rdW, 1e-5, "dW")
    if policy == GradientType.Internal:
        return  # the tables have just been updated in place
    # eval mode gives the same outputs and keeps no graph
    layer.eval()
    with torch.no_grad():
        ye = layer(xt.detach())
    golden_util.assert_close(ye.cpu().numpy().reshape(B, O), ry, 1e-5, "y eval")


def test_indices_callback_and_int_mode():
    B, I, Nt, Nc, O = 16, 64, 8, 4, 12
    x = synth.uniform(11, (B, I))
    anchors = synth.anchor_pairs(12, Nt, Nc, I)
    W = synth.normal(13, (Nt * (1 << Nc) * O,), 0.0, 0.02)
    layer = build_layer(I, Nc, Nt, O, anchors, W, summation_dtype=torch.int32, _int_rescaler=1.0)
    seen = {}
    layer._set_lookup_indices_callback(lambda idx, md, mk: seen.update(idx=idx.clone()))
    layer.train()
    y = layer(torch.from_numpy(x).view(B, 1, I).cuda())
    ry, ridx, _, _ = orc.nonseq_fc_forward(W, x, anchors, Nt, Nc, O, int_mode=True, int_rescaler=1.0)
    assert np.array_equal(seen["idx"].cpu().numpy().reshape(B, Nt), ridx)
    assert np.array_equal(y.detach().cpu().numpy().reshape(B, O), ry)


def test_state_dict_round_trip():
    from spiky_b200.lut_layer import LUTLayer

    a = LUTLayer(32, 4, 6, 8, random_seed=5, device="cuda:0")
    b = LUTLayer(32, 4, 6, 8, random_seed=9, device="cuda:0")
    b.load_state_dict(a.state_dict())
    assert torch.equal(a._detector_anchors, b._detector_anchors) and torch.equal(a._weights, b._weights)
    x = torch.rand(3, 1, 32, device="cuda:0")
    a.eval(); b.eval()
    assert torch.equal(a(x), b(x))
