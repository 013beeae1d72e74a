"""LUTTransformer (product-mode attention) forward + backward on the GPU against a CPU composition of the
oracle's layer functions: embedding -> [attention + residual, FFN + residual] x L -> unembedder."""
import numpy as np
import pytest
import torch

import golden_util
from oracle import lut_oracle as orc

pytestmark = pytest.mark.gpu


def oracle_transformer(model, tokens, dlogits):
    """Forward and manual backward with the oracle; returns logits and {layer name: dW}."""
    B, S = tokens.shape
    E, V = model._n_embeddings, model.vocab_size
    emb = model.token_embedder.weight.detach().cpu().numpy()
    z = emb[tokens]
    tape = []
    for bi, block in enumerate(model.layers):
        att = block["attention_lut"]
        A = att._detector_anchors.cpu().numpy()
        W = att._weights.detach().cpu().numpy()
        pe = att._prepare_positional_embeddings().detach().cpu().numpy().reshape(S - 1, att._n_detectors, -1)
        y = orc.product_forward(W, z, pe, A, att._n_detectors, att._n_anchors_per_detector, E, att._positional_dim)
        tape.append(("att", bi, z.copy(), (W, pe, A, att)))
        z = z + y
        ffn = block["ffn"]
        A2 = ffn._detector_anchors.cpu().numpy()
        W2 = ffn._weights.detach().cpu().numpy()
        y2, idx, md, mk = orc.nonseq_fc_forward(W2, z.reshape(B * S, E), A2, ffn._n_detectors, ffn._n_anchors_per_detector, E)
        tape.append(("ffn", bi, z.copy(), (W2, A2, idx, md, mk, ffn)))
        z = z + y2.reshape(B, S, E)
    un = model.unembedder
    Au, Wu = un._detector_anchors.cpu().numpy(), un._weights.detach().cpu().numpy()
    logits, idx, md, mk = orc.nonseq_fc_forward(Wu, z.reshape(B * S, E), Au, un._n_detectors, un._n_anchors_per_detector, V)
    grads = {}
    dz, grads["unembedder"] = orc.nonseq_fc_backward(Wu, dlogits.reshape(B * S, V), Au, idx, md, mk, E, un._n_anchors_per_detector)
    dz = dz.reshape(B, S, E)
    for kind, bi, zin, info in reversed(tape):
        if kind == "ffn":
            W2, A2, idx, md, mk, ffn = info
            dx, dw = orc.nonseq_fc_backward(W2, dz.reshape(B * S, E), A2, idx, md, mk, E, ffn._n_anchors_per_detector)
            grads[f"ffn{bi}"] = dw
            dz = dz + dx.reshape(B, S, E)
        else:
            W, pe, A, att = info
            dx, dw, dpe = orc.product_backward(W, zin, pe, A, dz, att._n_detectors, att._n_anchors_per_detector, att._positional_dim)
            grads[f"att{bi}"] = dw
            grads[f"pe{bi}"] = dpe
            dz = dz + dx
    return logits.reshape(B, S, V), grads


def test_product_transformer_matches_oracle_composition():
    from spiky_b200.lut_transformer import LUTTransformer
    from spiky_b200.lut_layer import SynapseMeta

    torch.manual_seed(0)
    V, E, S, B = 65, 32, 16, 3
    model = LUTTransformer(V, E, S, positional_dim=4, num_layers=2, num_heads=2, n_detectors=4,
                           n_anchors_per_detector=5, concatenation_product=False, seed=7, device="cuda:0",
                           synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.2,
                                                    initial_weight=-0.1))
    model.train()
    tokens = torch.randint(0, V, (B, S))
    dlogits = torch.randn(B, S, V)
    logits = model(tokens.cuda())
    logits.backward(dlogits.cuda())
    ref_logits, ref_grads = oracle_transformer(model, tokens.numpy(), dlogits.numpy())
    golden_util.assert_close(logits.detach().cpu().numpy(), ref_logits, 1e-5, "logits")
    golden_util.assert_close(model.unembedder._weights.grad.cpu().numpy(), ref_grads["unembedder"], 1e-5, "unembedder dW")
    for bi, block in enumerate(model.layers):
        golden_util.assert_close(block["ffn"]._weights.grad.cpu().numpy(), ref_grads[f"ffn{bi}"], 2e-5, f"ffn{bi} dW")
        golden_util.assert_close(block["attention_lut"]._weights.grad.cpu().numpy(), ref_grads[f"att{bi}"], 2e-5, f"att{bi} dW")
        golden_util.assert_close(block["attention_lut"]._positional_embeddings.grad.cpu().numpy(), ref_grads[f"pe{bi}"], 2e-5, f"pe{bi}")


@pytest.mark.parametrize("concat", [True, False])
def test_transformer_trains_one_step(concat):
    from spiky_b200.lut_transformer import LUTTransformer
    from spiky_b200.lut_layer import SynapseMeta, GradientPolicy, GradientType

    model = LUTTransformer(50, 16, 8, positional_dim=2, num_layers=1, num_heads=2, n_detectors=3,
                           n_anchors_per_detector=3, concatenation_product=concat, seed=1, device="cuda:0",
                           weights_gradient_policy=GradientPolicy(GradientType.Dense),
                           synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.2, initial_weight=-0.1))
    opt = torch.optim.SGD([p for p in model.parameters() if p.requires_grad], lr=0.1)
    tokens = torch.randint(0, 50, (4, 9), device="cuda:0")
    losses = []
    for _ in range(3):
        opt.zero_grad()
        logits = model(tokens[:, :-1])
        loss = torch.nn.functional.cross_entropy(logits.reshape(-1, 50), tokens[:, 1:].reshape(-1))
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert np.isfinite(losses).all() and losses[-1] < losses[0]
