"""LUTTransformer against whole models built and run by the reference (fixtures: every parameter and anchor of the
reference model, tokens, logits, gradients of all parameters).  On CPU the layers' runtime calls are served by the
oracle (tests/oracle_backend.py), which pins the Python side - block wiring, residuals, positional embedding handling,
autograd plumbing - without a GPU; on a GPU the same fixtures go through the CUDA library."""
import numpy as np
import pytest
import torch

import golden_util
from cases import transformer_inputs


def build(cfg, ref, device):
    from spiky_b200.lut_layer import GradientPolicy, GradientType, SynapseMeta
    from spiky_b200.lut_transformer import LUTTransformer

    int_mode = cfg.get("int_mode", False)
    model = LUTTransformer(
        vocab_size=cfg["V"], embedding_dim=cfg["E"] if isinstance(cfg["E"], int) else tuple(cfg["E"]),
        context_size=cfg["S"], positional_dim=cfg["Npe"], use_batch_norm=cfg.get("batch_norm", False),
        num_layers=cfg["layers"], num_heads=cfg["heads"], n_detectors=cfg["Nt"], n_anchors_per_detector=cfg["Nc"],
        n_anchors_per_detector_attention=cfg.get("Nc_att"), no_ffn=cfg.get("no_ffn", False),
        concatenation_product=cfg["concat"], unified_pe=cfg.get("unified_pe", False),
        weights_gradient_policy=GradientPolicy(GradientType.Dense), device=device,
        synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.4, initial_weight=-0.2),
        seed=cfg["seed"], summation_dtype=torch.int32 if int_mode else torch.float32,
        _int_rescaler=cfg.get("int_rescaler", 0.001))
    layers = {}
    for li, block in enumerate(model.layers):
        layers[f"att{li}"] = block["attention_lut"]
        if not cfg.get("no_ffn", False):
            layers[f"ffn{li}"] = block["ffn"]
    layers["unembedder"] = model.unembedder
    with torch.no_grad():
        model.token_embedder.weight.copy_(torch.from_numpy(ref["embedding"]))
        for prefix, layer in layers.items():
            layer._set_anchors(torch.from_numpy(ref[prefix + "_anchors"]))
            layer._weights.copy_(torch.from_numpy(ref[prefix + "_W"]))
            if prefix + "_pe" in ref:
                layer._positional_embeddings.copy_(torch.from_numpy(ref[prefix + "_pe"]).view_as(layer._positional_embeddings))
    model.train()
    return model, layers


def check(cfg, ref, model, layers, device, rel=1e-5):
    tokens, dlogits = transformer_inputs(cfg)
    logits = model(torch.from_numpy(tokens).to(device))
    logits.backward(torch.from_numpy(dlogits).to(device))
    int_mode = cfg.get("int_mode", False)

    def same(got, want, what):
        got = got.detach().cpu().numpy().reshape(-1)
        want = want.reshape(-1)
        if int_mode:
            assert np.array_equal(got, want), f"{what}: fixed-point results must be bit-exact"
        else:
            golden_util.assert_close(got, want, rel, what)

    same(logits, ref["logits"], "logits")
    if cfg.get("batch_norm", False):
        for li, block in enumerate(model.layers):
            for branch in ("attention", "ffn"):
                same(block[branch + "_bn"].weight.grad, ref[f"{branch}{li}_bn_dweight"], f"{branch}{li} bn dweight")
                same(block[branch + "_bn"].bias.grad, ref[f"{branch}{li}_bn_dbias"], f"{branch}{li} bn dbias")
    for prefix, layer in layers.items():
        same(layer._weights.grad, ref[prefix + "_dW"], prefix + " dW")
        if prefix + "_dpe" in ref:
            same(layer._positional_embeddings.grad, ref[prefix + "_dpe"], prefix + " dPE")


@pytest.mark.parametrize("name", golden_util.names("transformer_"))
def test_transformer_wiring_matches_reference_on_cpu(name):
    from oracle_backend import use_oracle_backend

    cfg, ref = golden_util.load(name)
    model, layers = build(cfg, ref, None)
    use_oracle_backend(model)
    check(cfg, ref, model, layers, torch.device("cpu"))


@pytest.mark.gpu
@pytest.mark.parametrize("name", golden_util.names("transformer_"))
def test_transformer_matches_reference_golden(name):
    cfg, ref = golden_util.load(name)
    model, layers = build(cfg, ref, "cuda:0")
    # gradients pass through up to five layers whose fp32 sums run in another order than the reference's
    check(cfg, ref, model, layers, torch.device("cuda:0"), rel=2e-5)
