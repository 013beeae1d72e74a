"""CUDA path of concatenation-mode sequence layers against the reference's golden vectors and the oracle."""
import numpy as np
import pytest
import torch

import golden_util
from cases import sequence_inputs
from oracle import lut_oracle as orc
from test_oracle_golden import expand_pe

pytestmark = pytest.mark.gpu
REL = 1e-5


def build_layer(cfg, anchors, W, pe, device="cuda:0"):
    from spiky_b200.lut_layer import LUTLayer, SynapseMeta, GradientPolicy, GradientType

    internal = cfg.get("policy") == "internal"
    layer = LUTLayer(
        cfg["E"], cfg["Nc"], cfg["Nt"], cfg["O"], sequence_length=cfg["S"],
        synapse_meta=SynapseMeta(learning_rate=cfg.get("lr_meta", 1.0), min_weight=-1.0, max_weight=1.0),
        concatenation_product=True, positional_dim=cfg["Npe"], unified_pe=cfg.get("unified_pe", False),
        weights_gradient_policy=GradientPolicy(GradientType.Internal if internal else GradientType.Dense),
        summation_dtype=torch.int32 if cfg.get("int_mode") else torch.float32,
        _explicit_anchors=torch.from_numpy(anchors.reshape(-1).copy()), _int_rescaler=cfg.get("int_rescaler", 0.001),
        _forward_group_size=cfg.get("G", 32), random_seed=1, device=device)
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
        if pe is not None:
            layer._positional_embeddings.copy_(torch.from_numpy(pe))
    if internal:
        layer.set_external_learning_rate_hook(lambda w: cfg["ext_lr"])
    return layer


def run_gpu(cfg, x, anchors, W, pe, dY, device="cuda:0", prepare=None):
    layer = build_layer(cfg, anchors, W, pe, device)
    if prepare is not None:
        prepare(layer)  # the CPU tests swap the runtime for the oracle here
    dev = torch.device("cpu" if device is None else device)
    xt = torch.from_numpy(x).to(dev)
    pos = layer._prepare_positional_embeddings()
    pos = None if pos is None else pos.detach()
    layer.eval()
    y_eval = layer.forward_step_concat(xt, pos)
    layer.train()
    y, idx, md, mk, pidx, pmd, pmk = layer.forward_step_concat(xt, pos)
    dx, dw, dpe = layer.backward_step_concat(xt, torch.from_numpy(dY).to(dev), idx, md, mk, pidx, pmd, pmk)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    n = cfg["B"] * cfg["S"]
    out = dict(y=y.cpu().numpy(), y_eval=y_eval.cpu().numpy(), dX=dx.cpu().numpy(),
               idx=idx.cpu().numpy().reshape(n, -1), min_k=mk.cpu().numpy().reshape(n, -1),
               min_delta=md.cpu().numpy().reshape(n, -1))
    if dpe is not None:
        out.update(dPE=dpe.cpu().numpy(), pidx=pidx.cpu().numpy().reshape(-1), pmin_k=pmk.cpu().numpy().reshape(-1),
                   pmin=pmd.cpu().numpy().reshape(-1))
    if cfg.get("policy") == "internal":
        out["W_after"] = layer._weights.detach().cpu().numpy()
    else:
        out["dW"] = dw.cpu().numpy()
    return out


def compare(cfg, got, ref):
    assert np.array_equal(got["idx"], ref["idx"]) and np.array_equal(got["min_k"], ref["min_k"])
    assert np.array_equal(got["min_delta"].view(np.int32), ref["min_delta"].view(np.int32))
    if cfg["Npe"] > 0:
        assert np.array_equal(got["pidx"], ref["pidx"]) and np.array_equal(got["pmin_k"], ref["pmin_k"])
        assert np.array_equal(got["pmin"].view(np.int32), ref["pmin"].view(np.int32))
    keys = ["y", "y_eval", "dX"] + (["dPE"] if cfg["Npe"] > 0 else []) + (["W_after"] if "W_after" in ref else ["dW"])
    for k in keys:
        if cfg.get("int_mode"):
            assert np.array_equal(got[k], ref[k]), f"{k}: fixed-point results must be bit-exact"
        else:
            golden_util.assert_close(got[k], ref[k], REL, k)


def inputs_for(cfg):
    n_pe = (cfg["S"] - 1) * (1 if cfg.get("unified_pe") else cfg["Nt"]) * cfg["Npe"]
    return sequence_inputs(cfg, cfg["Nt"] * (1 << (2 * cfg["Nc"] + cfg["Npe"])) * cfg["O"], n_pe)


@pytest.mark.parametrize("name", golden_util.names("concat_"))
def test_concat_matches_reference_golden(name):
    cfg, ref = golden_util.load(name)
    x, anchors, W, pe, dY = inputs_for(cfg)
    compare(cfg, run_gpu(cfg, x, anchors, W, pe, dY), ref)


ORACLE_CASES = {
    # shapes of the reference's own transformer test: 8 tokens, 3 pairs, 4 positional dims (1024-row tables)
    "ref_test_shape": dict(seed=800, B=4, S=8, E=32, Nt=8, Nc=3, Npe=4, O=32, G=24),
    "ref_test_shape_i32": dict(seed=801, B=4, S=8, E=32, Nt=8, Nc=3, Npe=4, O=32, G=24, int_mode=True, int_rescaler=10.0),
    "longer": dict(seed=802, B=2, S=70, E=24, Nt=5, Nc=3, Npe=2, O=48, unified_pe=True),
    "ragged_outputs": dict(seed=803, B=3, S=19, E=12, Nt=4, Nc=2, Npe=3, O=10, quantized_input=True),
    "wide_i32": dict(seed=804, B=1, S=20, E=12, Nt=3, Nc=2, Npe=2, O=70, int_mode=True, int_rescaler=0.1),
}


@pytest.mark.parametrize("name", sorted(ORACLE_CASES))
def test_concat_matches_oracle(name):
    cfg = ORACLE_CASES[name]
    x, anchors, W, pe, dY = inputs_for(cfg)
    pe3 = expand_pe(cfg, pe)
    kw = dict(int_mode=cfg.get("int_mode", False), int_rescaler=cfg.get("int_rescaler", 0.001))
    y, st = orc.concat_forward(W, x, pe3, anchors, cfg["Nt"], cfg["Nc"], cfg["O"], cfg["Npe"], **kw)
    dX, dW, dPE = orc.concat_backward(W, dY, anchors, st, cfg["E"], cfg["Nc"], cfg["Npe"],
                                      forward_group_size=cfg.get("G", 32), **kw)
    ref = dict(y=y, y_eval=y, dX=dX, dW=dW, dPE=dPE, idx=st["idx"], min_k=st["min_k"], min_delta=st["min_delta"],
               pidx=st["pidx"], pmin=st["pmin"], pmin_k=st["pmin_k"])
    compare(cfg, run_gpu(cfg, x, anchors, W, pe, dY), ref)
