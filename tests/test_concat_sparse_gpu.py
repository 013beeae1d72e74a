"""Concatenation-mode sequence layers with sparse lookup -> output connectivity (Conv2DLUTLayer with a second
sliding window, sequence_length > 1) against the reference's golden vectors and the oracle."""
import numpy as np
import pytest
import torch

import golden_util
import synth
from cases import concat_sparse_inputs
from oracle import lut_oracle as orc

pytestmark = pytest.mark.gpu
REL = 1e-5


def make_layer(cfg, int_mode=None, internal=None):
    from spiky_b200.lut_layer import Conv2DLUTLayer, SynapseMeta, GradientPolicy, GradientType

    internal = cfg.get("policy") == "internal" if internal is None else internal
    int_mode = cfg.get("int_mode", False) if int_mode is None else int_mode
    return Conv2DLUTLayer(
        input_shape=tuple(cfg["in_shape"]), n_anchors_per_detector=cfg["Nc"], detectors_shape=tuple(cfg["det_shape"]),
        output_kernel_shape=tuple(cfg["out_kernel"]), sequence_length=cfg["S"], receptive_field_shape=tuple(cfg["rf"]),
        receptive_field_stride_shape=tuple(cfg["rf_stride"]), lut_receptive_field_shape=tuple(cfg["lut_rf"]),
        lut_receptive_field_stride_shape=tuple(cfg["lut_rf_stride"]),
        synapse_meta=SynapseMeta(learning_rate=cfg.get("lr_meta", 1.0), min_weight=-1.0, max_weight=1.0,
                                 initial_noise_level=0.1, initial_weight=0.02),
        concatenation_product=True, positional_dim=cfg["Npe"], unified_pe=cfg.get("unified_pe", False),
        weights_gradient_policy=GradientPolicy(GradientType.Internal if internal else GradientType.Dense),
        summation_dtype=torch.int32 if int_mode else torch.float32, _int_rescaler=cfg.get("int_rescaler", 0.001),
        _forward_group_size=cfg.get("G", 32), random_seed=cfg["seed"], device="cuda:0")


def run_layer(layer, cfg, x, dY):
    B, S = cfg["B"], cfg["S"]
    xt = torch.from_numpy(x).view((B, S) + tuple(layer.input_shape())).cuda()
    pos = layer._prepare_positional_embeddings()
    pos = None if pos is None else pos.detach()
    layer.eval()
    y_eval = layer.forward_step_concat(xt, pos)
    layer.train()
    y, idx, md, mk, pidx, pmd, pmk = layer.forward_step_concat(xt, pos)
    if cfg.get("policy") == "internal":
        layer.set_external_learning_rate_hook(lambda w: cfg["ext_lr"])
    dyt = torch.from_numpy(dY).view((B, S) + tuple(layer.output_shape())).cuda()
    dx, dw, dpe = layer.backward_step_concat(xt, dyt, idx, md, mk, pidx, pmd, pmk)
    torch.cuda.synchronize()
    n = B * S
    out = dict(y=y.cpu().numpy().reshape(B, S, -1), y_eval=y_eval.cpu().numpy().reshape(B, S, -1),
               dX=dx.cpu().numpy().reshape(B, S, -1), idx=idx.cpu().numpy().reshape(n, -1),
               min_k=mk.cpu().numpy().reshape(n, -1))
    if dpe is not None:
        out["dPE"] = dpe.cpu().numpy().reshape(-1)
    if cfg.get("policy") == "internal":
        out["W_after"] = layer._weights.detach().cpu().numpy()
    else:
        out["dW"] = dw.cpu().numpy()
    return out


def compare(cfg, got, ref, keys):
    assert np.array_equal(got["idx"], ref["idx"]) and np.array_equal(got["min_k"], ref["min_k"])
    for k in keys:
        if cfg.get("int_mode"):
            assert np.array_equal(got[k], ref[k]), f"{k}: fixed-point results must be bit-exact"
        else:
            golden_util.assert_close(got[k], ref[k], REL, k)


@pytest.mark.parametrize("name", golden_util.names("sparse_concat_"))
def test_sparse_concat_matches_reference_golden(name):
    cfg, ref = golden_util.load(name)
    layer = make_layer(cfg)
    assert layer.n_detectors() == cfg["Nt"] and layer.n_outputs() == cfg["O"]
    layer.load_structure(ref["anchors"], ref["syn_source"], ref["syn_slot"], ref["syn_target"], cfg["n_weights"])
    x, W, pe, dY = concat_sparse_inputs(cfg, cfg["n_weights"], cfg["O"], cfg["Nt"])
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
    got = run_layer(layer, cfg, x, dY)
    compare(cfg, got, ref, ["y", "y_eval", "dX"] + (["W_after"] if "W_after" in ref else ["dW"]))


@pytest.mark.parametrize("int_mode", [False, True])
def test_sparse_concat_with_positional_embeddings_matches_oracle(int_mode):
    """Positional embeddings on top of sparse connectivity: the reference cannot build this layer (its output window
    assumes 2^(2*Nc) rows per detector), the kernels and the oracle handle 2^(2*Nc + Npe) rows."""
    cfg = dict(seed=520, B=2, S=9, in_shape=(4, 4), Nc=2, Npe=2, det_shape=(2, 1), out_kernel=(1, 2), rf=(2, 2),
               rf_stride=(2, 2), lut_rf=(2, 2), lut_rf_stride=(1, 1), G=2, int_mode=int_mode, int_rescaler=0.5)
    layer = make_layer(cfg)
    Nt, O, E = layer.n_detectors(), layer.n_outputs(), 16
    x = synth.uniform(521, (cfg["B"], cfg["S"], E), -1.0, 1.0)
    dY = synth.normal(522, (cfg["B"], cfg["S"], O))
    got = run_layer(layer, cfg, x, dY)
    index = layer._lut_dm._sparse
    sp = dict(index.numpy(), group_size=index.group_size)
    W = layer._weights.detach().cpu().numpy()
    anchors = layer._detector_anchors.cpu().numpy()
    pe = layer._prepare_positional_embeddings().detach().cpu().numpy().reshape(cfg["S"] - 1, Nt, cfg["Npe"])
    kw = dict(int_mode=int_mode, int_rescaler=0.5)
    y, st = orc.concat_sparse_forward(W, x, pe, anchors, sp, cfg["Nc"], O, cfg["Npe"], **kw)
    dX, dW, dPE = orc.concat_sparse_backward(W, dY, anchors, st, sp, E, cfg["Nc"], cfg["Npe"], **kw)
    ref = dict(y=y, y_eval=y, idx=st["idx"], min_k=st["min_k"], dX=dX, dW=dW, dPE=dPE)
    compare(cfg, got, ref, ["y", "y_eval", "dX", "dW", "dPE"])
