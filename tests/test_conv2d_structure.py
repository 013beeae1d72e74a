"""Conv2DLUTLayer geometry against the reference: shapes, the inputs each detector may compare (its receptive field)
and the outputs it feeds (second sliding window), from fixtures recorded with the reference's Conv2DLUTLayer; and, on a
GPU, the numeric results of those layers."""
import numpy as np
import pytest
import torch

import golden_util
from cases import conv2d_inputs


def geometry(cfg):
    from spiky_b200 import structure

    det_geo = structure.SlidingWindows(tuple(cfg["in_shape"]), tuple(cfg["rf"]), tuple(cfg["rf_stride"]),
                                       tuple(cfg["det_shape"]))
    out_geo = None
    if cfg["lut_rf"] is not None:
        out_geo = structure.SlidingWindows(det_geo.out_shape, tuple(cfg["lut_rf"]), tuple(cfg["lut_rf_stride"]),
                                           tuple(cfg["out_kernel"]))
    return det_geo, out_geo


@pytest.mark.parametrize("name", golden_util.names("conv2d_"))
def test_conv2d_geometry_matches_reference(name):
    cfg, ref = golden_util.load(name)
    det_geo, out_geo = geometry(cfg)
    Nt, Nc = cfg["Nt"], cfg["Nc"]
    assert det_geo.out_shape[0] * det_geo.out_shape[1] == Nt
    assert tuple(det_geo.out_shape) == tuple(cfg["lut_shape"][:2])
    # every anchor the reference sampled for a detector lies inside that detector's receptive field
    pools, counts = det_geo.input_pools()
    anchors = ref["anchors"].reshape(Nt, Nc, 2)
    for t in range(Nt):
        allowed = set(pools[t, :counts[t]].tolist())
        assert set(anchors[t].reshape(-1).tolist()) <= allowed, f"detector {t}"
    if out_geo is None:
        assert cfg["O"] == cfg["out_kernel"][0] * cfg["out_kernel"][1]
        return
    assert tuple(out_geo.out_shape) == tuple(cfg["out_shape"])
    # every lookup neuron of detector t feeds exactly the outputs of the windows that contain t
    rows = cfg["n_lookup_neurons"] // Nt
    targets, tcounts = out_geo.output_targets()
    src, tgt = ref["syn_source"].astype(np.int64), ref["syn_target"].astype(np.int64)
    for t in range(Nt):
        mine = sorted(targets[t, :tcounts[t]].tolist())
        for row in (0, rows - 1):
            theirs = sorted(tgt[src == t * rows + row].tolist())
            assert theirs == mine, f"detector {t}, row {row}"


@pytest.mark.gpu
@pytest.mark.parametrize("name", golden_util.names("conv2d_"))
def test_conv2d_layer_matches_reference_golden(name):
    from spiky_b200.lut_layer import Conv2DLUTLayer, SynapseMeta

    cfg, ref = golden_util.load(name)
    int_mode = cfg.get("int_mode", False)
    layer = Conv2DLUTLayer(
        input_shape=tuple(cfg["in_shape"]), n_anchors_per_detector=cfg["Nc"], detectors_shape=tuple(cfg["det_shape"]),
        output_kernel_shape=tuple(cfg["out_kernel"]), receptive_field_shape=tuple(cfg["rf"]),
        receptive_field_stride_shape=tuple(cfg["rf_stride"]),
        lut_receptive_field_shape=None if cfg["lut_rf"] is None else tuple(cfg["lut_rf"]),
        lut_receptive_field_stride_shape=None if cfg["lut_rf_stride"] is None else tuple(cfg["lut_rf_stride"]),
        synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
        summation_dtype=torch.int32 if int_mode else torch.float32, _int_rescaler=cfg.get("int_rescaler", 0.001),
        _explicit_anchors=torch.from_numpy(ref["anchors"].reshape(-1).copy()), random_seed=cfg["seed"], device="cuda:0")
    assert layer.n_detectors() == cfg["Nt"] and layer.n_outputs() == cfg["O"]
    assert tuple(layer.output_shape()) == tuple(cfg["out_shape"])
    if cfg["lut_rf"] is not None:
        layer.load_structure(ref["anchors"], ref["syn_source"], ref["syn_slot"], ref["syn_target"], cfg["n_weights"])
    B, O, Nt = cfg["B"], cfg["O"], cfg["Nt"]
    I = cfg["in_shape"][0] * cfg["in_shape"][1]
    x, W, dY = conv2d_inputs(cfg, cfg["n_weights"], O)
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
    layer.train()
    xt = torch.from_numpy(x).view((B, 1) + tuple(cfg["in_shape"])).cuda()
    y, idx, md, mk = layer.forward_step(xt)
    dx, dw = layer.backward_step(xt, torch.from_numpy(dY).view((B, 1) + tuple(layer.output_shape())).cuda(), idx, md, mk)
    torch.cuda.synchronize()
    assert np.array_equal(idx.cpu().numpy().reshape(B, Nt), ref["idx"])
    assert np.array_equal(mk.cpu().numpy().reshape(B, Nt), ref["min_k"])
    got = dict(y=y.cpu().numpy().reshape(B, O), dX=dx.cpu().numpy().reshape(B, I), dW=dw.cpu().numpy())
    for k in ("y", "dX", "dW"):
        if int_mode:
            assert np.array_equal(got[k], ref[k]), k
        else:
            golden_util.assert_close(got[k], ref[k], 1e-5, k)
