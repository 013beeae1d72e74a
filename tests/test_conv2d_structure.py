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


def _cpu_layer(cfg):
    from spiky_b200.lut_layer import Conv2DLUTLayer, SynapseMeta

    return Conv2DLUTLayer(
        input_shape=tuple(cfg["in_shape"]), n_anchors_per_detector=cfg["Nc"], detectors_shape=tuple(cfg["det_shape"]),
        output_kernel_shape=tuple(cfg["out_kernel"]), receptive_field_shape=tuple(cfg["rf"]),
        receptive_field_stride_shape=tuple(cfg["rf_stride"]),
        lut_receptive_field_shape=None if cfg["lut_rf"] is None else tuple(cfg["lut_rf"]),
        lut_receptive_field_stride_shape=None if cfg["lut_rf_stride"] is None else tuple(cfg["lut_rf_stride"]),
        synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
        summation_dtype=torch.int32 if cfg.get("int_mode") else torch.float32,
        _int_rescaler=cfg.get("int_rescaler", 0.001), random_seed=cfg["seed"], device=None)


@pytest.mark.parametrize("name", golden_util.names("conv2d_"))
def test_synapse_export_reproduces_the_reference_export(name):
    """A layer that adopted a reference-built structure exports the same synapse list, in the same order, as the
    reference layer did (source, weight slot read back through weights 0, 1, 2, ..., target)."""
    cfg, ref = golden_util.load(name)
    layer = _cpu_layer(cfg)
    n_lookup = cfg["n_lookup_neurons"]
    if cfg["lut_rf"] is None:
        # fully connected: every lookup neuron lists all outputs, weights are the table rows
        ids = torch.tensor([3, 0, n_lookup - 1], dtype=torch.int32)
        O = cfg["O"]
        assert layer._count_synapses(ids) == n_lookup * O
        src, w, tgt = torch.zeros(3 * O, dtype=torch.int32), torch.zeros(3 * O), torch.zeros(3 * O, dtype=torch.int32)
        layer._export_synapses(ids, src, w, tgt)
        assert torch.equal(src, ids.repeat_interleave(O))
        assert torch.equal(tgt, (torch.arange(O, dtype=torch.int32) + n_lookup).repeat(3))
        assert torch.equal(w, layer._weights.detach().view(n_lookup, O)[ids.long()].flatten())
        with pytest.raises(ValueError):
            layer._lut_dm.count_synapses(ids)
        return
    layer.load_structure(ref["anchors"], ref["syn_source"], ref["syn_slot"], ref["syn_target"], cfg["n_weights"])
    n = layer.n_synapses()
    assert n == ref["syn_source"].size == layer._count_synapses(layer.get_lookup_neuron_ids())
    with torch.no_grad():
        layer._weights.copy_(torch.arange(cfg["n_weights"], dtype=torch.float32))
    src, slot, tgt = torch.zeros(n, dtype=torch.int32), torch.zeros(n), torch.zeros(n, dtype=torch.int32)
    layer._export_synapses(layer.get_lookup_neuron_ids(), src, slot, tgt)
    assert np.array_equal(src.numpy(), ref["syn_source"])
    assert np.array_equal(slot.numpy().astype(np.int64), ref["syn_slot"])
    assert np.array_equal(tgt.numpy() - n_lookup, ref["syn_target"])
    # a subset, in the order asked for
    rows = n_lookup // cfg["Nt"]
    ids = torch.tensor([rows + 1, 0], dtype=torch.int32)
    k = layer._count_synapses(ids)
    s2, w2, t2 = torch.zeros(k, dtype=torch.int32), torch.zeros(k), torch.zeros(k, dtype=torch.int32)
    layer._export_synapses(ids, s2, w2, t2)
    first = ref["syn_source"] == rows + 1
    assert np.array_equal(w2.numpy()[:first.sum()].astype(np.int64), ref["syn_slot"][first])
    assert np.array_equal(s2.numpy()[first.sum():], np.zeros(k - first.sum(), dtype=np.int32))
    # export_weights: ordered by output, then lookup neuron
    if name.startswith("conv2d_sparse"):
        order = np.lexsort((ref["syn_source"], ref["syn_target"]))
        try:
            got = layer.export_weights()
        except RuntimeError:
            got = None  # windows at the border hold fewer synapses: the reference's reshape fails the same way
        if got is not None:
            assert np.array_equal(got.reshape(-1).numpy().astype(np.int64), ref["syn_slot"][order])


def test_own_structure_round_trips_through_export():
    from spiky_b200 import structure

    cfg, _ = golden_util.load("conv2d_sparse_f32")
    layer = _cpu_layer(cfg)
    index = layer._lut_dm._sparse
    n = layer.n_synapses()
    with torch.no_grad():
        layer._weights.copy_(torch.arange(index.n_weights, dtype=torch.float32))
    src, slot, tgt = torch.zeros(n, dtype=torch.int32), torch.zeros(n), torch.zeros(n, dtype=torch.int32)
    layer._export_synapses(layer.get_lookup_neuron_ids(), src, slot, tgt)
    again = structure.SparseIndex.from_export(src, slot.long(), tgt.long() - layer.n_lookup_neurons(), layer.n_detectors(),
                                              index.rows_per_detector, index.group_size, layer.n_outputs(), index.n_weights)
    for field in structure.SparseIndex._TENSORS:
        assert torch.equal(getattr(again, field), getattr(index, field)), field
    assert torch.equal(index.slot_mask().nonzero().flatten(), slot.long().sort().values)
