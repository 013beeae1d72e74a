"""The CPU oracle against the golden vectors recorded from the reference's own CPU build.

fp32 results are required to be bit-identical: the oracle follows the reference's host loop order,
so any difference means the restatement deviates from the reference's arithmetic.
"""
import numpy as np
import pytest

import golden_util
from cases import nonseq_fc_inputs
from oracle import lut_oracle as orc


@pytest.mark.parametrize("name", golden_util.names("fc_"))
def test_nonseq_fc_oracle_matches_reference(name):
    cfg, ref = golden_util.load(name)
    x, anchors, W, dY = nonseq_fc_inputs(cfg)
    if "in_x" in ref:  # small cases also store their inputs: the seeded builders must reproduce them
        assert np.array_equal(ref["in_x"], x) and np.array_equal(ref["in_anchors"], anchors)
        assert np.array_equal(ref["in_W"], W) and np.array_equal(ref["in_dY"], dY)
    Nt, Nc, O, I = cfg["Nt"], cfg["Nc"], cfg["O"], cfg["I"]
    kw = dict(int_mode=cfg.get("int_mode", False), int_rescaler=cfg.get("int_rescaler", 0.001))
    eps = cfg.get("cmp_eps", 0.0)
    y_eval, idx_eval, _, _ = orc.nonseq_fc_forward(W, x, anchors, Nt, Nc, O, eps, train=False,
                                                   backward_group_size=cfg.get("Gb", 32), **kw)
    y, idx, md, mk = orc.nonseq_fc_forward(W, x, anchors, Nt, Nc, O, eps, train=True,
                                           backward_group_size=cfg.get("Gb", 32), **kw)
    assert np.array_equal(idx, ref["idx"]) and np.array_equal(idx_eval, ref["idx"])
    assert np.array_equal(mk, ref["min_k"])
    assert np.array_equal(md.view(np.int32), ref["min_delta"].view(np.int32))
    assert np.array_equal(y, ref["y"]) and np.array_equal(y_eval, ref["y_eval"])
    internal = cfg.get("policy") == "internal"
    Wb = W.copy()
    dX, dW = orc.nonseq_fc_backward(Wb, dY, anchors, idx, md, mk, I, Nc, lr_meta=cfg.get("lr_meta", 1.0),
                                    external_lr=cfg["ext_lr"] if internal else -1.0,
                                    forward_group_size=cfg.get("G", 32), **kw)
    assert np.array_equal(dX, ref["dX"])
    if internal:
        assert dW is None and np.array_equal(Wb, ref["W_after"])
    else:
        assert np.array_equal(dW, ref["dW"])


def test_oracle_threads_do_not_change_results():
    cfg, ref = golden_util.load("fc_c1_slice_f32")
    x, anchors, W, dY = nonseq_fc_inputs(cfg)
    orc.set_threads(4)
    try:
        y, idx, md, mk = orc.nonseq_fc_forward(W, x, anchors, cfg["Nt"], cfg["Nc"], cfg["O"])
        dX, dW = orc.nonseq_fc_backward(W, dY, anchors, idx, md, mk, cfg["I"], cfg["Nc"])
    finally:
        orc.set_threads(1)
    assert np.array_equal(y, ref["y"]) and np.array_equal(dX, ref["dX"]) and np.array_equal(dW, ref["dW"])


def sparse_index_from_golden(cfg, ref):
    from spiky_b200.structure import SparseIndex

    rows = cfg["n_lookup_neurons"] // cfg["Nt"]
    O = cfg["out_shape"][0] * cfg["out_shape"][1]
    return SparseIndex.from_export(ref["syn_source"], ref["syn_slot"], ref["syn_target"], cfg["Nt"], rows,
                                   cfg.get("G", 32), O, cfg["n_weights"])


@pytest.mark.parametrize("name", golden_util.names("proj_"))
def test_sparse_oracle_matches_reference(name):
    from cases import projection_inputs

    cfg, ref = golden_util.load(name)
    index = sparse_index_from_golden(cfg, ref)
    sp = dict(index.numpy(), group_size=index.group_size)
    x, W, dY = projection_inputs(cfg, cfg["n_weights"])
    I = cfg["in_shape"][0] * cfg["in_shape"][1]
    O = cfg["out_shape"][0] * cfg["out_shape"][1]
    kw = dict(int_mode=cfg.get("int_mode", False), int_rescaler=cfg.get("int_rescaler", 0.001))
    anchors = ref["anchors"]
    y_eval, _, _, _ = orc.nonseq_sparse_forward(W, x, anchors, sp, cfg["Nc"], O, train=False, **kw)
    y, idx, md, mk = orc.nonseq_sparse_forward(W, x, anchors, sp, cfg["Nc"], O, train=True, **kw)
    assert np.array_equal(idx, ref["idx"]) and np.array_equal(mk, ref["min_k"])
    assert np.array_equal(md.view(np.int32), ref["min_delta"].view(np.int32))
    assert np.array_equal(y, ref["y"]) and np.array_equal(y_eval, ref["y_eval"])
    internal = cfg.get("policy") == "internal"
    Wb = W.copy()
    dX, dW = orc.nonseq_sparse_backward(Wb, dY, anchors, idx, md, mk, sp, I, cfg["Nc"],
                                        lr_meta=cfg.get("lr_meta", 1.0),
                                        external_lr=cfg["ext_lr"] if internal else -1.0, **kw)
    assert np.array_equal(dX, ref["dX"])
    if internal:
        assert np.array_equal(Wb, ref["W_after"])
    else:
        assert np.array_equal(dW, ref["dW"])


def test_own_sparse_construction_is_self_consistent():
    """Connectivity built without the reference: layout invariants of the flat weight array."""
    import torch
    from spiky_b200.structure import SparseIndex

    targets = torch.tensor([[3, 4, 9, -1], [0, 1, -1, -1], [5, 6, 7, 8]])
    counts = torch.tensor([3, 2, 4])
    sp = SparseIndex.from_detector_targets(targets, counts, rows_per_detector=4, group_size=2, n_outputs=10)
    # strides: P + 2*ceil(P/G) = 3+4, 2+2, 4+4
    assert sp.det_stride.tolist() == [7, 4, 8] and sp.det_wbase.tolist() == [0, 28, 44]
    assert sp.n_weights == 28 + 16 + 32 - 2 and sp.n_synapses == (3 + 2 + 4) * 4
    assert sp.syn_target.tolist() == [3, 4, 9, 0, 1, 5, 6, 7, 8] and sp.max_groups_per_neuron == 2
    assert int(sp.slot_mask().sum()) == sp.n_synapses


def expand_pe(cfg, pe):
    """Flat layer embeddings -> [(S-1), Nt, Npe] as the runtime sees them (unified ones repeated per detector)."""
    if pe is None:
        return None
    S, Nt, Npe = cfg["S"], cfg["Nt"], cfg["Npe"]
    if cfg.get("unified_pe"):
        return np.repeat(pe.reshape(S - 1, 1, Npe), Nt, axis=1).copy()
    return pe.reshape(S - 1, Nt, Npe)


@pytest.mark.parametrize("name", golden_util.names("prod_"))
def test_product_oracle_matches_reference(name):
    from cases import sequence_inputs

    cfg, ref = golden_util.load(name)
    S, Nt, Nc, O, Npe = cfg["S"], cfg["Nt"], cfg["Nc"], cfg["O"], cfg["Npe"]
    n_pe = (S - 1) * (1 if cfg.get("unified_pe") else Nt) * Npe
    x, anchors, W, pe, dY = sequence_inputs(cfg, Nt * (1 << Nc) * O, n_pe)
    assert np.array_equal(x, ref["in_x"]) and np.array_equal(anchors, ref["in_anchors"])
    pe3 = expand_pe(cfg, pe)
    kw = dict(sliced=cfg.get("sliced", False), cmp_eps=cfg.get("cmp_eps", 0.0), int_mode=cfg.get("int_mode", False),
              int_rescaler=cfg.get("int_rescaler", 0.001))
    y = orc.product_forward(W, x, pe3, anchors, Nt, Nc, O, Npe, **kw)
    assert np.array_equal(y, ref["y"])
    internal = cfg.get("policy") == "internal"
    Wb = W.copy()
    dX, dW, dPE = orc.product_backward(Wb, x, pe3, anchors, dY, Nt, Nc, Npe, lr_meta=cfg.get("lr_meta", 1.0),
                                       external_lr=cfg["ext_lr"] if internal else -1.0, **kw)
    assert np.array_equal(dX, ref["dX"])
    if Npe > 0:
        assert np.array_equal(dPE, ref["dPE"])
    if internal:
        assert np.array_equal(Wb, ref["W_after"])
    else:
        assert np.array_equal(dW, ref["dW"])


@pytest.mark.parametrize("name", golden_util.names("concat_"))
def test_concat_oracle_matches_reference(name):
    from cases import sequence_inputs

    cfg, ref = golden_util.load(name)
    S, Nt, Nc, O, Npe, E = cfg["S"], cfg["Nt"], cfg["Nc"], cfg["O"], cfg["Npe"], cfg["E"]
    n_pe = (S - 1) * (1 if cfg.get("unified_pe") else Nt) * Npe
    x, anchors, W, pe, dY = sequence_inputs(cfg, Nt * (1 << (2 * Nc + Npe)) * O, n_pe)
    assert np.array_equal(x, ref["in_x"]) and np.array_equal(anchors, ref["in_anchors"])
    pe3 = expand_pe(cfg, pe)
    kw = dict(int_mode=cfg.get("int_mode", False), int_rescaler=cfg.get("int_rescaler", 0.001))
    y_eval, _ = orc.concat_forward(W, x, pe3, anchors, Nt, Nc, O, Npe, train=False, **kw)
    y, st = orc.concat_forward(W, x, pe3, anchors, Nt, Nc, O, Npe, train=True, **kw)
    assert np.array_equal(st["idx"], ref["idx"]) and np.array_equal(st["min_k"], ref["min_k"])
    assert np.array_equal(st["min_delta"].view(np.int32), ref["min_delta"].view(np.int32))
    if Npe > 0:
        assert np.array_equal(st["pidx"], ref["pidx"]) and np.array_equal(st["pmin_k"], ref["pmin_k"])
        assert np.array_equal(st["pmin"].view(np.int32), ref["pmin"].view(np.int32))
    assert np.array_equal(y, ref["y"]) and np.array_equal(y_eval, ref["y_eval"])
    internal = cfg.get("policy") == "internal"
    Wb = W.copy()
    dX, dW, dPE = orc.concat_backward(Wb, dY, anchors, st, E, Nc, Npe, lr_meta=cfg.get("lr_meta", 1.0),
                                      external_lr=cfg["ext_lr"] if internal else -1.0,
                                      forward_group_size=cfg.get("G", 32), **kw)
    assert np.array_equal(dX, ref["dX"])
    if Npe > 0:
        assert np.array_equal(dPE, ref["dPE"])
    if internal:
        assert np.array_equal(Wb, ref["W_after"])
    else:
        assert np.array_equal(dW, ref["dW"])


@pytest.mark.parametrize("name", golden_util.names("sparse_concat_"))
def test_concat_sparse_oracle_matches_reference(name):
    """Concatenation-mode layers with sparse lookup -> output connectivity (reference: Conv2DLUTLayer with a second
    sliding window, sequence_length > 1)."""
    from cases import concat_sparse_inputs

    cfg, ref = golden_util.load(name)
    index = sparse_index_from_golden(cfg, ref)
    sp = dict(index.numpy(), group_size=index.group_size)
    x, W, pe, dY = concat_sparse_inputs(cfg, cfg["n_weights"], cfg["O"], cfg["Nt"])
    kw = dict(int_mode=cfg.get("int_mode", False), int_rescaler=cfg.get("int_rescaler", 0.001))
    anchors = ref["anchors"]
    y_eval, _ = orc.concat_sparse_forward(W, x, None, anchors, sp, cfg["Nc"], cfg["O"], cfg["Npe"], train=False, **kw)
    y, st = orc.concat_sparse_forward(W, x, None, anchors, sp, cfg["Nc"], cfg["O"], cfg["Npe"], train=True, **kw)
    assert np.array_equal(st["idx"], ref["idx"]) and np.array_equal(st["min_k"], ref["min_k"])
    assert np.array_equal(y, ref["y"]) and np.array_equal(y_eval, ref["y_eval"])
    internal = cfg.get("policy") == "internal"
    Wb = W.copy()
    dX, dW, _ = orc.concat_sparse_backward(Wb, dY, anchors, st, sp, cfg["E"], cfg["Nc"], cfg["Npe"],
                                           lr_meta=cfg.get("lr_meta", 1.0),
                                           external_lr=cfg["ext_lr"] if internal else -1.0, **kw)
    assert np.array_equal(dX, ref["dX"])
    if internal:
        assert np.array_equal(Wb, ref["W_after"])
    else:
        assert np.array_equal(dW, ref["dW"])
