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
