"""CUDA path of product-mode sequence (attention) layers against the reference's golden vectors and the oracle."""
import numpy as np
import pytest
import torch

import golden_util
from cases import sequence_inputs, PRODUCT_CASES
from oracle import lut_oracle as orc
from test_oracle_golden import expand_pe

pytestmark = pytest.mark.gpu
REL = 1e-5


def build_layer(cfg, anchors, W, pe, device="cuda:0"):
    from spiky_b200.lut_layer import LUTLayer, SynapseMeta, GradientPolicy, GradientType, LUTSharedContext

    internal = cfg.get("policy") == "internal"
    ctx = LUTSharedContext(_cmp_eps=cfg.get("cmp_eps", 0.0)).to_device("cpu" if device is None else device)
    layer = LUTLayer(
        cfg["E"], cfg["Nc"], cfg["Nt"], cfg["O"], sequence_length=cfg["S"],
        synapse_meta=SynapseMeta(learning_rate=cfg.get("lr_meta", 1.0), min_weight=-1.0, max_weight=1.0),
        concatenation_product=False, sliced_product_mode=cfg.get("sliced", False), positional_dim=cfg["Npe"],
        unified_pe=cfg.get("unified_pe", False),
        weights_gradient_policy=GradientPolicy(GradientType.Internal if internal else GradientType.Dense),
        shared_context=ctx, summation_dtype=torch.int32 if cfg.get("int_mode") else torch.float32,
        _explicit_anchors=torch.from_numpy(anchors.reshape(-1).copy()), _int_rescaler=cfg.get("int_rescaler", 0.001),
        random_seed=1, device=device)
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
        if pe is not None:
            layer._positional_embeddings.copy_(torch.from_numpy(pe))
    if internal:
        layer.set_external_learning_rate_hook(lambda w: cfg["ext_lr"])
    return layer


def run_gpu(cfg, x, anchors, W, pe, dY, variant=0, device="cuda:0", prepare=None):
    layer = build_layer(cfg, anchors, W, pe, device)
    if prepare is not None:
        prepare(layer)  # the CPU tests swap the runtime for the oracle here
    dev = torch.device("cpu" if device is None else device)
    layer._product_variant = variant  # 0 auto, 1 direct gathers, 2 histogram + tiled contraction
    layer.train()
    xt = torch.from_numpy(x).to(dev)
    pos = layer._prepare_positional_embeddings()
    pos = None if pos is None else pos.detach()
    y = layer.forward_step_product(xt, pos)
    dx, dw, dpe = layer.backward_step_product(xt, pos, torch.from_numpy(dY).to(dev))
    if dev.type == "cuda":
        torch.cuda.synchronize()
    out = dict(y=y.cpu().numpy(), dX=dx.cpu().numpy())
    if dpe is not None:
        out["dPE"] = dpe.cpu().numpy()
    if cfg.get("policy") == "internal":
        out["W_after"] = layer._weights.detach().cpu().numpy()
    else:
        out["dW"] = dw.cpu().numpy()
    return out


def compare(cfg, got, ref):
    keys = ["y", "dX"] + (["dPE"] if cfg["Npe"] > 0 else []) + (["W_after"] if "W_after" in ref else ["dW"])
    for k in keys:
        if cfg.get("int_mode"):
            assert np.array_equal(got[k], ref[k]), f"{k}: fixed-point results must be bit-exact"
        else:
            golden_util.assert_close(got[k], ref[k], cfg.get("rel", REL), k)


def inputs_for(cfg):
    n_pe = (cfg["S"] - 1) * (1 if cfg.get("unified_pe") else cfg["Nt"]) * cfg["Npe"]
    return sequence_inputs(cfg, cfg["Nt"] * (1 << cfg["Nc"]) * cfg["O"], n_pe)


@pytest.mark.parametrize("name", golden_util.names("prod_"))
def test_product_matches_reference_golden(name):
    cfg, ref = golden_util.load(name)
    x, anchors, W, pe, dY = inputs_for(cfg)
    compare(cfg, run_gpu(cfg, x, anchors, W, pe, dY), ref)


ORACLE_CASES = {
    # one attention layer of the character-level transformer configuration at reduced batch:
    # context 128, d_model 256, 64 detectors (16 x 4 heads), 8 pairs, 4 positional dims
    "c3_attention": dict(seed=700, B=2, S=128, E=256, Nt=64, Nc=8, Npe=4, O=256),
    "c3_attention_i32": dict(seed=701, B=1, S=48, E=64, Nt=16, Nc=8, Npe=4, O=64, int_mode=True, int_rescaler=0.01),
    "ragged_outputs": dict(seed=702, B=3, S=33, E=20, Nt=7, Nc=5, Npe=3, O=10, unified_pe=True),
    "long_rows": dict(seed=703, B=2, S=17, E=16, Nt=3, Nc=6, Npe=2, O=600),
    "sliced": dict(seed=704, B=2, S=40, E=12, Nt=6, Nc=7, Npe=12, O=12, sliced=True, unified_pe=True, cmp_eps=1e-4,
                   quantized_input=True),
    "two_tokens": dict(seed=705, B=2, S=2, E=8, Nt=2, Nc=3, Npe=2, O=4),
}
for _c in ORACLE_CASES.values():
    _c["n_virtual"] = 3 * _c["E"] if _c.get("sliced") else 2 * _c["E"] + _c["Npe"]


def hist_capable(cfg):
    return not cfg.get("int_mode") and 4 <= cfg["Nc"] <= 12 and cfg["O"] % 4 == 0 and cfg["S"] >= 2


# more than 512 tokens: the histogram and routing kernels switch to 16-warp blocks.  A table cell here sums up to ~1e5
# fp32 terms in the oracle and on the GPU alike, in different orders: the order-dependent rounding of such a sum is a
# few 1e-5 of its size, so this case is checked at 1e-4
ORACLE_CASES["long_sequence"] = dict(seed=707, B=1, S=520, E=8, Nt=3, Nc=6, Npe=2, O=8, n_virtual=18, rel=1e-4)
ORACLE_CASES["hist_no_positional"] = dict(seed=720, B=2, S=70, E=9, Nt=4, Nc=5, Npe=0, O=8, n_virtual=18)
ORACLE_CASES["hist_sliced"] = dict(seed=721, B=2, S=50, E=10, Nt=5, Nc=4, Npe=10, O=12, sliced=True, unified_pe=True,
                                   cmp_eps=1e-4, quantized_input=True, n_virtual=30)
ORACLE_CASES["hist_big_table"] = dict(seed=722, B=1, S=260, E=16, Nt=2, Nc=10, Npe=3, O=8, n_virtual=35)
ORACLE_CASES["hist_odd_shapes"] = dict(seed=723, B=3, S=67, E=7, Nt=37, Nc=4, Npe=1, O=20, n_virtual=15)
ORACLE_CASES["internal_sgd"] = dict(seed=706, B=3, S=24, E=16, Nt=5, Nc=5, Npe=3, O=12, policy="internal", ext_lr=0.25,
                                    lr_meta=0.5, n_virtual=35)
# 1 direct gathers, 2 histogram + contraction (tensor cores when the library has them), 3 histogram + fp32 FMA contraction
VARIANT_CASES = [(n, v) for n in sorted(ORACLE_CASES) for v in (1, 2, 3) if v == 1 or hist_capable(ORACLE_CASES[n])]


@pytest.mark.parametrize("name,variant", VARIANT_CASES)
def test_product_matches_oracle(name, variant):
    cfg = ORACLE_CASES[name]
    x, anchors, W, pe, dY = inputs_for(cfg)
    pe3 = expand_pe(cfg, pe)
    kw = dict(sliced=cfg.get("sliced", False), cmp_eps=cfg.get("cmp_eps", 0.0), int_mode=cfg.get("int_mode", False),
              int_rescaler=cfg.get("int_rescaler", 0.001))
    y = orc.product_forward(W, x, pe3, anchors, cfg["Nt"], cfg["Nc"], cfg["O"], cfg["Npe"], **kw)
    if cfg.get("policy") == "internal":
        W_after = W.copy()
        dX, _, dPE = orc.product_backward(W_after, x, pe3, anchors, dY, cfg["Nt"], cfg["Nc"], cfg["Npe"],
                                          lr_meta=cfg["lr_meta"], external_lr=cfg["ext_lr"], **kw)
        ref = dict(y=y, dX=dX, dPE=dPE, W_after=W_after)
    else:
        dX, dW, dPE = orc.product_backward(W, x, pe3, anchors, dY, cfg["Nt"], cfg["Nc"], cfg["Npe"], **kw)
        ref = dict(y=y, dX=dX, dW=dW, dPE=dPE)
    got = run_gpu(cfg, x, anchors, W, pe, dY, variant)
    assert not got["y"][:, 0].any()  # the first position has no earlier token to pair with
    compare(cfg, got, ref)


def test_product_histogram_chunks_match_single_pass():
    """A workspace that holds one sequence at a time gives the same result as one pass over the batch
    (in-place SGD then runs its table update as a second sweep)."""
    from spiky_b200.lut_data_manager import _LUTDataManager
    for name in ("c3_attention", "internal_sgd"):
        cfg = ORACLE_CASES[name]
        x, anchors, W, pe, dY = inputs_for(cfg)
        full = run_gpu(cfg, x, anchors, W, pe, dY, 2)
        saved = _LUTDataManager.product_scratch_limit, _LUTDataManager.product_keep_limit
        _LUTDataManager.product_scratch_limit = 0
        _LUTDataManager.product_keep_limit = 0   # (a forward pass that keeps its histogram takes the whole batch at once)
        _LUTDataManager._product_scratch.clear()
        try:
            chunked = run_gpu(cfg, x, anchors, W, pe, dY, 2)
        finally:
            _LUTDataManager.product_scratch_limit, _LUTDataManager.product_keep_limit = saved
            _LUTDataManager._product_scratch.clear()
        for k in full:
            golden_util.assert_close(chunked[k], full[k], REL, f"{name}.{k}")


def test_product_histogram_rejects_unsupported():
    cfg = dict(seed=711, B=1, S=4, E=6, Nt=2, Nc=3, Npe=2, O=4, n_virtual=14)
    x, anchors, W, pe, dY = inputs_for(cfg)
    with pytest.raises(ValueError, match="histogram variant"):
        run_gpu(cfg, x, anchors, W, pe, dY, 2)


def test_product_autograd_unified_pe():
    """Gradients reach the (unified) positional embeddings through the layer's autograd function."""
    cfg = dict(seed=710, B=2, S=12, E=10, Nt=4, Nc=4, Npe=3, O=8, unified_pe=True, n_virtual=23)
    x, anchors, W, pe, dY = inputs_for(cfg)
    layer = build_layer(cfg, anchors, W, pe)
    layer.train()
    xt = torch.from_numpy(x).cuda().requires_grad_(True)
    y = layer(xt)
    y.backward(torch.from_numpy(dY).cuda())
    pe3 = expand_pe(cfg, pe)
    dX, dW, dPE = orc.product_backward(W, x, pe3, anchors, dY, cfg["Nt"], cfg["Nc"], cfg["Npe"])
    golden_util.assert_close(xt.grad.cpu().numpy(), dX, REL, "dX")
    golden_util.assert_close(layer._weights.grad.cpu().numpy(), dW, REL, "dW")
    want = dPE.reshape(cfg["S"] - 1, cfg["Nt"], cfg["Npe"]).sum(axis=1).reshape(-1)
    golden_util.assert_close(layer._positional_embeddings.grad.cpu().numpy(), want, REL, "dPE (summed over detectors)")


@pytest.mark.parametrize("variant", [2, 3], ids=["tensor_cores", "fma"])
def test_backward_reuses_the_histogram_of_the_forward_pass(variant):
    """Training: the forward pass leaves its row histogram for the backward pass (KEEP / REUSE flags of the C ABI).  Same
    results as when the backward pass counts the rows itself; the workspace is held exactly from forward to backward."""
    import ctypes
    from spiky_b200 import _native
    from spiky_b200.lut_data_manager import _LUTDataManager

    cfg = ORACLE_CASES["c3_attention"]
    x, anchors, W, pe, dY = inputs_for(cfg)
    seen = {}

    def spy(layer):
        dm = layer._lut_dm
        fwd = dm.forward_step_product

        def wrapped(*a, **k):
            fwd(*a, **k)
            seen["kept"] = dm._kept_histogram is not None
        dm.forward_step_product = wrapped
        seen["dm"] = dm

    kept = run_gpu(cfg, x, anchors, W, pe, dY, variant, prepare=spy)
    assert seen["kept"] and seen["dm"]._kept_histogram is None   # held after forward, released by backward
    saved = _LUTDataManager.product_keep_limit
    _LUTDataManager.product_keep_limit = 0
    try:
        plain = run_gpu(cfg, x, anchors, W, pe, dY, variant, prepare=spy)
    finally:
        _LUTDataManager.product_keep_limit = saved
    assert not seen["kept"]
    assert np.array_equal(kept["y"], plain["y"])
    assert np.array_equal(kept["dW"], plain["dW"])   # same integer counts into the same contraction
    golden_util.assert_close(kept["dX"], plain["dX"], 1e-6, "dX")   # (shared-memory atomics: order of the adds varies)
    golden_util.assert_close(kept["dPE"], plain["dPE"], 1e-6, "dPE")
    # the C ABI's own statement of when the flags take effect
    dm = seen["dm"]
    c = dm._cfg(0.0, sliced=False)
    L = _native.lib()
    full = L.lutb_product_workspace(ctypes.byref(c), cfg["B"], cfg["S"], 1)
    one = L.lutb_product_workspace(ctypes.byref(c), 1, cfg["S"], 1)
    buf = torch.empty(full, dtype=torch.uint8, device="cuda")
    e = cfg["E"]
    assert L.lutb_product_keeps_histogram(ctypes.byref(c), cfg["B"], cfg["S"], e, e, variant, buf.data_ptr(), full) == 1
    # room for one sequence only (the FMA contraction's uint16 counters are half the size: two of them fit `one`)
    small = one if variant == 2 else one // 3
    assert L.lutb_product_keeps_histogram(ctypes.byref(c), cfg["B"], cfg["S"], e, e, variant, buf.data_ptr(), small) == 0
    assert L.lutb_product_keeps_histogram(ctypes.byref(c), cfg["B"], cfg["S"], e, e, 1, buf.data_ptr(), full) == 0
