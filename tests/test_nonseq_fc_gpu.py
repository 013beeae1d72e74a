"""CUDA path of the non-sequence fully connected layer, called through the C ABI, against
(1) the golden vectors recorded from the reference and (2) the CPU oracle on larger seeded inputs.

Bar: indices, min-margin anchors, min deltas and every fixed-point (int32) result bit-exact;
fp32 outputs and gradients within 1e-5 of the tensor's scale (summation order only)."""
import numpy as np
import pytest
import torch

import golden_util
import synth
from cases import nonseq_fc_inputs
from oracle import lut_oracle as orc

pytestmark = pytest.mark.gpu
REL = 1e-5


def make_dm(cfg):
    from spiky_b200.lut_data_manager import LUTDataManagerF, LUTDataManagerI

    args = (cfg["I"], cfg["O"], cfg["Nt"], cfg["Nc"], 1, 0, 0, cfg.get("G", 32), cfg.get("Gb", 32))
    dm = LUTDataManagerI(*args, cfg.get("int_rescaler", 0.001)) if cfg.get("int_mode") else LUTDataManagerF(*args)
    dm.register_synapse_meta(learning_rate=cfg.get("lr_meta", 1.0), min_synaptic_weight=-1.0, max_synaptic_weight=1.0,
                             initial_noise_level=0.0, initial_weight=0.0)
    dm.initialize_neurons(True)
    dm.to_device(0)
    return dm


def run_gpu(cfg, x, anchors, W, dY, dw_variant=0):
    dev = torch.device("cuda:0")
    dm = make_dm(cfg)
    B, I, Nt, O = cfg["B"], cfg["I"], cfg["Nt"], cfg["O"]
    tW = torch.from_numpy(W).to(dev)
    tx = torch.from_numpy(x).reshape(-1).to(dev)
    ta = torch.from_numpy(anchors).reshape(-1).to(dev)
    eps = cfg.get("cmp_eps", 0.0)
    out = {}
    y_eval = torch.zeros(B * O, device=dev)
    idx_eval = torch.zeros(B * Nt, dtype=torch.int32, device=dev)
    dm.forward_step(tW, B, tx, ta, y_eval, idx_eval, eps, None, None, None)
    y = torch.zeros(B * O, device=dev)
    idx = torch.zeros(B * Nt, dtype=torch.int32, device=dev)
    md = torch.zeros(B * Nt, device=dev)
    mk = torch.zeros(B * Nt, dtype=torch.int32, device=dev)
    dm.forward_step(tW, B, tx, ta, y, idx, eps, None, md, mk)
    dX = torch.zeros(B * I, device=dev)
    internal = cfg.get("policy") == "internal"
    dW = None if internal else torch.zeros_like(tW)
    dm.backward_backprop(tW, B, torch.from_numpy(dY).reshape(-1).to(dev), ta, idx, md, mk, dX,
                         cfg["ext_lr"] if internal else -1.0, dW, None, dw_variant=dw_variant)
    torch.cuda.synchronize()
    out.update(y_eval=y_eval.cpu().numpy().reshape(B, O), idx_eval=idx_eval.cpu().numpy().reshape(B, Nt),
               y=y.cpu().numpy().reshape(B, O), idx=idx.cpu().numpy().reshape(B, Nt),
               min_delta=md.cpu().numpy().reshape(B, Nt), min_k=mk.cpu().numpy().reshape(B, Nt),
               dX=dX.cpu().numpy().reshape(B, I))
    if internal:
        out["W_after"] = tW.cpu().numpy()
    else:
        out["dW"] = dW.cpu().numpy()
    return out


def compare(cfg, got, ref):
    assert np.array_equal(got["idx"], ref["idx"]) and np.array_equal(got["idx_eval"], ref["idx"])
    assert np.array_equal(got["min_k"], ref["min_k"])
    assert np.array_equal(got["min_delta"].view(np.int32), ref["min_delta"].view(np.int32))
    keys = ["y", "y_eval", "dX"] + (["W_after"] if "W_after" in ref else ["dW"])
    for k in keys:
        if cfg.get("int_mode"):
            assert np.array_equal(got[k], ref[k]), f"{k}: fixed-point results must be bit-exact"
        else:
            golden_util.assert_close(got[k], ref[k], REL, k)


@pytest.mark.parametrize("name", golden_util.names("fc_"))
def test_nonseq_fc_matches_reference_golden(name):
    cfg, ref = golden_util.load(name)
    x, anchors, W, dY = nonseq_fc_inputs(cfg)
    compare(cfg, run_gpu(cfg, x, anchors, W, dY), ref)


def oracle_reference(cfg, x, anchors, W, dY):
    kw = dict(int_mode=cfg.get("int_mode", False), int_rescaler=cfg.get("int_rescaler", 0.001))
    y, idx, md, mk = orc.nonseq_fc_forward(W, x, anchors, cfg["Nt"], cfg["Nc"], cfg["O"], cfg.get("cmp_eps", 0.0),
                                           True, cfg.get("Gb", 32), **kw)
    dX, dW = orc.nonseq_fc_backward(W, dY, anchors, idx, md, mk, cfg["I"], cfg["Nc"], cfg.get("lr_meta", 1.0), -1.0,
                                    cfg.get("G", 32), **kw)
    return dict(y=y, y_eval=y, idx=idx, min_delta=md, min_k=mk, dX=dX, dW=dW)


ORACLE_CASES = {
    # the single-layer benchmark configuration at full size (batch 256 x 784 -> 64 tables x 6 pairs -> 32)
    "c1_full_f32": dict(seed=500, B=256, I=784, Nt=64, Nc=6, O=32),
    "c1_full_i32": dict(seed=501, B=256, I=784, Nt=64, Nc=6, O=32, int_mode=True),
    "c1_sparse_images": dict(seed=502, B=64, I=784, Nt=64, Nc=6, O=32, sparse_input=True),
    # output rows wider than one warp pass, table of 256 rows, odd batch
    "ffn_like": dict(seed=503, B=67, I=256, Nt=16, Nc=8, O=1024),
    "ffn_like_i32": dict(seed=504, B=33, I=256, Nt=16, Nc=8, O=640, int_mode=True, int_rescaler=0.01),
    # outputs not a multiple of 4 (scalar path), many detectors
    "ragged": dict(seed=505, B=19, I=333, Nt=150, Nc=5, O=10),
    "ragged_i32": dict(seed=506, B=19, I=333, Nt=150, Nc=5, O=10, int_mode=True, G=3, Gb=7),
    # every lane-group width of the vectorised forward gather: 1, 2, 4, 8 (c1), 16 (c5), 32 float4 per row, two chunks
    "rows_of_4": dict(seed=510, B=37, I=64, Nt=45, Nc=5, O=4),
    "rows_of_8": dict(seed=511, B=37, I=64, Nt=45, Nc=5, O=8),
    "rows_of_16": dict(seed=512, B=37, I=64, Nt=45, Nc=5, O=16),
    "rows_of_128": dict(seed=513, B=21, I=64, Nt=33, Nc=5, O=128),
    "rows_of_260": dict(seed=514, B=21, I=64, Nt=33, Nc=5, O=260),
    # one sample; more detectors than threads of a row group; inputs not a multiple of 4
    "one_sample": dict(seed=515, B=1, I=50, Nt=300, Nc=7, O=12),
    "odd_inputs": dict(seed=516, B=13, I=4099, Nt=64, Nc=8, O=32, normal_input=True),
    # input rows so long that fewer rows are staged together (2, then 1), and rows that do not fit shared memory at all
    "inputs_10k": dict(seed=517, B=5, I=10001, Nt=20, Nc=5, O=8, normal_input=True),
    "inputs_20k": dict(seed=518, B=3, I=20002, Nt=20, Nc=5, O=8, normal_input=True),
    "inputs_60k": dict(seed=519, B=3, I=60001, Nt=20, Nc=5, O=8, normal_input=True),
    # a slice of the large inference layer (4096 inputs, 8 pairs, 64 outputs)
    "c5_slice": dict(seed=507, B=40, I=4096, Nt=512, Nc=8, O=64, normal_input=True),
    "nan_inputs": dict(seed=508, B=8, I=32, Nt=8, Nc=4, O=8, nan_input=True),
}


@pytest.mark.parametrize("name", sorted(ORACLE_CASES))
def test_nonseq_fc_matches_oracle(name):
    cfg = ORACLE_CASES[name]
    x, anchors, W, dY = nonseq_fc_inputs(cfg)
    if cfg.get("nan_input"):
        x[:, 3] = np.nan  # NaN deltas: bit 0, never the minimum unless first (reference compare semantics)
    ref = oracle_reference(cfg, x, anchors, W, dY)
    got = run_gpu(cfg, x, anchors, W, dY)
    if cfg.get("nan_input"):
        assert np.array_equal(got["idx"], ref["idx"]) and np.array_equal(got["min_k"], ref["min_k"])
        return
    compare(cfg, got, ref)


def test_large_batch_properties():
    """Full-size batch of the single-layer configuration: size-independent properties.
    (1) duplicating the batch doubles dW and leaves per-sample outputs unchanged;
    (2) dX rows sum to zero (+du and -du per detector); (3) two runs give identical indices."""
    cfg = dict(seed=600, B=8192, I=784, Nt=64, Nc=6, O=32)
    x, anchors, W, dY = nonseq_fc_inputs(cfg)
    a = run_gpu(cfg, x, anchors, W, dY)
    cfg2 = dict(cfg, B=2 * cfg["B"])
    b = run_gpu(cfg2, np.concatenate([x, x]), anchors, W, np.concatenate([dY, dY]))
    assert np.array_equal(b["idx"][: cfg["B"]], a["idx"]) and np.array_equal(b["idx"][cfg["B"]:], a["idx"])
    golden_util.assert_close(b["y"][: cfg["B"]], a["y"], 1e-6, "y")
    golden_util.assert_close(b["dW"], 2.0 * a["dW"], REL, "dW linearity")
    assert np.abs(a["dX"].astype(np.float64).sum(axis=1)).max() <= 1e-4 * np.abs(a["dX"]).max()
    sample = slice(0, 64)
    ref = oracle_reference(dict(cfg, B=64), x[sample], anchors, W, dY[sample])
    assert np.array_equal(a["idx"][sample], ref["idx"])
    golden_util.assert_close(a["y"][sample], ref["y"], REL, "y vs oracle")
    golden_util.assert_close(a["dX"][sample], ref["dX"], REL, "dX vs oracle")


def test_runtime_errors_mirror_reference():
    dm = make_dm(dict(I=8, O=4, Nt=4, Nc=2))
    dev = torch.device("cuda:0")
    w = torch.zeros(4 * 4 * 4, device=dev)
    with pytest.raises(RuntimeError):  # dtype mismatch -> RuntimeError like checkTensor
        dm.forward_step(w, 1, torch.zeros(8, device=dev, dtype=torch.float64), torch.zeros(16, dtype=torch.int32, device=dev),
                        torch.zeros(4, device=dev), torch.zeros(4, dtype=torch.int32, device=dev))
    with pytest.raises(ValueError):  # backward before any forward -> "no active context"
        dm.backward_backprop(w, 1, torch.zeros(4, device=dev), torch.zeros(16, dtype=torch.int32, device=dev),
                             torch.zeros(4, dtype=torch.int32, device=dev), torch.zeros(4, device=dev),
                             torch.zeros(4, dtype=torch.int32, device=dev), torch.zeros(8, device=dev), -1.0,
                             torch.zeros_like(w))
    with pytest.raises(ValueError):
        dm.forward_step(w, 0, torch.zeros(8, device=dev), torch.zeros(16, dtype=torch.int32, device=dev),
                        torch.zeros(4, device=dev), torch.zeros(4, dtype=torch.int32, device=dev))


@pytest.mark.parametrize("name", ["c1_full_f32", "ragged", "ffn_like"])
def test_sorted_table_gradient_is_bit_exact_and_deterministic(name):
    """LUTB_DW_SORTED adds every cell's contributions in ascending sample order with one fp32 rounding each,
    the order of the reference's host loop: dW equals the oracle's bit for bit, run after run."""
    cfg = ORACLE_CASES[name]
    x, anchors, W, dY = nonseq_fc_inputs(cfg)
    ref = oracle_reference(cfg, x, anchors, W, dY)
    a = run_gpu(cfg, x, anchors, W, dY, dw_variant=3)
    b = run_gpu(cfg, x, anchors, W, dY, dw_variant=3)
    assert np.array_equal(a["dW"], ref["dW"])
    assert np.array_equal(a["dW"], b["dW"])
    golden_util.assert_close(a["dX"], ref["dX"], REL, "dX")


def test_sorted_variant_rejects_missing_workspace():
    import ctypes
    from spiky_b200 import _native

    dm = make_dm(dict(I=8, O=4, Nt=4, Nc=2))
    cfg = dm._cfg()
    L = _native.lib()
    need = L.lutb_nonseq_fc_backward_workspace(ctypes.byref(cfg), 16, 3)
    assert need > 0 and L.lutb_nonseq_fc_backward_workspace(ctypes.byref(cfg), 16, 1) == 0
    dev = torch.device("cuda:0")
    t = lambda n, dt=torch.float32: torch.zeros(n, dtype=dt, device=dev)
    p = lambda z: ctypes.c_void_p(z.data_ptr())
    rc = L.lutb_nonseq_fc_backward(ctypes.byref(cfg), 16, p(t(64)), p(t(64)), p(t(16, torch.int32)), p(t(64, torch.int32)),
                                   p(t(64)), p(t(64, torch.int32)), p(t(128)), p(t(64)), -1.0, 3, None, 0, None)
    assert rc == -4 and b"workspace" in L.lutb_last_error()
