"""The benchmark configurations at their own shapes, CUDA library against the oracle, at the reference's own bar
(1e-5, src/spiky/lut/tests/test_lut_fully_connected_small.py:119,126; indices and fixed-point results bit-exact).

  conv-net     the default bench workload (bench.SparseConvNetWorkload, batch 512): every layer forward + backward
  transformer  the character-level model of bench.CharTransformerWorkload (d_model 256, 4 layers, context 128)
  attention    one head of the large transformer's attention layer (context 1024, 1024-row tables, 1024 outputs)
  inference    the large single layer (4096 inputs, 4096 tables x 8 pairs, 64 outputs), fp32 and int8 tables

Each layer is given the ORACLE's activations of the layer below as its input: table indices are discontinuous in the
input, so one last-bit difference between two summation orders can flip an index further up and turn a rounding
difference into a different table row; layer by layer on identical inputs every index must agree exactly.
Where a sum is too long for two fp32 summation orders to agree to 1e-5, both results are compared with an fp64
accumulation of the same terms and the CUDA result must be as close to it as the oracle's is (fp64_* helpers).
"""
import os
import sys

import numpy as np
import pytest
import torch

import golden_util
from oracle import lut_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu
REL = 1e-5


def close_or_as_close_as_oracle(got, ref, exact64, what):
    """|got - ref| <= 1e-5 max|ref|; failing that, got must be no further from the fp64 result than the oracle is
    (both are fp32 sums of the same terms in different orders)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    scale = max(np.abs(ref).max(), 1e-30)
    err = np.abs(got - ref).max()
    if err <= REL * scale:
        return
    assert exact64 is not None, f"{what}: max abs err {err:.3e} > {REL:g} * {scale:.3e}"
    e_got, e_ref = np.abs(got - exact64).max(), np.abs(ref - exact64).max()
    assert e_got <= max(1.5 * e_ref, REL * scale), (
        f"{what}: CUDA is {e_got:.3e} from the fp64 sum, the oracle {e_ref:.3e} (scale {scale:.3e})")


# ------------------------------------------------------------------------------------------ conv-net
@pytest.mark.parametrize("internal", [False, True])
def test_sparse_convnet_step_at_batch_512(internal):
    import bench
    from spiky_b200 import _native

    wl = bench.SparseConvNetWorkload(batch=512, internal=internal)
    layers = wl.build(torch.device("cuda:0"))
    for l in layers:
        l.train()
    B = wl.B
    x, labels = wl.host_inputs(1000, B)
    I, O, Nt, Nc = wl.READOUT
    lr = wl.LR

    # oracle forward; the CUDA layer gets the oracle's input
    acts, saved, gpu_saved = [x], [], []
    for l in layers[:-1]:
        index = l._lut_dm._sparse
        sp = dict(index.numpy(), group_size=index.group_size)
        W = l._weights.detach().cpu().numpy().copy()
        an = l._detector_anchors.cpu().numpy()
        y, idx, md, mk = orc.nonseq_sparse_forward(W, acts[-1], an, sp, wl.NC, l.n_outputs())
        xt = torch.from_numpy(acts[-1]).view((B, 1) + tuple(l.input_shape())).cuda()
        gy, gidx, gmd, gmk = l.forward_step(xt)
        torch.cuda.synchronize()
        assert np.array_equal(gidx.cpu().numpy().reshape(idx.shape), idx), "table indices"
        assert np.array_equal(gmk.cpu().numpy().reshape(mk.shape), mk), "minimum-margin pairs"
        assert np.array_equal(gmd.cpu().numpy().reshape(md.shape).view(np.int32), md.view(np.int32)), "min deltas"
        golden_util.assert_close(gy.cpu().numpy().reshape(y.shape), y, REL, "y")
        saved.append((W, an, sp, idx, md, mk))
        gpu_saved.append((xt, gidx, gmd, gmk))
        acts.append(y)
    r = layers[-1]
    Wr, Ar = r._weights.detach().cpu().numpy().copy(), r._detector_anchors.cpu().numpy()
    logits, ridx, rmd, rmk = orc.nonseq_fc_forward(Wr, acts[-1], Ar, Nt, Nc, O)
    xr = torch.from_numpy(acts[-1]).view(B, 1, I).cuda()
    glog, gridx, grmd, grmk = r.forward_step(xr)
    assert np.array_equal(gridx.cpu().numpy().reshape(ridx.shape), ridx)
    golden_util.assert_close(glog.cpu().numpy().reshape(logits.shape), logits, REL, "logits")

    # cross-entropy gradient on the oracle's logits, then backward layer by layer on the oracle's gradients
    z = logits - logits.max(axis=1, keepdims=True)
    p = np.exp(z)
    p /= p.sum(axis=1, keepdims=True)
    p[np.arange(B), labels] -= 1.0
    g = (p / B).astype(np.float32)

    def check_update(layer, W_before, dW_ref, gdw, what):
        if internal:
            want = W_before - np.float32(lr) * dW_ref
            golden_util.assert_close(layer._weights.detach().cpu().numpy(), want, REL, what + " W_after")
        else:
            golden_util.assert_close(gdw.cpu().numpy().reshape(-1), dW_ref.reshape(-1), REL, what + " dW")

    dX, dW = orc.nonseq_fc_backward(Wr, g, Ar, ridx, rmd, rmk, I, Nc)
    gdx, gdw = r.backward_step(xr, torch.from_numpy(g).view(B, 1, O).cuda(), gridx, grmd, grmk)
    golden_util.assert_close(gdx.cpu().numpy().reshape(dX.shape), dX, REL, "readout dX")
    check_update(r, Wr, dW, gdw, "readout")
    g = dX
    for li in (2, 1, 0):
        l = layers[li]
        W, an, sp, idx, md, mk = saved[li]
        xt, gidx, gmd, gmk = gpu_saved[li]
        dX, dW = orc.nonseq_sparse_backward(W, g, an, idx, md, mk, sp, l.n_inputs(), wl.NC)
        gdx, gdw = l.backward_step(xt, torch.from_numpy(g).view((B, 1) + tuple(l.output_shape())).cuda(), gidx, gmd, gmk)
        torch.cuda.synchronize()
        golden_util.assert_close(gdx.cpu().numpy().reshape(dX.shape), dX, REL, f"layer {li} dX")
        check_update(l, W, dW, gdw, f"layer {li}")
        g = dX
    assert _native.device_wait_errors() == 0


def test_sparse_convnet_loss_of_the_chained_step_matches_the_oracle():
    """The whole step as bench.py runs it (layers chained on the GPU) gives the oracle's loss: an index flipped by a
    last-bit difference further down moves the mean loss of 512 samples by far less than 1e-4."""
    import bench

    wl = bench.SparseConvNetWorkload(batch=512)
    wl.setup(torch.device("cuda:0"), 0)
    x, labels = wl.host_inputs(1000, wl.B)
    loss = float(wl._run(torch.from_numpy(x).view(wl.B, 1, 28, 28).cuda(), torch.from_numpy(labels).cuda()))
    assert abs(loss - wl.cpu_loss(x, labels)) <= 1e-4 * abs(loss)


# ------------------------------------------------------------------------------------------ character transformer
def oracle_transformer_tape(model, tokens, dlogits):
    """Oracle forward + backward of a product-mode LUTTransformer; one record per LUT layer with the layer's input,
    its upstream gradient and every result, so that the CUDA layer can be run on exactly the oracle's operands."""
    B, S = tokens.shape
    E, V = model._n_embeddings, model.vocab_size
    z = model.token_embedder.weight.detach().cpu().numpy()[tokens]
    tape = []
    for block in model.layers:
        att = block["attention_lut"]
        A, W = att._detector_anchors.cpu().numpy(), att._weights.detach().cpu().numpy()
        pe = att._prepare_positional_embeddings().detach().cpu().numpy().reshape(S - 1, att._n_detectors, -1)
        y = orc.product_forward(W, z, pe, A, att._n_detectors, att._n_anchors_per_detector, E, att._positional_dim)
        tape.append(dict(kind="att", layer=att, x=z.copy(), y=y, W=W, A=A, pe=pe))
        z = z + y
        ffn = block["ffn"]
        A2, W2 = ffn._detector_anchors.cpu().numpy(), ffn._weights.detach().cpu().numpy()
        y2, idx, md, mk = orc.nonseq_fc_forward(W2, z.reshape(B * S, E), A2, ffn._n_detectors, ffn._n_anchors_per_detector, E)
        tape.append(dict(kind="fc", layer=ffn, x=z.reshape(B * S, E).copy(), y=y2, W=W2, A=A2, idx=idx, md=md, mk=mk))
        z = z + y2.reshape(B, S, E)
    un = model.unembedder
    Au, Wu = un._detector_anchors.cpu().numpy(), un._weights.detach().cpu().numpy()
    logits, idx, md, mk = orc.nonseq_fc_forward(Wu, z.reshape(B * S, E), Au, un._n_detectors, un._n_anchors_per_detector, V)
    tape.append(dict(kind="fc", layer=un, x=z.reshape(B * S, E).copy(), y=logits, W=Wu, A=Au, idx=idx, md=md, mk=mk))
    dz = None
    for rec in reversed(tape):
        l = rec["layer"]
        if rec["kind"] == "fc":
            rec["dY"] = dlogits.reshape(B * S, V) if dz is None else dz.reshape(B * S, E)
            dx, dw = orc.nonseq_fc_backward(rec["W"], rec["dY"], rec["A"], rec["idx"], rec["md"], rec["mk"], E,
                                            l._n_anchors_per_detector)
            rec.update(dX=dx, dW=dw)
            dz = dx.reshape(B, S, E) if dz is None else dz + dx.reshape(B, S, E)
        else:
            rec["dY"] = dz.copy()
            dx, dw, dpe = orc.product_backward(rec["W"], rec["x"], rec["pe"], rec["A"], dz, l._n_detectors,
                                               l._n_anchors_per_detector, l._positional_dim)
            rec.update(dX=dx, dW=dw, dPE=dpe)
            dz = dz + dx
    return tape


def test_char_transformer_config_layer_by_layer():
    """d_model 256, 4 layers, 4 heads x 16 detectors, context 128, 2 sequences: every LUT layer of the model on the
    oracle's input and upstream gradient."""
    import bench

    wl = bench.CharTransformerWorkload(batch=2)
    model = wl.build(torch.device("cuda:0"))
    model.train()
    B, S, E, V = 2, wl.S, wl.E, wl.V
    tokens = wl.host_tokens(1000, B)[:, :-1].numpy()
    dlogits = (torch.randn(B, S, V, generator=torch.Generator().manual_seed(5)) / (B * S)).numpy()
    tape = oracle_transformer_tape(model, tokens, dlogits)
    assert len(tape) == 2 * wl.L + 1
    for n, rec in enumerate(tape):
        l, what = rec["layer"], f"layer {n} ({rec['kind']})"
        if rec["kind"] == "fc":
            rows = rec["x"].shape[0]
            xt = torch.from_numpy(rec["x"]).view(rows, 1, E).cuda()
            y, idx, md, mk = l.forward_step(xt)
            assert np.array_equal(idx.cpu().numpy().reshape(rec["idx"].shape), rec["idx"]), what
            assert np.array_equal(mk.cpu().numpy().reshape(rec["mk"].shape), rec["mk"]), what
            dx, dw = l.backward_step(xt, torch.from_numpy(rec["dY"]).view(rows, 1, -1).cuda(), idx, md, mk)
            dpe = None
        else:
            xt = torch.from_numpy(rec["x"]).cuda()
            pos = l._prepare_positional_embeddings().detach()
            y = l.forward_step_product(xt, pos)
            dx, dw, dpe = l.backward_step_product(xt, pos, torch.from_numpy(rec["dY"]).cuda())
        torch.cuda.synchronize()
        y64 = dw64 = None
        if rec["kind"] == "att":
            # an output of the attention layer sums up to 127 x 64 table rows, a table cell hundreds of gradient rows:
            # two fp32 summation orders need not agree to 1e-5; both are then held against the fp64 sums
            cfg = dict(B=B, S=S, E=E, Nt=l._n_detectors, Nc=l._n_anchors_per_detector, Npe=l._positional_dim, O=E)
            y64, dw64 = fp64_product_sums(cfg, rec["x"], rec["A"], rec["W"], rec["pe"], rec["dY"])
        close_or_as_close_as_oracle(y.cpu().numpy().reshape(rec["y"].shape), rec["y"], y64, what + " y")
        golden_util.assert_close(dx.cpu().numpy().reshape(rec["dX"].shape), rec["dX"], REL, what + " dX")
        close_or_as_close_as_oracle(dw.cpu().numpy().reshape(-1), rec["dW"].reshape(-1), dw64, what + " dW")
        if dpe is not None:
            golden_util.assert_close(dpe.cpu().numpy().reshape(-1), rec["dPE"].reshape(-1), REL, what + " dPE")


# ------------------------------------------------------------------------------------------ large attention layer
def fp64_product_sums(cfg, x, anchors, W, pe3, dY):
    """y and dW of a product-mode layer accumulated in fp64: per query j and detector t the selected rows are counted
    (H[j, t, r] = number of keys i < j whose pair picks row r; indices from the oracle's detector check on the
    materialised pair vectors [x_i | x_j | pe[j - i - 1, t]]), then y[j] = sum_t H[j, t] . W_t and
    dW_t = H[:, t]^T . dY in double."""
    B, S, E, Nt, Nc, Npe, O = (cfg[k] for k in ("B", "S", "E", "Nt", "Nc", "Npe", "O"))
    T = 1 << Nc
    anchors = np.asarray(anchors).reshape(Nt, Nc, 2)
    pe3 = None if pe3 is None else np.asarray(pe3).reshape(S - 1, Nt, Npe)
    W64 = W.reshape(Nt, T, O).astype(np.float64)
    y = np.zeros((B, S, O))
    dW = np.zeros((Nt, T, O))
    for b in range(B):
        H = np.zeros((S, Nt, T))
        pairs = np.empty((S - 1, 2 * E + Npe), np.float32)
        for j in range(1, S):
            # one block of pair vectors per query; only the positional columns depend on the detector
            blk = pairs[:j]
            blk[:, :E] = x[b, :j]
            blk[:, E:2 * E] = x[b, j]
            for t in range(Nt):
                if Npe:
                    blk[:, 2 * E:] = pe3[j - 1 - np.arange(j), t]
                idx = orc.check_detectors(blk, anchors[t:t + 1], 1, Nc, train=False).reshape(-1)
                H[j, t] = np.bincount(idx, minlength=T)
        for t in range(Nt):
            y[b] += H[:, t, :] @ W64[t]
            dW[t] += H[:, t, :].T @ dY[b].astype(np.float64)
    return y, dW.reshape(-1)


@pytest.mark.parametrize("variant", [1, 2, 3], ids=["direct", "histogram", "histogram_fma"])
def test_large_transformer_attention_head_shape(variant):
    """Context 1024, 1024-row tables, 1024 outputs, the 16 detectors of one head, one sequence."""
    from cases import sequence_inputs
    from test_product_gpu import run_gpu

    cfg = dict(seed=800, B=1, S=1024, E=1024, Nt=16, Nc=10, Npe=4, O=1024, n_virtual=2 * 1024 + 4)
    x, anchors, W, pe, dY = sequence_inputs(cfg, cfg["Nt"] * (1 << cfg["Nc"]) * cfg["O"], (cfg["S"] - 1) * cfg["Nt"] * cfg["Npe"])
    pe3 = pe.reshape(cfg["S"] - 1, cfg["Nt"], cfg["Npe"])
    ref = _large_attention_reference(cfg, x, anchors, W, pe3, dY)
    got = run_gpu(cfg, x, anchors, W, pe, dY, variant)
    close_or_as_close_as_oracle(got["y"], ref["y"], ref["y64"], "y")
    close_or_as_close_as_oracle(got["dW"], ref["dW"], ref["dW64"], "dW")
    golden_util.assert_close(got["dX"], ref["dX"], REL, "dX")
    golden_util.assert_close(got["dPE"].reshape(-1), ref["dPE"].reshape(-1), REL, "dPE")


_LARGE_REF = {}


def _large_attention_reference(cfg, x, anchors, W, pe3, dY):
    """Oracle results (and the fp64 sums) of the large attention case, computed once for both kernel variants."""
    if not _LARGE_REF:
        y = orc.product_forward(W, x, pe3, anchors, cfg["Nt"], cfg["Nc"], cfg["O"], cfg["Npe"])
        dX, dW, dPE = orc.product_backward(W, x, pe3, anchors, dY, cfg["Nt"], cfg["Nc"], cfg["Npe"])
        y64, dW64 = fp64_product_sums(cfg, x, anchors, W, pe3, dY)
        _LARGE_REF.update(y=y, dX=dX, dW=dW, dPE=dPE, y64=y64, dW64=dW64)
    return _LARGE_REF


# ------------------------------------------------------------------------------------------ large inference layer
def test_large_inference_layer_full_width():
    """4096 inputs, 4096 tables x 8 pairs, 64 outputs at batch 64: fp32 tables within 1e-5, int8 tables bit-exact under
    both de-quantisation rules."""
    import bench
    from spiky_b200.inference import LUTInference

    B = 64
    x = np.random.default_rng(7).standard_normal((B, 4096), dtype=np.float32)
    xt = torch.from_numpy(x).cuda()
    wl = bench.LutInferWorkload("fp32", batch=B)
    anchors, tables, _ = wl.structure()
    layer = LUTInference(wl.I, wl.O, wl.Nt, wl.Nc, anchors, tables, None, device=torch.device("cuda:0"))
    y = layer(xt).cpu().numpy()
    ref, ridx, _, _ = orc.nonseq_fc_forward(tables.numpy(), x, anchors.numpy(), wl.Nt, wl.Nc, wl.O, train=False)
    assert np.array_equal(layer.last_indices.cpu().numpy(), ridx)
    golden_util.assert_close(y, ref, REL, "fp32 tables")

    wl = bench.LutInferWorkload("int8", batch=B)
    anchors, q, s = wl.structure()
    for rule, exact in (("exact", True), ("f32", False)):
        layer = LUTInference(wl.I, wl.O, wl.Nt, wl.Nc, anchors, q, s, int_rescaler=0.05, dequant=rule,
                             device=torch.device("cuda:0"))
        acc = layer.partial(xt).cpu().numpy()
        want, widx = orc.infer_int8(q.numpy(), s.numpy(), x, anchors.numpy(), wl.Nt, wl.Nc, wl.O, int_rescaler=0.05,
                                    exact=exact)
        assert np.array_equal(layer.last_indices.cpu().numpy(), widx), rule
        assert np.array_equal(acc, want), rule
