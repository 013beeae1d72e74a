"""Query-range stages of the concatenation-mode layer on the GPU at the reference notebook's table size
(6 anchor pairs, 4 positional dims: 2^16 rows per detector), through the C ABI: the two halves of the queries, run
one after the other the way two ranks would run them, add up to the unsharded layer and to the oracle."""
import numpy as np
import pytest
import torch

import golden_util
from oracle import lut_oracle as orc

pytestmark = pytest.mark.gpu
REL = 1e-5


def test_query_ranges_add_up_to_the_unsharded_layer_and_the_oracle():
    from spiky_b200.lut_layer import LUTLayer, SynapseMeta

    B, S, E, Nt, Nc, Npe, O = 2, 16, 32, 8, 6, 4, 32
    layer = LUTLayer(E, Nc, Nt, O, sequence_length=S, synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
                     concatenation_product=True, positional_dim=Npe, random_seed=5, device="cuda:0")
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        layer._weights.copy_(torch.empty(layer._weights.shape).normal_(0.0, 0.05, generator=g))
    layer.train()
    x = (torch.rand(B, S, E, generator=g) * 2 - 1)
    dy = torch.randn(B, S, O, generator=g)
    W = layer._weights.detach().cpu().numpy()
    anchors = layer._detector_anchors.cpu().numpy()
    pe = layer._prepare_positional_embeddings().detach()
    pe3 = pe.cpu().numpy().reshape(S - 1, Nt, Npe)

    # oracle
    y_ref, state = orc.concat_forward(W, x.numpy(), pe3, anchors, Nt, Nc, O, Npe)
    dX_ref, dW_ref, dPE_ref = orc.concat_backward(W, dy.numpy(), anchors, state, E, Nc, Npe)

    # unsharded layer
    xt, dyt = x.cuda(), dy.cuda()
    y, idx, md, mk, pidx, pmd, pmk = layer.forward_step_concat(xt, pe)
    dx, dw, dpe = layer.backward_step_concat(xt, dyt, idx, md, mk, pidx, pmd, pmk)
    torch.cuda.synchronize()
    assert np.array_equal(idx.cpu().numpy().reshape(B * S, Nt), state["idx"])
    golden_util.assert_close(y.cpu().numpy().reshape(B, S, O), y_ref, REL, "y")
    golden_util.assert_close(dx.cpu().numpy().reshape(B, S, E), dX_ref, REL, "dX")
    golden_util.assert_close(dw.cpu().numpy(), dW_ref, REL, "dW")
    golden_util.assert_close(dpe.cpu().numpy(), dPE_ref, REL, "dPE")

    # the two halves of the queries, each from the table indices of ALL tokens
    dm = layer._lut_dm
    dev = xt.device
    idx2 = torch.empty(B * S * Nt, dtype=torch.int32, device=dev)
    md2 = torch.empty(B * S * Nt, dtype=torch.float32, device=dev)
    mk2 = torch.empty(B * S * Nt, dtype=torch.int32, device=dev)
    dm.check_detectors(B * S, xt.view(-1), layer._detector_anchors, idx2, 0.0, md2, mk2)
    pidx2 = torch.empty((S - 1) * Nt, dtype=torch.int32, device=dev)
    pmd2 = torch.empty((S - 1) * Nt, dtype=torch.float32, device=dev)
    pmk2 = torch.empty((S - 1) * Nt, dtype=torch.int32, device=dev)
    dm.check_positional(pe.contiguous().view(-1), pidx2, 0.0, pmd2, pmk2)
    assert torch.equal(idx2, idx.reshape(-1)) and torch.equal(mk2, mk.reshape(-1)) and torch.equal(md2, md.reshape(-1))
    assert torch.equal(pidx2, pidx.reshape(-1)) and torch.equal(pmk2, pmk.reshape(-1))
    y_parts, sums = [], None
    for j0, j1 in ((0, S // 2), (S // 2, S)):
        yp = torch.zeros(B * S * O, device=dev)
        dm.concat_pairs_forward(layer._weights.detach(), B, idx2, pidx2, yp, j0, j1)
        yp = yp.view(B, S, O)
        assert not yp[:, :j0].any() and not yp[:, j1:].any(), "a rank writes the rows of its own queries only"
        y_parts.append(yp)
        dX = torch.zeros(B * S * E, device=dev)
        dW = torch.zeros_like(layer._weights)
        dPE = torch.zeros((S - 1) * Nt * Npe, device=dev)
        dm.concat_pairs_backward(layer._weights.detach(), B, dyt.contiguous().view(-1), layer._detector_anchors, idx2, md2,
                                 mk2, dX, -1.0, pidx2, pmd2, pmk2, dPE, dW, j0, j1)
        parts = (dX, dW.detach(), dPE)
        sums = parts if sums is None else tuple(a + b for a, b in zip(sums, parts))
    torch.cuda.synchronize()
    # (the detectors of a query add into its output row in no fixed order, so the sums agree to rounding only)
    golden_util.assert_close((y_parts[0] + y_parts[1]).cpu().numpy(), y_ref, REL, "sum of the two query ranges")
    golden_util.assert_close(sums[0].cpu().numpy().reshape(B, S, E), dX_ref, REL, "sum of partial dX")
    golden_util.assert_close(sums[1].cpu().numpy(), dW_ref, REL, "sum of partial dW")
    golden_util.assert_close(sums[2].cpu().numpy(), dPE_ref, REL, "sum of partial dPE")
    # the first half's pairs never touch the second half's tokens
    assert y_parts[0][:, S // 2:].abs().sum() == 0


def test_query_range_is_validated():
    from spiky_b200.lut_layer import LUTLayer, SynapseMeta

    layer = LUTLayer(8, 2, 2, 4, sequence_length=4, synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
                     concatenation_product=True, positional_dim=2, random_seed=5, device="cuda:0")
    dm = layer._lut_dm
    idx = torch.zeros(4 * 2, dtype=torch.int32, device="cuda:0")
    pidx = torch.zeros(3 * 2, dtype=torch.int32, device="cuda:0")
    y = torch.zeros(4 * 4, device="cuda:0")
    with pytest.raises(ValueError, match="query range"):
        dm.concat_pairs_forward(layer._weights.detach(), 1, idx, pidx, y, 2, 9)
