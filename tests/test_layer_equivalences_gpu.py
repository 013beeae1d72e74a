"""Equivalences the reference's own tests rely on, checked between independent CUDA paths at sizes beyond the fixtures:
a sparse layer whose every detector reaches every output computes what the fully connected layer computes
(reference: src/spiky/lut/tests/test_lut_fully_connected_small.py), and a product-mode sequence layer computes what
a plain layer computes on the materialised pair vectors [x_i | x_j | pe(j-i-1)] (test_lut_transformer_product.py)."""
import numpy as np
import pytest
import torch

import golden_util
import synth

pytestmark = pytest.mark.gpu
REL = 1e-5


def test_sparse_layer_with_full_connectivity_equals_fully_connected():
    from spiky_b200.lut_layer import Conv2DLUTLayer, SynapseMeta

    meta = SynapseMeta(min_weight=-1.0, max_weight=1.0)
    # one receptive field over the whole 12x12 input with a 6x7 block of detectors; one output window over all of
    # them with a 5x9 block of outputs: 42 detectors, each connected to all 45 outputs (two synapse groups of 32)
    common = dict(input_shape=(12, 12), n_anchors_per_detector=6, detectors_shape=(6, 7), output_kernel_shape=(5, 9),
                  receptive_field_shape=(12, 12), receptive_field_stride_shape=(12, 12), synapse_meta=meta,
                  random_seed=4, device="cuda:0")
    sparse = Conv2DLUTLayer(lut_receptive_field_shape=(6, 7), lut_receptive_field_stride_shape=(6, 7), **common)
    dense = Conv2DLUTLayer(_explicit_anchors=sparse._detector_anchors.cpu(), **common)
    Nt, T, O = 42, 64, 45
    assert sparse.n_detectors() == Nt and sparse.n_outputs() == O and dense.n_outputs() == O
    index = sparse._lut_dm._sparse
    assert int(index.det_count.min()) == O and int(index.det_count.max()) == O
    # weight slot of (detector, row, synapse p) in the sparse layout, and the output that synapse feeds
    wbase = index.det_wbase.cpu().numpy().astype(np.int64)
    stride = index.det_stride.cpu().numpy().astype(np.int64)
    tgt = index.syn_target.cpu().numpy().reshape(Nt, O).astype(np.int64)
    p = np.arange(O)
    slot = (wbase[:, None, None] + np.arange(T)[None, :, None] * stride[:, None, None]
            + (p + 2 * (p // index.group_size))[None, None, :])                       # [Nt, T, O] by synapse
    fc_cell = (np.arange(Nt)[:, None, None] * T + np.arange(T)[None, :, None]) * O + tgt[:, None, :]
    W = synth.normal(21, (Nt * T * O,), 0.0, 0.05)
    Ws = np.zeros(index.n_weights, dtype=np.float32)
    Ws[slot.reshape(-1)] = W[fc_cell.reshape(-1)]
    with torch.no_grad():
        dense._weights.copy_(torch.from_numpy(W))
        sparse._weights.copy_(torch.from_numpy(Ws))
    B = 300
    x = torch.from_numpy(synth.sparse_images(22, (B, 144))).view(B, 1, 12, 12).cuda()
    dY = torch.from_numpy(synth.normal(23, (B, O))).view(B, 1, 5, 9).cuda()
    out = {}
    for name, layer in (("sparse", sparse), ("dense", dense)):
        layer.train()
        y, idx, md, mk = layer.forward_step(x)
        dx, dw = layer.backward_step(x, dY, idx, md, mk)
        torch.cuda.synchronize()
        out[name] = (y.cpu().numpy(), idx.cpu().numpy(), md.cpu().numpy(), mk.cpu().numpy(), dx.cpu().numpy(),
                     dw.cpu().numpy())
    ys, idxs, mds, mks, dxs, dws = out["sparse"]
    yd, idxd, mdd, mkd, dxd, dwd = out["dense"]
    assert np.array_equal(idxs, idxd) and np.array_equal(mks, mkd) and np.array_equal(mds, mdd)
    golden_util.assert_close(ys, yd, REL, "y")
    golden_util.assert_close(dxs, dxd, REL, "dX")
    golden_util.assert_close(dws[slot.reshape(-1)], dwd[fc_cell.reshape(-1)], REL, "dW")


@pytest.mark.parametrize("variant", [1, 2, 3])
def test_product_layer_equals_plain_layer_on_materialised_pairs(variant):
    from spiky_b200.lut_layer import LUTLayer, SynapseMeta

    B, S, E, Npe, Nt, Nc, O = 3, 40, 24, 6, 5, 6, 16
    meta = SynapseMeta(min_weight=-1.0, max_weight=1.0)
    rng = np.random.default_rng(31)
    # anchors over the virtual vector [x_i | x_j | pe]; both ends distinct
    a1 = rng.integers(0, 2 * E + Npe, size=(Nt, Nc))
    a2 = (a1 + rng.integers(1, 2 * E + Npe, size=(Nt, Nc))) % (2 * E + Npe)
    anchors = np.stack([a1, a2], axis=-1).astype(np.int32)
    product = LUTLayer(E, Nc, Nt, O, sequence_length=S, synapse_meta=meta, concatenation_product=False,
                       positional_dim=Npe, _explicit_anchors=torch.from_numpy(anchors.reshape(-1).copy()),
                       random_seed=1, device="cuda:0")
    # plain layer over [x_i | x_j | pe[d, 0, :] | ... | pe[d, Nt-1, :]]: detector t reads its own embedding
    I2 = 2 * E + Nt * Npe
    shifted = np.where(anchors >= 2 * E, anchors + np.arange(Nt, dtype=np.int32)[:, None, None] * Npe, anchors)
    plain = LUTLayer(I2, Nc, Nt, O, synapse_meta=meta, _explicit_anchors=torch.from_numpy(shifted.reshape(-1).copy()),
                     random_seed=1, device="cuda:0")
    W = synth.normal(32, (Nt * (1 << Nc) * O,), 0.0, 0.05)
    pe = synth.uniform(33, ((S - 1) * Nt * Npe,), -1.0, 1.0)
    with torch.no_grad():
        product._weights.copy_(torch.from_numpy(W))
        plain._weights.copy_(torch.from_numpy(W))
        product._positional_embeddings.copy_(torch.from_numpy(pe))
    product._product_variant = variant
    product.train()
    plain.train()
    x = torch.from_numpy(synth.normal(34, (B, S, E))).cuda()
    dY = torch.from_numpy(synth.normal(35, (B, S, O))).cuda()
    pos = product._prepare_positional_embeddings().detach()
    y = product.forward_step_product(x, pos)
    dx, dw, dpe = product.backward_step_product(x, pos, dY)
    # materialise every causal pair
    ii, jj = torch.triu_indices(S, S, offset=1, device="cuda")
    P = ii.numel()
    pe_t = torch.from_numpy(pe).cuda().view(S - 1, Nt * Npe)
    xp = torch.cat([x[:, ii], x[:, jj], pe_t[jj - ii - 1].unsqueeze(0).expand(B, P, -1)], dim=2).reshape(B * P, 1, I2)
    yp, idx, md, mk = plain.forward_step(xp.contiguous())
    dYp = dY[:, jj].reshape(B * P, 1, O).contiguous()
    dxp, dwp = plain.backward_step(xp.contiguous(), dYp, idx, md, mk)
    torch.cuda.synchronize()
    y2 = torch.zeros(B, S, O, device="cuda").index_add_(1, jj, yp.view(B, P, O))
    dxp = dxp.view(B, P, I2)
    dx2 = torch.zeros(B, S, E, device="cuda")
    dx2.index_add_(1, ii, dxp[:, :, :E])
    dx2.index_add_(1, jj, dxp[:, :, E:2 * E])
    dpe2 = torch.zeros(S - 1, Nt * Npe, device="cuda").index_add_(0, jj - ii - 1, dxp[:, :, 2 * E:].sum(0))
    golden_util.assert_close(y.cpu().numpy(), y2.cpu().numpy(), REL, "y")
    golden_util.assert_close(dx.cpu().numpy(), dx2.cpu().numpy(), REL, "dX")
    golden_util.assert_close(dw.cpu().numpy(), dwp.cpu().numpy(), REL, "dW")
    golden_util.assert_close(dpe.cpu().numpy().reshape(-1), dpe2.cpu().numpy().reshape(-1), REL, "dPE")
