"""Sparse gradient policy of fully connected layers: the (cell, value) lists taken straight from the table-gradient
pass (lutb_nonseq_fc_table_grad_rows) against the reference's route, the dense gradient compacted afterwards
(LUTLayer.py:567-609), and against the oracle."""
import ctypes

import numpy as np
import pytest
import torch

import golden_util
import synth
from oracle import lut_oracle as orc

pytestmark = pytest.mark.gpu


def make_layer(I, Nc, Nt, O, seed):
    from spiky_b200.lut_layer import LUTLayer, SynapseMeta, GradientPolicy, GradientType

    layer = LUTLayer(I, Nc, Nt, O, synapse_meta=SynapseMeta(learning_rate=0.5, min_weight=-1.0, max_weight=1.0),
                     weights_gradient_policy=GradientPolicy(GradientType.Sparse), random_seed=seed, device="cuda:0")
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(synth.normal(seed + 1, (layer._weights.numel(),), 0.0, 0.05)))
    layer.train()
    return layer


@pytest.mark.parametrize("shape", [(64, 40, 6, 4, 12), (300, 24, 5, 3, 10), (7, 30, 9, 6, 33), (2100, 16, 3, 5, 8)])
def test_row_lists_equal_the_compacted_dense_gradient(shape):
    from spiky_b200.torch_utils import DenseToSparseConverter
    from spiky_b200 import _native

    B, I, Nt, Nc, O = shape
    layer = make_layer(I, Nc, Nt, O, seed=40 + B)
    x = torch.from_numpy(synth.uniform(1, (B, 1, I))).cuda()
    dY = synth.normal(2, (B, 1, O))
    dY[:, :, 1::5] = 0.0   # cells that receive nothing must not appear in the lists
    dYt = torch.from_numpy(dY).cuda()
    y, idx, md, mk = layer.forward_step(x)

    dx_direct, g_direct = layer.backward_step(x, dYt, idx, md, mk)
    layer._sparse_rows_direct = False
    dx_dense, g_dense = layer.backward_step(x, dYt, idx, md, mk)
    assert g_direct.is_sparse and g_direct.is_coalesced() and g_dense.is_sparse
    assert torch.equal(dx_direct, dx_dense)
    assert torch.equal(g_direct.indices(), g_dense.indices()), "same cells, same (ascending) order"
    golden_util.assert_close(g_direct.values().cpu().numpy(), g_dense.values().cpu().numpy(), 1e-5, "values")

    # bit for bit against the compaction of the deterministic (sorted) dense gradient: same order of additions
    dm = layer._lut_dm
    dW = torch.zeros(((layer._weights.numel() + 3) // 4) * 4, device="cuda:0")
    dX = torch.zeros(B * I, device="cuda:0")
    dm.backward_backprop(layer._weights.detach(), B, dYt.view(-1), layer._detector_anchors, idx.reshape(-1),
                         md.reshape(-1), mk.reshape(-1), dX, -1.0, dW, None, dw_variant=_native.DW_SORTED)
    cells, values = DenseToSparseConverter().dense_to_sparse_32(dW)
    assert torch.equal(cells, g_direct.indices()[0]) and torch.equal(values, g_direct.values())

    # and against the oracle's dense gradient
    W = layer._weights.detach().cpu().numpy()
    anchors = layer._detector_anchors.cpu().numpy()
    _, ref = orc.nonseq_fc_backward(W, dY.reshape(B, O), anchors, idx.cpu().numpy().reshape(B, Nt),
                                    md.cpu().numpy().reshape(B, Nt), mk.cpu().numpy().reshape(B, Nt), I, Nc, lr_meta=0.5)
    golden_util.assert_close(g_direct.to_dense().cpu().numpy(), ref.reshape(-1), 1e-5, "dense view of the lists")


def test_row_list_entry_point_counts_rows_beyond_the_capacity():
    from spiky_b200 import _native

    B, I, Nt, Nc, O = 50, 20, 4, 3, 8
    layer = make_layer(I, Nc, Nt, O, seed=9)
    x = torch.from_numpy(synth.uniform(1, (B, 1, I))).cuda()
    _, idx, _, _ = layer.forward_step(x)
    dY = torch.from_numpy(synth.normal(2, (B, O))).cuda()
    L = _native.lib()
    cfg = layer._lut_dm._cfg()
    need = L.lutb_nonseq_fc_table_grad_rows_workspace(ctypes.byref(cfg), B)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda:0")
    cap = 3
    rows = torch.full((cap,), -1, dtype=torch.int64, device="cuda:0")
    vals = torch.zeros(cap * O, device="cuda:0")
    count = torch.zeros(1, dtype=torch.int64, device="cuda:0")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    _native.check(L.lutb_nonseq_fc_table_grad_rows(ctypes.byref(cfg), B, ptr(dY), ptr(idx.reshape(-1).contiguous()), ptr(rows),
                                                   ptr(vals), cap, ptr(count), ptr(ws), need, stream))
    touched = np.unique(np.arange(Nt)[None, :] * (1 << Nc) + idx.cpu().numpy().reshape(B, Nt))
    assert int(count.item()) == touched.size > cap
    assert np.array_equal(rows.cpu().numpy(), touched[:cap])
    rc = L.lutb_nonseq_fc_table_grad_rows(ctypes.byref(cfg), B, ptr(dY), ptr(idx.reshape(-1).contiguous()), ptr(rows), ptr(vals),
                                          cap, ptr(count), ptr(ws), need - 1, stream)
    assert rc == -4
