"""The two kernel families of the sparse non-sequence layer (gather and staged, include/spiky_b200.h:
lutb_sparse_kernel_select) against the oracle and against each other, through the C ABI.

The staged kernels stream whole tables through a shared-memory ring behind bounded mbarrier waits; every case also
checks that no wait ran out (lutb_device_wait_errors)."""
import numpy as np
import pytest
import torch

import golden_util
import synth
from oracle import lut_oracle as orc

pytestmark = pytest.mark.gpu
REL = 1e-5


@pytest.fixture(autouse=True)
def restore_kernel_choice():
    from spiky_b200 import _native
    yield
    _native.sparse_kernel_select(_native.SPARSE_AUTO)


def run_layer(layer, x, dY):
    B = x.shape[0]
    I, O, Nt = layer.n_inputs(), layer.n_outputs(), layer.n_detectors()
    xt = torch.from_numpy(x).view((B, 1) + tuple(layer.input_shape())).cuda()
    layer.eval()
    y_eval = layer.forward_step(xt).cpu().numpy().reshape(B, O)
    layer.train()
    y, idx, md, mk = layer.forward_step(xt)
    dx, dw = layer.backward_step(xt, torch.from_numpy(dY).view((B, 1) + tuple(layer.output_shape())).cuda(), idx, md, mk)
    torch.cuda.synchronize()
    return dict(y=y.cpu().numpy().reshape(B, O), y_eval=y_eval, idx=idx.cpu().numpy().reshape(B, Nt),
                dX=dx.cpu().numpy().reshape(B, I), dW=dw.cpu().numpy())


def oracle_layer(layer, x, dY, nc):
    index = layer._lut_dm._sparse
    sp = dict(index.numpy(), group_size=index.group_size)
    W = layer._weights.detach().cpu().numpy()
    anchors = layer._detector_anchors.cpu().numpy()
    y, idx, md, mk = orc.nonseq_sparse_forward(W, x, anchors, sp, nc, layer.n_outputs())
    dX, dW = orc.nonseq_sparse_backward(W, dY, anchors, idx, md, mk, sp, layer.n_inputs(), nc)
    return dict(y=y, y_eval=y, idx=idx, dX=dX, dW=dW)


def check(got, ref, what):
    assert np.array_equal(got["idx"], ref["idx"]), what
    for k in ("y", "y_eval", "dX", "dW"):
        golden_util.assert_close(got[k], ref[k], REL, f"{what}: {k}")


# (input hw, output hw, Nc, groups, detectors per group, projection, batch, forward_group_size)
SHAPES = {
    # the detector groups of the conv-net configuration: 32 detectors per group, rows of 16 / 20 / 25 synapses
    "convnet_l1_b512": ((28, 28), (24, 24), 8, 144, 32, (4, 4), 512, 32),
    # a batch that is neither a multiple of the 512-sample tile nor of a warp's 32 samples; two chunks per group
    "two_tiles_ragged": ((20, 20), (16, 16), 6, 64, 40, (4, 4), 530, 32),
    # few samples: most consumer warps have no sample at all
    "tiny_batch": ((14, 14), (12, 12), 5, 36, 9, (3, 3), 7, 32),
    # rows of at most 8 / 16 synapses with holes inside the rows (forward groups of 4 synapses)
    "short_rows_inner_holes": ((14, 14), (12, 12), 5, 36, 5, (3, 3), 70, 4),
    # single-detector chunks
    "one_detector_per_group": ((14, 14), (12, 12), 4, 36, 1, (4, 4), 130, 32),
}


def build(shape):
    from spiky_b200.lut_layer import ProjectionLUTLayer, SynapseMeta, PointSamplingPolicy, PointSamplingType

    ihw, ohw, nc, groups, per, proj, batch, fg = SHAPES[shape]
    g = int(round(groups ** 0.5))
    layer = ProjectionLUTLayer(
        ihw, ohw, nc, groups, per, (5, 5), proj,
        synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.1, initial_weight=-0.05),
        detectors_sampling_policy=PointSamplingPolicy(PointSamplingType.Grid, grid_h=g, grid_w=g, stride_h=2,
                                                      stride_w=2, pad_h=2, pad_w=2),
        _forward_group_size=fg, random_seed=3, device="cuda:0")
    x = synth.sparse_images(5, (batch, ihw[0] * ihw[1]))
    dY = synth.normal(6, (batch, ohw[0] * ohw[1]))
    return layer, x, dY, nc


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_staged_and_gather_kernels_match_oracle(shape):
    from spiky_b200 import _native

    layer, x, dY, nc = build(shape)
    ref = oracle_layer(layer, x, dY, nc)
    assert layer._lut_dm._sparse.tables_aligned16 == 1
    for fwd, dx in ((_native.SPARSE_STAGED, _native.SPARSE_STAGED), (_native.SPARSE_GATHER, _native.SPARSE_GATHER),
                    (_native.SPARSE_STAGED, _native.SPARSE_GATHER)):
        _native.sparse_kernel_select(fwd, dx)
        check(run_layer(layer, x, dY), ref, f"{shape}/forward {fwd}, input gradient {dx}")
    assert _native.device_wait_errors() == 0


def test_staged_is_refused_for_rows_longer_than_a_warp_and_auto_falls_back():
    from spiky_b200 import _native
    from spiky_b200.lut_layer import ProjectionLUTLayer, SynapseMeta

    layer = ProjectionLUTLayer((14, 14), (12, 12), 5, 6, 5, (5, 5), (6, 6),
                               synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.1,
                                                        initial_weight=0.02), random_seed=7, device="cuda:0")
    assert layer._lut_dm._sparse.max_count > 32
    x = synth.sparse_images(15, (6, 14 * 14))
    dY = synth.normal(16, (6, 12 * 12))
    ref = oracle_layer(layer, x, dY, 5)
    check(run_layer(layer, x, dY), ref, "auto")
    _native.sparse_kernel_select(_native.SPARSE_STAGED)
    with pytest.raises(ValueError, match="staged"):
        run_layer(layer, x, dY)


def test_tables_that_cannot_be_bulk_copied_use_the_gather_kernels():
    """Two-row tables of 11 slots per row: 22 slots per table, so tables start at 8-byte offsets."""
    from spiky_b200 import _native
    from spiky_b200.lut_layer import ProjectionLUTLayer, SynapseMeta

    layer = ProjectionLUTLayer((14, 14), (12, 12), 1, 6, 5, (5, 5), (3, 3),
                               synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.1,
                                                        initial_weight=0.02), random_seed=7, device="cuda:0")
    assert layer._lut_dm._sparse.tables_aligned16 == 0
    x = synth.sparse_images(15, (40, 14 * 14))
    dY = synth.normal(16, (40, 12 * 12))
    check(run_layer(layer, x, dY), oracle_layer(layer, x, dY, 1), "auto")
    _native.sparse_kernel_select(_native.SPARSE_STAGED)
    with pytest.raises(ValueError, match="staged"):
        run_layer(layer, x, dY)


def test_kernel_select_rejects_unknown_values():
    from spiky_b200 import _native

    with pytest.raises(ValueError):
        _native.sparse_kernel_select(7)
    with pytest.raises(ValueError):
        _native.sparse_kernel_select(_native.SPARSE_AUTO, -1)
