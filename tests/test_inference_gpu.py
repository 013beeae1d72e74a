"""int8-table inference and detector sharding of the large inference layer.

The reference has no quantised tables: the int8 results are pinned by DEFINITION to its int32 fixed-point
forward on the de-quantised table, which the (reference-pinned) oracle computes.  Shards are emulated on one GPU
(partial accumulators of the shards are added on the host the way the all-reduce adds them)."""
import numpy as np
import pytest
import torch

import golden_util
import synth
from oracle import lut_oracle as orc

pytestmark = pytest.mark.gpu


def make_problem(seed, B, I, Nt, Nc, O):
    x = synth.normal(seed + 1, (B, I))
    anchors = synth.anchor_pairs(seed + 2, Nt, Nc, I)
    q = synth.integers(seed + 3, (Nt * (1 << Nc) * O,), -127, 128).astype(np.int8)
    s = (0.02 / 127 * synth.uniform(seed + 4, (Nt,), 0.5, 1.5)).astype(np.float32)
    return x, anchors, q, s


def dequantize(q, s, Nt):
    return (s[:, None] * q.reshape(Nt, -1).astype(np.float32)).astype(np.float32).reshape(-1)


@pytest.mark.parametrize("shape", [(33, 256, 64, 8, 64), (16, 4096, 512, 8, 64), (9, 40, 96, 5, 12)])
def test_int8_inference_is_bit_exact_with_fixed_point_reference_on_dequantized_table(shape):
    from spiky_b200.inference import LUTInference

    B, I, Nt, Nc, O = shape
    x, anchors, q, s = make_problem(900, B, I, Nt, Nc, O)
    layer = LUTInference(I, O, Nt, Nc, torch.from_numpy(anchors), torch.from_numpy(q), torch.from_numpy(s),
                         int_rescaler=0.05, dequant="f32")
    y = layer(torch.from_numpy(x).cuda()).cpu().numpy()
    ref, ridx, _, _ = orc.nonseq_fc_forward(dequantize(q, s, Nt), x, anchors, Nt, Nc, O, train=False, int_mode=True,
                                            int_rescaler=0.05)
    assert np.array_equal(layer.last_indices.cpu().numpy(), ridx)
    assert np.array_equal(y, ref)
    # the dedicated int8 oracle function agrees with the pinned fixed-point forward on the de-quantised table
    acc, _ = orc.infer_int8(q, s, x, anchors, Nt, Nc, O, int_rescaler=0.05, exact=False)
    assert np.array_equal(orc.int_to_float(acc, 0.05), ref)


def test_int8_inference_detector_ranges_and_odd_blocks():
    """Tables larger than one L2 range (two launches over detector ranges), detector blocks of 7 with a ragged last
    block, 4-wide rows."""
    from spiky_b200.inference import LUTInference

    for (B, I, Nt, Nc, O, blk) in [(5, 64, 700, 8, 256, 32), (11, 30, 45, 3, 4, 7)]:
        x, anchors, q, s = make_problem(930, B, I, Nt, Nc, O)
        for rule, exact in (("exact", True), ("f32", False)):
            layer = LUTInference(I, O, Nt, Nc, torch.from_numpy(anchors), torch.from_numpy(q), torch.from_numpy(s),
                                 int_rescaler=0.05, backward_group_size=blk, dequant=rule)
            acc = layer.partial(torch.from_numpy(x).cuda()).cpu().numpy()
            want, _ = orc.infer_int8(q, s, x, anchors, Nt, Nc, O, backward_group_size=blk, int_rescaler=0.05, exact=exact)
            assert np.array_equal(acc, want), (B, I, Nt, Nc, O, blk, rule)


@pytest.mark.parametrize("shape", [(33, 256, 64, 8, 64), (16, 4096, 512, 8, 64), (9, 40, 96, 5, 12), (5, 64, 70, 6, 128)])
def test_int8_inference_exact_product_rule_is_bit_exact(shape):
    """Entries taken as the exact reals scale * q (the default, fast rule): bit-exact against the oracle's
    restatement, and within one fp32 rounding per entry of the f32 rule."""
    from spiky_b200.inference import LUTInference

    B, I, Nt, Nc, O = shape
    x, anchors, q, s = make_problem(905, B, I, Nt, Nc, O)
    layer = LUTInference(I, O, Nt, Nc, torch.from_numpy(anchors), torch.from_numpy(q), torch.from_numpy(s),
                         int_rescaler=0.05)
    xt = torch.from_numpy(x).cuda()
    acc = layer.partial(xt).cpu().numpy()
    want, ridx = orc.infer_int8(q, s, x, anchors, Nt, Nc, O, int_rescaler=0.05, exact=True)
    assert np.array_equal(layer.last_indices.cpu().numpy(), ridx)
    assert np.array_equal(acc, want)
    other, _ = orc.infer_int8(q, s, x, anchors, Nt, Nc, O, int_rescaler=0.05, exact=False)
    assert np.abs(acc.astype(np.int64) - other).max() <= (Nt + 31) // 32   # at most one unit per detector block


@pytest.mark.parametrize("world", [2, 4])
def test_detector_shards_combine_exactly_int8_and_within_tolerance_fp32(world):
    from spiky_b200.inference import LUTInference

    B, I, Nt, Nc, O = 21, 512, 256, 6, 32
    x, anchors, q, s = make_problem(910, B, I, Nt, Nc, O)
    xt = torch.from_numpy(x).cuda()
    args = (I, O, Nt, Nc, torch.from_numpy(anchors), torch.from_numpy(q), torch.from_numpy(s))
    full = LUTInference(*args, int_rescaler=0.05)
    want = full(xt).cpu().numpy()
    shards = [LUTInference.shard_of(r, world, *args, int_rescaler=0.05) for r in range(world)]
    acc = sum(sh.partial(xt) for sh in shards)          # what the integer all-reduce computes
    got = shards[0].finish(acc.contiguous()).cpu().numpy()
    assert np.array_equal(got, want)
    # fp32 tables: partial sums add up to the unsharded result within summation-order tolerance
    W = torch.from_numpy(dequantize(q, s, Nt))
    fargs = (I, O, Nt, Nc, torch.from_numpy(anchors), W)
    want32 = LUTInference(*fargs)(xt).cpu().numpy()
    got32 = sum(LUTInference.shard_of(r, world, *fargs).partial(xt) for r in range(world)).cpu().numpy()
    golden_util.assert_close(got32, want32, 1e-5, "sharded fp32")
    ref32, _, _, _ = orc.nonseq_fc_forward(W.numpy(), x, anchors, Nt, Nc, O, train=False)
    golden_util.assert_close(want32, ref32, 1e-5, "fp32 vs oracle")
