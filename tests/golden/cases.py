"""Golden-case definitions: scalar configurations and the seeded input builders.

Imported both by make_golden.py (which runs the reference on these inputs) and by the tests
(which rebuild the same inputs and compare against the recorded reference outputs).  This module
must not import the reference.
"""
import synth


def nonseq_fc_inputs(cfg):
    """Inputs of a fully connected non-sequence case, rebuilt from cfg seeds (used by tests too)."""
    s = cfg["seed"]
    B, I, Nt, Nc, O = cfg["B"], cfg["I"], cfg["Nt"], cfg["Nc"], cfg["O"]
    T = 1 << Nc
    if cfg.get("sparse_input"):
        x = synth.sparse_images(s + 11, (B, I))
    elif cfg.get("normal_input"):
        x = synth.normal(s + 11, (B, I))
    else:
        x = synth.uniform(s + 11, (B, I))
    anchors = synth.anchor_pairs(s + 12, Nt, Nc, I)
    if cfg.get("unused_pair"):
        anchors[0, Nc - 1, :] = -1  # a disabled pair (0xFFFFFFFF), spiky_cuda/lut/lut_runtime_kernels_logic.proto:1077
    if cfg.get("unused_leading_pairs"):
        anchors[1, :Nc - 1, :] = -1  # only the last pair of detector 1 is live: indices are 0 or 2^(Nc-1)
    W = synth.normal(s + 13, (Nt * T * O,), 0.0, cfg.get("w_std", 0.02))
    dY = synth.normal(s + 14, (B, O))
    if cfg.get("zero_dy"):
        dY[:, ::3] = 0.0
    return x, anchors, W, dY



NONSEQ_FC_CASES = {
    # tiny ragged shapes: O not a multiple of 4, Nt not a multiple of the block sizes
    "fc_tiny_f32": dict(seed=100, B=5, I=20, Nt=7, Nc=3, O=5, G=2, Gb=3),
    "fc_tiny_i32": dict(seed=101, B=5, I=20, Nt=7, Nc=3, O=5, G=2, Gb=3, int_mode=True, int_rescaler=10.0),
    "fc_tiny_b1": dict(seed=102, B=1, I=9, Nt=1, Nc=1, O=1),
    "fc_unused_pair": dict(seed=103, B=6, I=16, Nt=4, Nc=4, O=6, unused_pair=True),
    "fc_cmp_eps": dict(seed=104, B=8, I=24, Nt=6, Nc=5, O=8, cmp_eps=0.05, normal_input=True),
    "fc_internal": dict(seed=105, B=9, I=30, Nt=5, Nc=4, O=7, policy="internal", ext_lr=0.25, lr_meta=0.5),
    "fc_lr_meta_zero_dy": dict(seed=106, B=7, I=18, Nt=6, Nc=3, O=9, lr_meta=0.125, zero_dy=True, G=4),
    # exact ties are the common case with sparse inputs: first minimal |delta| wins, up(0) < 0
    "fc_sparse_input_f32": dict(seed=107, B=12, I=64, Nt=16, Nc=6, O=12, sparse_input=True),
    "fc_sparse_input_i32": dict(seed=108, B=12, I=64, Nt=16, Nc=6, O=12, sparse_input=True, int_mode=True,
                                int_rescaler=0.5),
    # a slice of the single-layer benchmark configuration (784 inputs, 64 tables x 6 pairs, 32 outputs)
    "fc_c1_slice_f32": dict(seed=109, B=16, I=784, Nt=64, Nc=6, O=32),
    "fc_c1_slice_i32": dict(seed=110, B=16, I=784, Nt=64, Nc=6, O=32, int_mode=True),
    # wider outputs than one forward group, more detectors than one backward group
    "fc_wide_f32": dict(seed=111, B=4, I=40, Nt=35, Nc=3, O=35, G=32, Gb=32),
    "fc_wide_i32": dict(seed=112, B=4, I=40, Nt=35, Nc=3, O=35, G=32, Gb=32, int_mode=True, int_rescaler=3.0),
    # rows far longer than one warp pass, odd length; more detectors than one block of 32
    "fc_long_rows_f32": dict(seed=113, B=3, I=24, Nt=37, Nc=2, O=515),
    "fc_long_rows_i32": dict(seed=114, B=3, I=24, Nt=37, Nc=2, O=515, int_mode=True, int_rescaler=0.25),
    # 1024-row tables; a detector with a single live pair
    "fc_big_table_f32": dict(seed=115, B=10, I=50, Nt=3, Nc=10, O=8, unused_leading_pairs=True),
    "fc_rows_vec4_f32": dict(seed=116, B=9, I=33, Nt=40, Nc=4, O=64, cmp_eps=0.01),
}




def projection_inputs(cfg, n_weights):
    """Batch, table weights and upstream gradient of a sparse projection-layer case."""
    s = cfg["seed"]
    B = cfg["B"]
    I = cfg["in_shape"][0] * cfg["in_shape"][1]
    O = cfg["out_shape"][0] * cfg["out_shape"][1]
    x = synth.sparse_images(s + 21, (B, I)) if cfg.get("sparse_input") else synth.uniform(s + 21, (B, I))
    W = synth.normal(s + 23, (n_weights,), 0.0, 0.05)
    dY = synth.normal(s + 24, (B, O))
    if cfg.get("zero_dy"):
        dY[:, ::4] = 0.0
    return x, W, dY


PROJECTION_CASES = {
    "proj_grid_f32": dict(seed=200, B=6, in_shape=(12, 12), out_shape=(10, 10), Nc=3, groups=9, per_group=4,
                          receptive=(5, 5), projection=(4, 4), grid=(3, 3, 3, 3, 2, 2)),
    "proj_grid_i32": dict(seed=201, B=6, in_shape=(12, 12), out_shape=(10, 10), Nc=3, groups=9, per_group=4,
                          receptive=(5, 5), projection=(4, 4), grid=(3, 3, 3, 3, 2, 2), int_mode=True,
                          int_rescaler=2.0),
    "proj_random_f32": dict(seed=202, B=5, in_shape=(16, 16), out_shape=(12, 12), Nc=4, groups=7, per_group=3,
                            receptive=(5, 5), projection=(4, 4), sparse_input=True, zero_dy=True),
    "proj_random_i32": dict(seed=203, B=5, in_shape=(16, 16), out_shape=(12, 12), Nc=4, groups=7, per_group=3,
                            receptive=(5, 5), projection=(4, 4), sparse_input=True, int_mode=True, int_rescaler=1.0),
    # several synapse groups per lookup neuron (group size 8 < synapses per row)
    "proj_multigroup_f32": dict(seed=204, B=4, in_shape=(14, 14), out_shape=(14, 14), Nc=3, groups=5, per_group=2,
                                receptive=(7, 7), projection=(4, 4), G=8),
    "proj_multigroup_i32": dict(seed=205, B=4, in_shape=(14, 14), out_shape=(14, 14), Nc=3, groups=5, per_group=2,
                                receptive=(7, 7), projection=(4, 4), G=8, int_mode=True, int_rescaler=0.25),
    # rows longer than a warp (7x7 projections: up to 49 targets, two synapse groups of 32 per row)
    "proj_longrows_f32": dict(seed=207, B=5, in_shape=(14, 14), out_shape=(14, 14), Nc=3, groups=4, per_group=3,
                              receptive=(5, 5), projection=(7, 7)),
    "proj_longrows_i32": dict(seed=208, B=5, in_shape=(14, 14), out_shape=(14, 14), Nc=3, groups=4, per_group=3,
                              receptive=(5, 5), projection=(7, 7), int_mode=True, int_rescaler=0.5),
    # a slice of the first layer of the sparse conv-net configuration: 256-row tables, more samples than one sample run
    "proj_c2_slice_f32": dict(seed=209, B=21, in_shape=(28, 28), out_shape=(24, 24), Nc=8, groups=6, per_group=8,
                              receptive=(5, 5), projection=(4, 4), sparse_input=True),
    # short rows (2x2 projections: 4 to 9 targets) take the 8-lane row groups
    "proj_shortrows_f32": dict(seed=210, B=9, in_shape=(12, 12), out_shape=(12, 12), Nc=4, groups=8, per_group=5,
                               receptive=(5, 5), projection=(2, 2)),
    "proj_internal": dict(seed=206, B=7, in_shape=(12, 12), out_shape=(8, 8), Nc=3, groups=6, per_group=3,
                          receptive=(5, 5), projection=(3, 3), policy="internal", ext_lr=0.5, lr_meta=0.25),
}


def sequence_inputs(cfg, n_weights, n_pe):
    """Inputs of a sequence-layer case (product or concatenation mode): x [B,S,E], anchors over the
    layer's (virtual) input vector, tables, positional embeddings (flat, as the layer stores them), dY."""
    s = cfg["seed"]
    B, S, E, Nt, Nc, O = cfg["B"], cfg["S"], cfg["E"], cfg["Nt"], cfg["Nc"], cfg["O"]
    x = synth.uniform(s + 31, (B, S, E), -1.0, 1.0)
    if cfg.get("quantized_input"):  # coarse values make exact ties and dead-band hits common
        x = (x * 4).round().astype("float32") / 4
    n_virtual = cfg.get("n_virtual", E)
    anchors = synth.anchor_pairs(s + 32, Nt, Nc, n_virtual)
    W = synth.normal(s + 33, (n_weights,), 0.0, 0.05)
    pe = synth.uniform(s + 34, (n_pe,), -1.0, 1.0) if n_pe else None
    dY = synth.normal(s + 35, (B, S, O))
    return x, anchors, W, pe, dY


PRODUCT_CASES = {
    "prod_plain_f32": dict(seed=300, B=3, S=6, E=7, Nt=4, Nc=3, Npe=2, O=5),
    "prod_plain_i32": dict(seed=301, B=3, S=6, E=7, Nt=4, Nc=3, Npe=2, O=5, int_mode=True, int_rescaler=5.0),
    "prod_sliced_f32": dict(seed=302, B=2, S=7, E=5, Nt=3, Nc=4, Npe=5, O=6, sliced=True, unified_pe=True,
                            cmp_eps=1e-4, quantized_input=True),
    "prod_sliced_i32": dict(seed=303, B=2, S=7, E=5, Nt=3, Nc=4, Npe=5, O=6, sliced=True, unified_pe=True,
                            cmp_eps=1e-4, int_mode=True, int_rescaler=1.0),
    "prod_nope_f32": dict(seed=304, B=2, S=5, E=6, Nt=3, Nc=3, Npe=0, O=4),
    "prod_internal": dict(seed=305, B=2, S=6, E=6, Nt=3, Nc=3, Npe=3, O=7, policy="internal", ext_lr=0.5,
                          lr_meta=0.5),
    "prod_wide_f32": dict(seed=306, B=2, S=9, E=12, Nt=5, Nc=4, Npe=4, O=40, unified_pe=True),
    "prod_wide_i32": dict(seed=307, B=2, S=9, E=12, Nt=5, Nc=4, Npe=4, O=40, int_mode=True, int_rescaler=0.5),
    # sequences longer than the table (2^4 rows): the CUDA path takes the histogram / contraction kernels in both passes
    "prod_long_f32": dict(seed=308, B=2, S=24, E=6, Nt=3, Nc=4, Npe=2, O=8),
    "prod_long_internal": dict(seed=309, B=3, S=20, E=6, Nt=4, Nc=4, Npe=3, O=12, policy="internal", ext_lr=0.25,
                               lr_meta=0.5, quantized_input=True, cmp_eps=1e-4),
    "prod_two_tokens": dict(seed=310, B=3, S=2, E=5, Nt=2, Nc=3, Npe=1, O=4),
}
for _c in PRODUCT_CASES.values():
    _c["n_virtual"] = 3 * _c["E"] if _c.get("sliced") else 2 * _c["E"] + _c["Npe"]


CONCAT_CASES = {
    "concat_f32": dict(seed=400, B=3, S=6, E=9, Nt=4, Nc=2, Npe=2, O=5, G=4),
    "concat_i32": dict(seed=401, B=3, S=6, E=9, Nt=4, Nc=2, Npe=2, O=5, G=4, int_mode=True, int_rescaler=10.0),
    "concat_unified_f32": dict(seed=402, B=2, S=7, E=8, Nt=3, Nc=3, Npe=3, O=6, unified_pe=True, quantized_input=True),
    "concat_nope_f32": dict(seed=403, B=2, S=5, E=8, Nt=3, Nc=2, Npe=0, O=7),
    "concat_internal": dict(seed=404, B=2, S=6, E=8, Nt=3, Nc=2, Npe=2, O=6, policy="internal", ext_lr=0.25,
                            lr_meta=0.5),
    # more than one 32x32 pair tile, outputs wider than one forward group
    "concat_long_f32": dict(seed=405, B=1, S=40, E=10, Nt=2, Nc=2, Npe=1, O=35),
    "concat_long_i32": dict(seed=406, B=1, S=40, E=10, Nt=2, Nc=2, Npe=1, O=35, int_mode=True, int_rescaler=0.5),
    # one key more than a 32-wide pair tile, dead band, vector-width rows
    "concat_tile_edge_f32": dict(seed=407, B=2, S=34, E=12, Nt=3, Nc=2, Npe=2, O=16, cmp_eps=0.02, quantized_input=True),
}


# Concatenation-mode sequence layers whose lookup -> output connectivity is sparse (Conv2DLUTLayer with a second
# sliding window over the detector grid): geometry arguments of the layer plus batch / sequence sizes.
CONCAT_SPARSE_CASES = {
    # (the reference can only build these layers without positional embeddings: its output window counts
    # 2^(2*Nc) lookup channels per detector, LUTLayer.py:199-203 against :1370)
    "sparse_concat_f32": dict(seed=500, B=2, S=6, in_shape=(4, 4), Nc=2, Npe=0, det_shape=(2, 2), out_kernel=(2, 2),
                              rf=(2, 2), rf_stride=(2, 2), lut_rf=(2, 2), lut_rf_stride=(2, 2)),
    "sparse_concat_i32": dict(seed=501, B=2, S=6, in_shape=(4, 4), Nc=2, Npe=0, det_shape=(2, 2), out_kernel=(2, 2),
                              rf=(2, 2), rf_stride=(2, 2), lut_rf=(2, 2), lut_rf_stride=(2, 2), int_mode=True,
                              int_rescaler=2.0),
    # more than one 32x32 pair tile; rows longer than one synapse group (group size 4 < 9 targets)
    "sparse_concat_long_f32": dict(seed=502, B=1, S=35, in_shape=(4, 6), Nc=2, Npe=0, det_shape=(1, 2), out_kernel=(1, 1),
                                   rf=(2, 2), rf_stride=(2, 2), lut_rf=(2, 3), lut_rf_stride=(1, 1), G=4,
                                   quantized_input=True),
    "sparse_concat_internal": dict(seed=503, B=2, S=5, in_shape=(4, 4), Nc=2, Npe=0, det_shape=(2, 1), out_kernel=(1, 2),
                                   rf=(2, 2), rf_stride=(2, 2), lut_rf=(2, 1), lut_rf_stride=(1, 1), policy="internal",
                                   ext_lr=0.25, lr_meta=0.5),
}


def concat_sparse_inputs(cfg, n_weights, n_outputs, n_detectors):
    """x [B,S,E], tables (flat, reference layout), positional embeddings (flat, as stored) and dY [B,S,O]."""
    s = cfg["seed"]
    B, S = cfg["B"], cfg["S"]
    E = cfg["in_shape"][0] * cfg["in_shape"][1]
    x = synth.uniform(s + 41, (B, S, E), -1.0, 1.0)
    if cfg.get("quantized_input"):
        x = (x * 4).round().astype("float32") / 4
    W = synth.normal(s + 42, (n_weights,), 0.0, 0.1)
    n_pe = (S - 1) * (1 if cfg.get("unified_pe") else n_detectors) * cfg["Npe"]
    pe = synth.uniform(s + 43, (n_pe,), -1.0, 1.0) if n_pe > 0 else None
    dY = synth.normal(s + 44, (B, S, n_outputs))
    return x, W, pe, dY



# Non-sequence Conv2DLUTLayer: detectors on sliding receptive fields, outputs through a second sliding window over the
# detector grid (sparse) or fully connected (lut_rf None).  The fixtures also pin the geometry: which inputs a
# detector may compare and which outputs it feeds.
CONV2D_CASES = {
    "conv2d_sparse_f32": dict(seed=700, B=5, in_shape=(8, 10), Nc=3, det_shape=(2, 3), out_kernel=(2, 2), rf=(4, 4),
                              rf_stride=(2, 3), lut_rf=(3, 3), lut_rf_stride=(1, 2)),
    "conv2d_sparse_i32": dict(seed=701, B=5, in_shape=(8, 10), Nc=3, det_shape=(2, 3), out_kernel=(2, 2), rf=(4, 4),
                              rf_stride=(2, 3), lut_rf=(3, 3), lut_rf_stride=(1, 2), int_mode=True, int_rescaler=0.5),
    "conv2d_fc_f32": dict(seed=702, B=4, in_shape=(6, 6), Nc=4, det_shape=(1, 2), out_kernel=(3, 2), rf=(3, 3),
                          rf_stride=(3, 3), lut_rf=None, lut_rf_stride=None),
}


def conv2d_inputs(cfg, n_weights, n_outputs):
    s = cfg["seed"]
    B = cfg["B"]
    I = cfg["in_shape"][0] * cfg["in_shape"][1]
    x = synth.uniform(s + 51, (B, I), -1.0, 1.0)
    W = synth.normal(s + 52, (n_weights,), 0.0, 0.1)
    dY = synth.normal(s + 53, (B, n_outputs))
    return x, W, dY


# Whole LUTTransformer models (reference: src/spiky/lut/LUTTransformer.py): the fixture carries every parameter and
# anchor of the reference-built model, the tokens, the logits and the gradients of all parameters for a seeded
# upstream gradient, so that the block wiring (attention -> residual, feed-forward -> residual, unembedder) is pinned.
TRANSFORMER_CASES = {
    "transformer_product_f32": dict(seed=31, B=3, V=23, E=16, S=8, Npe=4, layers=2, heads=2, Nt=3, Nc=4, concat=False),
    "transformer_concat_f32": dict(seed=32, B=2, V=19, E=12, S=6, Npe=2, layers=2, heads=2, Nt=2, Nc=3, concat=True),
    "transformer_concat_i32": dict(seed=33, B=2, V=19, E=12, S=6, Npe=2, layers=1, heads=2, Nt=2, Nc=3, concat=True,
                                   int_mode=True, int_rescaler=10.0),
    # 2-D embeddings: the attention layer is a Conv2DLUTLayer whose single receptive field covers the whole input
    "transformer_concat_2d_f32": dict(seed=35, B=2, V=15, E=(3, 4), S=5, Npe=2, layers=2, heads=2, Nt=2, Nc=3, concat=True),
    # BatchNorm1d on every branch before the residual addition (training mode: batch statistics)
    "transformer_product_bn_f32": dict(seed=36, B=3, V=21, E=16, S=6, Npe=3, layers=2, heads=2, Nt=3, Nc=4, concat=False,
                                       batch_norm=True),
    "transformer_product_unified_noffn_f32": dict(seed=34, B=2, V=17, E=16, S=7, Npe=4, layers=2, heads=1, Nt=4, Nc=4,
                                                  concat=False, unified_pe=True, no_ffn=True, Nc_att=5),
}


def transformer_inputs(cfg):
    """tokens int64 [B, S] and the upstream gradient of the logits fp32 [B, S, V]."""
    s = cfg["seed"]
    tokens = synth.integers(s + 51, (cfg["B"], cfg["S"]), 0, cfg["V"]).astype("int64")
    dlogits = synth.normal(s + 52, (cfg["B"], cfg["S"], cfg["V"]))
    return tokens, dlogits
