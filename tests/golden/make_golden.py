"""Records golden vectors from the REAL reference (its CPU build) for the LUT hot path.

Run in a container that has the reference checkout:

    tests/golden/build_reference_cpu.sh <reference checkout>  # once, builds into /tmp/spiky_ref
    PYTHONPATH=/tmp/spiky_ref/spiky_cuda:/tmp/spiky_ref/src \
        python tests/golden/make_golden.py [case-name-prefix ...]

Each case is written to tests/golden/<name>.npz: the scalar configuration, the seeds of the
hashed synthetic inputs (see synth.py; small inputs are stored verbatim as well) and every tensor
the reference produced.  The tests rebuild the inputs from the seeds and compare the oracle and
the CUDA path with the stored reference outputs.
"""
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import synth  # noqa: E402,F401
from cases import (CONCAT_CASES, CONCAT_SPARSE_CASES, CONV2D_CASES, TRANSFORMER_CASES, transformer_inputs, concat_sparse_inputs, conv2d_inputs, NONSEQ_FC_CASES, PROJECTION_CASES, PRODUCT_CASES, nonseq_fc_inputs, projection_inputs,  # noqa: E402
                   sequence_inputs)

from spiky.lut.LUTLayer import (  # noqa: E402  (the reference)
    LUTLayer, ProjectionLUTLayer, SynapseMeta, GradientPolicy, GradientType, LUTSharedContext,
)
from spiky.util.synapse_growth import PointSamplingPolicy, PointSamplingType  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def save(name, cfg, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, cfg=np.frombuffer(json.dumps(cfg).encode(), dtype=np.uint8), **arrays)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def t2n(t):
    return None if t is None else t.detach().cpu().numpy().copy()


# ----------------------------------------------------------------------------- non-seq FC
def run_nonseq_fc(name, cfg):
    x, anchors, W, dY = nonseq_fc_inputs(cfg)
    B, I, Nt, Nc, O = cfg["B"], cfg["I"], cfg["Nt"], cfg["Nc"], cfg["O"]
    int_mode = cfg.get("int_mode", False)
    policy = {"dense": GradientType.Dense, "internal": GradientType.Internal}[cfg.get("policy", "dense")]
    ctx = LUTSharedContext(_cmp_eps=cfg.get("cmp_eps", 0.0))
    ctx.to_device(torch.device("cpu"))
    layer = LUTLayer(
        n_inputs=I, n_anchors_per_detector=Nc, n_detectors=Nt, n_outputs=O,
        synapse_meta=SynapseMeta(learning_rate=cfg.get("lr_meta", 1.0), min_weight=-1.0, max_weight=1.0),
        weights_gradient_policy=GradientPolicy(policy),
        shared_context=ctx,
        summation_dtype=torch.int32 if int_mode else torch.float32,
        _explicit_anchors=torch.from_numpy(anchors.reshape(-1).copy()),
        _int_rescaler=cfg.get("int_rescaler", 0.001),
        _forward_group_size=cfg.get("G", 32), _backward_group_size=cfg.get("Gb", 32),
        random_seed=1,
    )
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
    xt = torch.from_numpy(x).view(B, 1, I)
    out = {}
    layer.eval()
    out["y_eval"] = t2n(layer.forward_step(xt)).reshape(B, O)
    layer.train()
    y, idx, md, mk = layer.forward_step(xt)
    out.update(y=t2n(y).reshape(B, O), idx=t2n(idx).reshape(B, Nt), min_delta=t2n(md).reshape(B, Nt),
               min_k=t2n(mk).reshape(B, Nt))
    if policy == GradientType.Internal:
        layer.set_external_learning_rate_hook(lambda w: cfg["ext_lr"])
    dx, dw = layer.backward_step(xt, torch.from_numpy(dY).view(B, 1, O), idx, md, mk)
    out["dX"] = t2n(dx).reshape(B, I)
    if policy == GradientType.Internal:
        out["W_after"] = t2n(layer._weights)
    else:
        out["dW"] = t2n(dw)
    extra = {}
    if x.size <= 4096:
        extra = dict(in_x=x, in_anchors=anchors, in_W=W, in_dY=dY)
    save(name, dict(cfg, kind="nonseq_fc"), **out, **extra)


# ----------------------------------------------------------------------------- sparse projection
def export_structure(layer):
    """Per synapse of a reference-built sparse layer: lookup neuron, slot in the flat weight array and
    output index.  The slot is read back by exporting with the weights set to 0, 1, 2, ..."""
    n = layer.n_synapses()
    saved = layer._weights.detach().clone()
    with torch.no_grad():
        layer._weights.copy_(torch.arange(layer._weights.numel(), dtype=torch.float32))
    src = torch.zeros(n, dtype=torch.int32)
    tgt = torch.zeros(n, dtype=torch.int32)
    slot = torch.zeros(n, dtype=torch.float32)
    layer._export_synapses(layer.get_lookup_neuron_ids(), src, slot, tgt)
    with torch.no_grad():
        layer._weights.copy_(saved)
    assert layer._weights.numel() < (1 << 24), "slots must be exactly representable in fp32"
    return src.numpy().astype(np.int64), slot.numpy().astype(np.int64), tgt.numpy().astype(np.int64) - layer.n_lookup_neurons()


def run_projection(name, cfg):
    int_mode = cfg.get("int_mode", False)
    policy = {"dense": GradientType.Dense, "internal": GradientType.Internal}[cfg.get("policy", "dense")]
    if "grid" in cfg:
        gh, gw, sh, sw, ph, pw = cfg["grid"]
        sampling = PointSamplingPolicy(PointSamplingType.Grid, grid_h=gh, grid_w=gw, stride_h=sh, stride_w=sw,
                                       pad_h=ph, pad_w=pw)
    else:
        sampling = PointSamplingPolicy(PointSamplingType.RandomUniform)
    layer = ProjectionLUTLayer(
        input_shape=cfg["in_shape"], output_shape=cfg["out_shape"], n_anchors_per_detector=cfg["Nc"],
        n_detector_groups=cfg["groups"], n_detectors_in_group=cfg["per_group"], receptive_shape=cfg["receptive"],
        projection_shape=cfg["projection"],
        synapse_meta=SynapseMeta(learning_rate=cfg.get("lr_meta", 1.0), min_weight=-1.0, max_weight=1.0),
        detectors_sampling_policy=sampling, weights_gradient_policy=GradientPolicy(policy),
        summation_dtype=torch.int32 if int_mode else torch.float32, _int_rescaler=cfg.get("int_rescaler", 0.001),
        _forward_group_size=cfg.get("G", 32), random_seed=cfg["seed"],
    )
    src, slot, tgt = export_structure(layer)
    n_weights = layer._weights.numel()
    x, W, dY = projection_inputs(cfg, n_weights)
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
    B = cfg["B"]
    I = cfg["in_shape"][0] * cfg["in_shape"][1]
    O = cfg["out_shape"][0] * cfg["out_shape"][1]
    Nt = layer.n_detectors()
    xt = torch.from_numpy(x).view((B, 1) + tuple(cfg["in_shape"]))
    out = {}
    layer.eval()
    out["y_eval"] = t2n(layer.forward_step(xt)).reshape(B, O)
    layer.train()
    y, idx, md, mk = layer.forward_step(xt)
    out.update(y=t2n(y).reshape(B, O), idx=t2n(idx).reshape(B, Nt), min_delta=t2n(md).reshape(B, Nt),
               min_k=t2n(mk).reshape(B, Nt))
    if policy == GradientType.Internal:
        layer.set_external_learning_rate_hook(lambda w: cfg["ext_lr"])
    dx, dw = layer.backward_step(xt, torch.from_numpy(dY).view((B, 1) + tuple(cfg["out_shape"])), idx, md, mk)
    out["dX"] = t2n(dx).reshape(B, I)
    if policy == GradientType.Internal:
        out["W_after"] = t2n(layer._weights)
    else:
        out["dW"] = t2n(dw)
    save(name, dict(cfg, kind="projection", Nt=Nt, n_weights=n_weights, n_lookup_neurons=layer.n_lookup_neurons()),
         anchors=t2n(layer._detector_anchors), syn_source=src.astype(np.int32), syn_slot=slot.astype(np.int32),
         syn_target=tgt.astype(np.int32), **out)


# ----------------------------------------------------------------------------- product-mode sequence layers
def run_product(name, cfg):
    B, S, E, Nt, Nc, O, Npe = cfg["B"], cfg["S"], cfg["E"], cfg["Nt"], cfg["Nc"], cfg["O"], cfg["Npe"]
    int_mode = cfg.get("int_mode", False)
    policy = {"dense": GradientType.Dense, "internal": GradientType.Internal}[cfg.get("policy", "dense")]
    unified = cfg.get("unified_pe", False)
    n_weights = Nt * (1 << Nc) * O
    n_pe = (S - 1) * (1 if unified else Nt) * Npe
    x, anchors, W, pe, dY = sequence_inputs(cfg, n_weights, n_pe)
    ctx = LUTSharedContext(_cmp_eps=cfg.get("cmp_eps", 0.0))
    ctx.to_device(torch.device("cpu"))
    layer = LUTLayer(
        n_inputs=E, n_anchors_per_detector=Nc, n_detectors=Nt, n_outputs=O, sequence_length=S,
        synapse_meta=SynapseMeta(learning_rate=cfg.get("lr_meta", 1.0), min_weight=-1.0, max_weight=1.0),
        concatenation_product=False, sliced_product_mode=cfg.get("sliced", False), positional_dim=Npe,
        unified_pe=unified, weights_gradient_policy=GradientPolicy(policy), shared_context=ctx,
        summation_dtype=torch.int32 if int_mode else torch.float32,
        _explicit_anchors=torch.from_numpy(anchors.reshape(-1).copy()), _int_rescaler=cfg.get("int_rescaler", 0.001),
        random_seed=1,
    )
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
        if pe is not None:
            layer._positional_embeddings.copy_(torch.from_numpy(pe))
    xt = torch.from_numpy(x)
    layer.train()
    pos = layer._prepare_positional_embeddings() if Npe > 0 else None
    if pos is not None:
        pos = pos.detach()
    out = {"y": t2n(layer.forward_step_product(xt, pos)).reshape(B, S, O)}
    if policy == GradientType.Internal:
        layer.set_external_learning_rate_hook(lambda w: cfg["ext_lr"])
    dx, dw, dpe = layer.backward_step_product(xt, pos, torch.from_numpy(dY))
    out["dX"] = t2n(dx).reshape(B, S, E)
    if dpe is not None:
        out["dPE"] = t2n(dpe)  # per (distance, detector, dim): gradient of the repeated embeddings
    if policy == GradientType.Internal:
        out["W_after"] = t2n(layer._weights)
    else:
        out["dW"] = t2n(dw)
    save(name, dict(cfg, kind="product"), in_x=x, in_anchors=anchors, **out)


# ----------------------------------------------------------------------------- concatenation-mode sequence layers
def run_concat(name, cfg):
    B, S, E, Nt, Nc, O, Npe = cfg["B"], cfg["S"], cfg["E"], cfg["Nt"], cfg["Nc"], cfg["O"], cfg["Npe"]
    int_mode = cfg.get("int_mode", False)
    policy = {"dense": GradientType.Dense, "internal": GradientType.Internal}[cfg.get("policy", "dense")]
    unified = cfg.get("unified_pe", False)
    n_weights = Nt * (1 << (2 * Nc + Npe)) * O
    n_pe = (S - 1) * (1 if unified else Nt) * Npe
    x, anchors, W, pe, dY = sequence_inputs(cfg, n_weights, n_pe)
    layer = LUTLayer(
        n_inputs=E, n_anchors_per_detector=Nc, n_detectors=Nt, n_outputs=O, sequence_length=S,
        synapse_meta=SynapseMeta(learning_rate=cfg.get("lr_meta", 1.0), min_weight=-1.0, max_weight=1.0),
        concatenation_product=True, positional_dim=Npe, unified_pe=unified,
        weights_gradient_policy=GradientPolicy(policy),
        summation_dtype=torch.int32 if int_mode else torch.float32,
        _explicit_anchors=torch.from_numpy(anchors.reshape(-1).copy()), _int_rescaler=cfg.get("int_rescaler", 0.001),
        _forward_group_size=cfg.get("G", 32), random_seed=1,
    )
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
        if pe is not None:
            layer._positional_embeddings.copy_(torch.from_numpy(pe))
    xt = torch.from_numpy(x)
    pos = layer._prepare_positional_embeddings() if Npe > 0 else None
    if pos is not None:
        pos = pos.detach()
    layer.eval()
    out = {"y_eval": t2n(layer.forward_step_concat(xt, pos)).reshape(B, S, O)}
    layer.train()
    y, idx, md, mk, pidx, pmd, pmk = layer.forward_step_concat(xt, pos)
    out.update(y=t2n(y).reshape(B, S, O), idx=t2n(idx).reshape(B * S, Nt), min_delta=t2n(md).reshape(B * S, Nt),
               min_k=t2n(mk).reshape(B * S, Nt))
    if Npe > 0:
        out.update(pidx=t2n(pidx).reshape(-1), pmin=t2n(pmd).reshape(-1), pmin_k=t2n(pmk).reshape(-1))
    if policy == GradientType.Internal:
        layer.set_external_learning_rate_hook(lambda w: cfg["ext_lr"])
    dx, dw, dpe = layer.backward_step_concat(xt, torch.from_numpy(dY), idx, md, mk, pidx, pmd, pmk)
    out["dX"] = t2n(dx).reshape(B, S, E)
    if dpe is not None:
        out["dPE"] = t2n(dpe)
    if policy == GradientType.Internal:
        out["W_after"] = t2n(layer._weights)
    else:
        out["dW"] = t2n(dw)
    save(name, dict(cfg, kind="concat"), in_x=x, in_anchors=anchors, **out)


# ----------------------------------------------------------------------------- sparse concatenation-mode layers
def run_concat_sparse(name, cfg):
    from spiky.lut.LUTLayer import Conv2DLUTLayer
    int_mode = cfg.get("int_mode", False)
    policy = {"dense": GradientType.Dense, "internal": GradientType.Internal}[cfg.get("policy", "dense")]
    B, S, Nc, Npe = cfg["B"], cfg["S"], cfg["Nc"], cfg["Npe"]
    layer = Conv2DLUTLayer(
        input_shape=cfg["in_shape"], n_anchors_per_detector=Nc, detectors_shape=cfg["det_shape"],
        output_kernel_shape=cfg["out_kernel"], sequence_length=S, receptive_field_shape=cfg["rf"],
        receptive_field_stride_shape=cfg["rf_stride"], lut_receptive_field_shape=cfg["lut_rf"],
        lut_receptive_field_stride_shape=cfg["lut_rf_stride"],
        synapse_meta=SynapseMeta(learning_rate=cfg.get("lr_meta", 1.0), min_weight=-1.0, max_weight=1.0),
        concatenation_product=True, positional_dim=Npe, unified_pe=cfg.get("unified_pe", False),
        weights_gradient_policy=GradientPolicy(policy), summation_dtype=torch.int32 if int_mode else torch.float32,
        _int_rescaler=cfg.get("int_rescaler", 0.001), _forward_group_size=cfg.get("G", 32), random_seed=cfg["seed"],
    )
    src, slot, tgt = export_structure(layer)
    n_weights = layer._weights.numel()
    Nt, O = layer.n_detectors(), layer.n_outputs()
    E = cfg["in_shape"][0] * cfg["in_shape"][1]
    x, W, pe, dY = concat_sparse_inputs(cfg, n_weights, O, Nt)
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
        if pe is not None:
            layer._positional_embeddings.copy_(torch.from_numpy(pe))
    xt = torch.from_numpy(x).view((B, S) + tuple(cfg["in_shape"]))
    pos = layer._prepare_positional_embeddings() if Npe > 0 else None
    if pos is not None:
        pos = pos.detach()
    layer.eval()
    out = {"y_eval": t2n(layer.forward_step_concat(xt, pos)).reshape(B, S, O)}
    layer.train()
    y, idx, md, mk, pidx, pmd, pmk = layer.forward_step_concat(xt, pos)
    out.update(y=t2n(y).reshape(B, S, O), idx=t2n(idx).reshape(B * S, Nt), min_delta=t2n(md).reshape(B * S, Nt),
               min_k=t2n(mk).reshape(B * S, Nt))
    if Npe > 0:
        out.update(pidx=t2n(pidx).reshape(-1), pmin=t2n(pmd).reshape(-1), pmin_k=t2n(pmk).reshape(-1))
    if policy == GradientType.Internal:
        layer.set_external_learning_rate_hook(lambda w: cfg["ext_lr"])
    dyt = torch.from_numpy(dY).view((B, S) + tuple(layer.output_shape()))
    dx, dw, dpe = layer.backward_step_concat(xt, dyt, idx, md, mk, pidx, pmd, pmk)
    out["dX"] = t2n(dx).reshape(B, S, E)
    if dpe is not None:
        out["dPE"] = t2n(dpe)
    if policy == GradientType.Internal:
        out["W_after"] = t2n(layer._weights)
    else:
        out["dW"] = t2n(dw)
    save(name, dict(cfg, kind="concat_sparse", Nt=Nt, O=O, E=E, n_weights=n_weights,
                    n_lookup_neurons=layer.n_lookup_neurons(), out_shape=tuple(layer.output_shape())),
         anchors=t2n(layer._detector_anchors), syn_source=src.astype(np.int32), syn_slot=slot.astype(np.int32),
         syn_target=tgt.astype(np.int32), **out)



# ----------------------------------------------------------------------------- non-sequence Conv2DLUTLayer
def run_conv2d(name, cfg):
    from spiky.lut.LUTLayer import Conv2DLUTLayer
    int_mode = cfg.get("int_mode", False)
    layer = Conv2DLUTLayer(
        input_shape=cfg["in_shape"], n_anchors_per_detector=cfg["Nc"], detectors_shape=cfg["det_shape"],
        output_kernel_shape=cfg["out_kernel"], receptive_field_shape=cfg["rf"],
        receptive_field_stride_shape=cfg["rf_stride"], lut_receptive_field_shape=cfg["lut_rf"],
        lut_receptive_field_stride_shape=cfg["lut_rf_stride"],
        synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0),
        summation_dtype=torch.int32 if int_mode else torch.float32, _int_rescaler=cfg.get("int_rescaler", 0.001),
        random_seed=cfg["seed"],
    )
    sparse = cfg["lut_rf"] is not None
    extra = {}
    if sparse:
        src, slot, tgt = export_structure(layer)
        extra = dict(syn_source=src.astype(np.int32), syn_slot=slot.astype(np.int32), syn_target=tgt.astype(np.int32))
    n_weights = layer._weights.numel()
    Nt, O = layer.n_detectors(), layer.n_outputs()
    I = cfg["in_shape"][0] * cfg["in_shape"][1]
    B = cfg["B"]
    x, W, dY = conv2d_inputs(cfg, n_weights, O)
    with torch.no_grad():
        layer._weights.copy_(torch.from_numpy(W))
    xt = torch.from_numpy(x).view((B, 1) + tuple(cfg["in_shape"]))
    layer.train()
    y, idx, md, mk = layer.forward_step(xt)
    out = dict(y=t2n(y).reshape(B, O), idx=t2n(idx).reshape(B, Nt), min_delta=t2n(md).reshape(B, Nt),
               min_k=t2n(mk).reshape(B, Nt))
    dx, dw = layer.backward_step(xt, torch.from_numpy(dY).view((B, 1) + tuple(layer.output_shape())), idx, md, mk)
    out.update(dX=t2n(dx).reshape(B, I), dW=t2n(dw))
    save(name, dict(cfg, kind="conv2d", Nt=Nt, O=O, n_weights=n_weights, n_lookup_neurons=layer.n_lookup_neurons(),
                    out_shape=tuple(layer.output_shape()), lut_shape=tuple(layer.lut_shape())),
         anchors=t2n(layer._detector_anchors), **extra, **out)


# ----------------------------------------------------------------------------- whole LUTTransformer models
def run_transformer(name, cfg):
    from spiky.lut.LUTTransformer import LUTTransformer

    int_mode = cfg.get("int_mode", False)
    model = LUTTransformer(
        vocab_size=cfg["V"], embedding_dim=cfg["E"] if isinstance(cfg["E"], int) else tuple(cfg["E"]),
        context_size=cfg["S"], positional_dim=cfg["Npe"],
        num_layers=cfg["layers"], num_heads=cfg["heads"], n_detectors=cfg["Nt"], n_anchors_per_detector=cfg["Nc"],
        n_anchors_per_detector_attention=cfg.get("Nc_att"), no_ffn=cfg.get("no_ffn", False),
        concatenation_product=cfg["concat"], unified_pe=cfg.get("unified_pe", False),
        use_batch_norm=cfg.get("batch_norm", False),
        weights_gradient_policy=GradientPolicy(GradientType.Dense), device=torch.device("cpu"),
        synapse_meta=SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.4, initial_weight=-0.2),
        seed=cfg["seed"], summation_dtype=torch.int32 if int_mode else torch.float32,
        _int_rescaler=cfg.get("int_rescaler", 0.001))
    model.train()
    tokens, dlogits = transformer_inputs(cfg)
    logits = model(torch.from_numpy(tokens))
    logits.backward(torch.from_numpy(dlogits))
    arrays = dict(embedding=t2n(model.token_embedder.weight), logits=t2n(logits))

    def put(prefix, layer):
        arrays[prefix + "_anchors"] = t2n(layer._detector_anchors)
        arrays[prefix + "_W"] = t2n(layer._weights)
        arrays[prefix + "_dW"] = t2n(layer._weights.grad)
        if getattr(layer, "_positional_embeddings", None) is not None:
            arrays[prefix + "_pe"] = t2n(layer._positional_embeddings)
            arrays[prefix + "_dpe"] = t2n(layer._positional_embeddings.grad)

    for li, block in enumerate(model.layers):
        put(f"att{li}", block["attention_lut"])
        if not cfg.get("no_ffn", False):
            put(f"ffn{li}", block["ffn"])
        if cfg.get("batch_norm", False):
            for branch in ("attention", "ffn"):
                bn = block[branch + "_bn"]
                arrays[f"{branch}{li}_bn_dweight"] = t2n(bn.weight.grad)
                arrays[f"{branch}{li}_bn_dbias"] = t2n(bn.bias.grad)
    put("unembedder", model.unembedder)
    save(name, dict(cfg, kind="transformer"), **arrays)


def main():
    prefixes = sys.argv[1:]
    for name, cfg in NONSEQ_FC_CASES.items():
        if not prefixes or any(name.startswith(p) for p in prefixes):
            run_nonseq_fc(name, cfg)
    for name, cfg in CONCAT_CASES.items():
        if not prefixes or any(name.startswith(p) for p in prefixes):
            run_concat(name, cfg)
    for name, cfg in PRODUCT_CASES.items():
        if not prefixes or any(name.startswith(p) for p in prefixes):
            run_product(name, cfg)
    for name, cfg in PROJECTION_CASES.items():
        if not prefixes or any(name.startswith(p) for p in prefixes):
            run_projection(name, cfg)
    for name, cfg in TRANSFORMER_CASES.items():
        if not prefixes or any(name.startswith(p) for p in prefixes):
            run_transformer(name, cfg)
    for name, cfg in CONV2D_CASES.items():
        if not prefixes or any(name.startswith(p) for p in prefixes):
            run_conv2d(name, cfg)
    for name, cfg in CONCAT_SPARSE_CASES.items():
        if not prefixes or any(name.startswith(p) for p in prefixes):
            run_concat_sparse(name, cfg)


if __name__ == "__main__":
    main()
