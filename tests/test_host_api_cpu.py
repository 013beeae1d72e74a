"""Host-side behaviour of the layer mirror that needs no GPU: pickling (the reference's data manager is picklable,
spiky_cuda/lut/lut.cu:1652-1655), the no-CPU-execution rule, constructor argument errors."""
import pickle

import pytest
import torch


def _meta():
    from spiky_b200.lut_layer import SynapseMeta

    return SynapseMeta(min_weight=-1.0, max_weight=1.0, initial_noise_level=0.1)


def _layers():
    from spiky_b200.lut_layer import Conv2DLUTLayer, LUTLayer, ProjectionLUTLayer

    yield LUTLayer(16, 3, 4, 5, synapse_meta=_meta(), random_seed=1, device=None)
    yield LUTLayer(8, 3, 4, 8, sequence_length=6, positional_dim=2, concatenation_product=False, synapse_meta=_meta(),
                   random_seed=1, device=None)
    yield ProjectionLUTLayer((16, 16), (12, 12), 4, 10, 4, (5, 5), (3, 3), synapse_meta=_meta(), random_seed=2,
                             device=None)
    yield Conv2DLUTLayer(input_shape=(8, 8), n_anchors_per_detector=3, detectors_shape=(2, 2),
                         output_kernel_shape=(2, 2), receptive_field_shape=(4, 4), receptive_field_stride_shape=(2, 2),
                         lut_receptive_field_shape=(2, 2), lut_receptive_field_stride_shape=(2, 2),
                         synapse_meta=_meta(), random_seed=3, device=None)


def test_layers_pickle_with_structure_and_weights():
    for layer in _layers():
        copy = pickle.loads(pickle.dumps(layer))
        assert type(copy) is type(layer)
        assert torch.equal(copy._weights, layer._weights)
        assert torch.equal(copy._detector_anchors, layer._detector_anchors)
        assert copy.n_synapses() == layer.n_synapses() and copy.n_outputs() == layer.n_outputs()
        assert repr(copy._lut_dm) == repr(layer._lut_dm)
        a, b = layer._lut_dm._sparse, copy._lut_dm._sparse
        assert (a is None) == (b is None)
        if a is not None:
            for field in a._TENSORS:
                assert torch.equal(getattr(a, field), getattr(b, field)), field
        if layer._positional_embeddings is not None:
            assert torch.equal(copy._positional_embeddings, layer._positional_embeddings)


def test_transformer_pickles_and_state_dict_round_trips():
    from spiky_b200.lut_transformer import LUTTransformer

    kw = dict(vocab_size=20, embedding_dim=16, context_size=8, positional_dim=4, num_layers=2, num_heads=2,
              n_detectors=4, n_anchors_per_detector=4, concatenation_product=False, device=None, synapse_meta=_meta())
    model = LUTTransformer(seed=1, **kw)
    copy = pickle.loads(pickle.dumps(model))
    other = LUTTransformer(seed=2, **kw)
    other.load_state_dict(model.state_dict())
    for twin in (copy, other):
        for (ka, va), (kb, vb) in zip(model.state_dict().items(), twin.state_dict().items()):
            assert ka == kb and torch.equal(va, vb), ka
    # anchors are structure, carried as buffers: a checkpoint restores them too
    assert any("anchors" in k for k in model.state_dict())


def test_cpu_resident_layer_refuses_to_run():
    """There is no CPU execution path: a runtime call on a layer that was never moved to a GPU raises instead of
    computing something somewhere else."""
    layer = next(_layers())
    with pytest.raises((RuntimeError, ValueError, AssertionError)):
        layer(torch.rand(2, 1, 16))


def test_constructor_argument_errors():
    from spiky_b200.lut_layer import GradientPolicy, GradientType, LUTLayer

    with pytest.raises(ValueError):
        GradientPolicy(GradientType.Internal, normalized=True)
    with pytest.raises(ValueError):
        LUTLayer(16, 3, 4, 5, synapse_meta=_meta(), summation_dtype=torch.int32,
                 weights_gradient_policy=GradientPolicy(GradientType.Internal), device=None)
    layer = LUTLayer(16, 3, 4, 5, synapse_meta=_meta(), device=None)
    with pytest.raises(ValueError):
        layer.set_external_learning_rate_hook(lambda w: 0.1)  # only for the Internal policy


def test_quantize_tables_is_symmetric_per_table():
    from spiky_b200.inference import LUTInference, quantize_tables

    gen = torch.Generator().manual_seed(9)
    Nt, T, O = 5, 8, 4
    w = torch.randn(Nt * T * O, generator=gen) * torch.tensor([0.01, 0.1, 1.0, 3.0, 0.0]).repeat_interleave(T * O)
    q, scale = quantize_tables(w, Nt, T, O)
    assert q.dtype == torch.int8 and q.shape == w.shape and scale.shape == (Nt,)
    per = w.view(Nt, -1)
    assert torch.allclose(scale[:4], per[:4].abs().amax(dim=1) / 127.0)
    assert scale[4] > 0 and not q.view(Nt, -1)[4].any()          # an all-zero table keeps a usable scale
    assert int(q.abs().max()) == 127 and int(q.min()) >= -127    # symmetric range, -128 unused
    back = q.view(Nt, -1).float() * scale[:, None]
    assert bool(((back - per).abs() <= scale[:, None] / 2 + 1e-12).all())
    # shard boundaries must keep whole detector blocks
    anchors = torch.zeros(64 * 3 * 2, dtype=torch.int32)
    tables = torch.zeros(64 * 8 * 4)
    with pytest.raises(AssertionError):
        LUTInference.shard_of(0, 3, 16, 4, 64, 3, anchors, tables)          # 64 detectors over 3 ranks
    with pytest.raises(AssertionError):
        LUTInference.shard_of(0, 4, 16, 4, 64, 3, anchors, tables)          # 16 per rank, blocks of 32
