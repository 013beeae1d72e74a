"""LUT transformer built from the LUT layers of :mod:`spiky_b200.lut_layer`.

Same constructor arguments, attribute names and forward contract as the reference's
``spiky.lut.LUTTransformer`` (src/spiky/lut/LUTTransformer.py:69-271): a frozen token embedding, then
``num_layers`` blocks of [LUT attention over the whole context -> dropout -> (BatchNorm1d) -> residual,
LUT feed-forward on every token -> dropout -> (BatchNorm1d) -> residual], then a LUT unembedder to the
vocabulary.  ``forward(tokens[B, S]) -> logits[B, S, V]``.
"""
import torch
import torch.nn as nn

from .lut_layer import (Conv2DLUTLayer, GradientPolicy, GradientType, LUTLayer, LUTSharedContext,  # noqa: F401
                        SynapseMeta, _normalise_device)


class LUTTransformer(nn.Module):
    def __init__(self, vocab_size, embedding_dim, context_size, positional_dim, num_layers, num_heads, n_detectors,
                 n_anchors_per_detector, n_anchors_per_detector_attention=None, no_ffn=False,
                 concatenation_product=True, sliced_product_mode=False, unified_pe=False, do_normalise_weights=False,
                 weights_gradient_policy=None, device=None, synapse_meta=SynapseMeta(), lut_shared_context=None,
                 seed=None, summation_dtype=torch.float32, _int_rescaler=0.001, _forward_group_size=32,
                 _backward_group_size=32, dropout=0.0, use_batch_norm=False):
        super().__init__()
        self.vocab_size = vocab_size
        self.embedding_dim = embedding_dim
        self.context_size = context_size
        self.positional_dim = positional_dim
        self.num_layers = num_layers
        self.num_heads = num_heads
        self.n_detectors = n_detectors
        self.n_anchors_per_detector = n_anchors_per_detector
        self.n_anchors_per_detector_attention = (n_anchors_per_detector_attention
                                                 if n_anchors_per_detector_attention is not None
                                                 else n_anchors_per_detector)
        self.concatenation_product = concatenation_product
        self.sliced_product_mode = sliced_product_mode
        self.weights_gradient_policy = weights_gradient_policy
        self.dropout = dropout
        self.use_batch_norm = use_batch_norm
        self.unified_pe = unified_pe
        self.no_ffn = no_ffn
        self.device = torch.device("cpu") if device is None else _normalise_device(device)
        self.lut_shared_context = (LUTSharedContext().to_device(self.device) if lut_shared_context is None
                                   else lut_shared_context)
        self._debug_last_forward = None

        flat = isinstance(embedding_dim, int)
        n_emb = embedding_dim if flat else embedding_dim[0] * embedding_dim[1]
        self._n_embeddings = n_emb

        # frozen random token embedding in [-1, 1]
        self.token_embedder = nn.Embedding(vocab_size, n_emb, device=self.device)
        self.token_embedder.weight.requires_grad_(False)
        with torch.no_grad():
            if seed is not None:
                gen = torch.Generator(device="cpu").manual_seed(seed)
                table = 2 * torch.rand(self.token_embedder.weight.shape, generator=gen) - 1.0
                self.token_embedder.weight.copy_(table)
            else:
                nn.init.uniform_(self.token_embedder.weight, -1.0, 1.0)

        common = dict(synapse_meta=synapse_meta, do_normalise_weights=do_normalise_weights,
                      weights_gradient_policy=weights_gradient_policy, shared_context=self.lut_shared_context,
                      summation_dtype=summation_dtype, _int_rescaler=_int_rescaler, device=self.device,
                      _forward_group_size=_forward_group_size, _backward_group_size=_backward_group_size)

        def per_token_lut(n_outputs, layer_seed):
            # sequences are processed token by token through a reshape [B, S, E] -> [B * S, 1, E]
            return LUTLayer(n_inputs=n_emb, n_outputs=n_outputs, n_detectors=n_detectors,
                            n_anchors_per_detector=n_anchors_per_detector, sequence_length=1, random_seed=layer_seed,
                            **common)

        def attention_lut(layer_seed):
            seq = dict(sequence_length=context_size, concatenation_product=concatenation_product,
                       sliced_product_mode=sliced_product_mode, positional_dim=positional_dim, unified_pe=unified_pe,
                       n_anchors_per_detector=self.n_anchors_per_detector_attention, random_seed=layer_seed, **common)
            if flat:
                return LUTLayer(n_inputs=embedding_dim, n_outputs=embedding_dim, n_detectors=n_detectors * num_heads,
                                **seq)
            # 2-D embeddings (used by the reference's tests only): one receptive field covering the whole input
            return Conv2DLUTLayer(input_shape=embedding_dim, detectors_shape=(1, n_detectors * num_heads),
                                  output_kernel_shape=embedding_dim, receptive_field_shape=embedding_dim,
                                  receptive_field_stride_shape=embedding_dim, **seq)

        self.layers = nn.ModuleList()
        for li in range(num_layers):
            block = nn.ModuleDict()
            base = None if seed is None else seed + li * num_heads
            block["attention_lut"] = attention_lut(base)
            block["attention_dropout"] = nn.Dropout(dropout)
            block["attention_bn"] = nn.BatchNorm1d(n_emb, device=self.device) if use_batch_norm else None
            if not no_ffn:
                block["ffn"] = per_token_lut(n_emb, None if seed is None else base + num_heads)
                block["ffn_dropout"] = nn.Dropout(dropout)
                block["ffn_bn"] = nn.BatchNorm1d(n_emb, device=self.device) if use_batch_norm else None
            self.layers.append(block)
        self.unembedder = per_token_lut(vocab_size, seed)

    # ------------------------------------------------------------------ helpers
    def _lut_layers(self):
        for block in self.layers:
            yield block["attention_lut"]
            if not self.no_ffn:
                yield block["ffn"]
        yield self.unembedder

    def set_external_learning_rate_hook(self, lr_hook):
        for layer in self._lut_layers():
            layer.set_external_learning_rate_hook(lr_hook)

    def _reset_shared_context(self, new_context):
        for layer in self._lut_layers():
            layer._reset_shared_context(new_context)

    def to(self, *args, **kwargs):
        device = kwargs.get("device", None)
        if device is None and args and not isinstance(args[0], torch.dtype):
            device = args[0]
        # strings and ordinals name a device in both the positional and the keyword form
        if isinstance(device, (str, int)) and not isinstance(device, bool):
            try:
                device = torch.device(device)
            except (RuntimeError, ValueError):
                device = None
        super().to(*args, **kwargs)
        if isinstance(device, torch.device):
            dev = _normalise_device(device)
            self.device = dev
            self.lut_shared_context.to_device(dev)
            for layer in self._lut_layers():
                layer.to(device=dev)
        return self

    @staticmethod
    def _residual_branch(z, out, dropout, bn):
        out = dropout(out)
        if bn is not None:
            out = bn(out.reshape(-1, out.shape[-1])).reshape(out.shape)
        return z + out

    # ------------------------------------------------------------------ forward
    def forward(self, tokens):
        """tokens: int64 [B, context_size] -> logits fp32 [B, context_size, vocab_size]."""
        B, S, E = tokens.shape[0], self.context_size, self._n_embeddings
        record = self._debug_last_forward is not None
        if record:
            self._debug_last_forward = [tokens.to(dtype=torch.float32)]
        z = self.token_embedder(tokens)
        if record:
            self._debug_last_forward.append(z.detach().clone())
        flat = isinstance(self.embedding_dim, int)
        for block in self.layers:
            att_in = z if flat else z.reshape((B, S) + tuple(self.embedding_dim))
            att = block["attention_lut"](att_in.contiguous()).reshape(B, S, E)
            if record:
                self._debug_last_forward.append(att.detach().clone())
            z = self._residual_branch(z, att, block["attention_dropout"], block["attention_bn"])
            if not self.no_ffn:
                ffn = block["ffn"](z.reshape(B * S, 1, E)).reshape(B, S, E)
                if record:
                    self._debug_last_forward.append(ffn.detach().clone())
                z = self._residual_branch(z, ffn, block["ffn_dropout"], block["ffn_bn"])
        return self.unembedder(z.reshape(B * S, 1, E)).reshape(B, S, self.vocab_size)

    def get_profile_statistics(self) -> str:
        """Kernel timings collected by the opt-in profiler of the CUDA library, one line per kernel family."""
        from . import _native

        lines = []
        for name, rec in _native.profiler_read().items():
            if rec["launches"]:
                avg = rec["ms"] / rec["timed"] if rec["timed"] else 0.0
                lines.append(f"lut::runtime::{name}: {rec['ms']:.4f} ms / {rec['launches']} = {avg:.4f} ms")
        return "\n".join(lines)
