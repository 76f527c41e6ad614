"""T5 encoder-decoder with Hugging Face parameter names.

Attention has no 1/sqrt(d) scaling and adds a learned relative-position bias
(bucketed distances, one table per stack owned by block 0).  The bias is not
materialised as ``[H, Sq, Sk]``: the table itself is handed to
:func:`slapo_b200.ops.functional.flash_attention`, whose CUDA kernels look it
up in-line and accumulate its gradient.  The feed-forward is ``relu`` or
gated GeLU (``wi_0`` / ``wi_1``), both shardable.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import functional as NF


@dataclass
class T5Config:
    vocab_size: int = 32128
    d_model: int = 512
    d_kv: int = 64
    d_ff: int = 2048
    num_layers: int = 6
    num_decoder_layers: int = None
    num_heads: int = 8
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128
    dropout_rate: float = 0.1
    layer_norm_epsilon: float = 1e-6
    feed_forward_proj: str = "relu"   # or "gated-gelu"
    initializer_factor: float = 1.0
    tie_word_embeddings: bool = True
    attn_op_name: str = "auto"
    model_type: str = "t5"

    def __post_init__(self):
        if self.num_decoder_layers is None:
            self.num_decoder_layers = self.num_layers

    @property
    def is_gated_act(self):
        return self.feed_forward_proj.startswith("gated")

    @property
    def hidden_size(self):
        return self.d_model

    @classmethod
    def t5_large(cls, **kw):
        return cls(d_model=1024, d_kv=64, d_ff=2816, num_layers=24, num_heads=16,
                   feed_forward_proj="gated-gelu", **kw)


class T5LayerNorm(nn.Module):
    """RMS norm (no mean subtraction, no bias)."""

    def __init__(self, hidden_size, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, x):
        return NF.rms_norm(x, self.weight, self.variance_epsilon)


class T5DenseActDense(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.wi = nn.Linear(config.d_model, config.d_ff, bias=False)
        self.wo = nn.Linear(config.d_ff, config.d_model, bias=False)
        self.dropout = nn.Dropout(config.dropout_rate)

    def forward(self, x):
        return self.wo(self.dropout(F.relu(self.wi(x))))


class T5DenseGatedActDense(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.wi_0 = nn.Linear(config.d_model, config.d_ff, bias=False)
        self.wi_1 = nn.Linear(config.d_model, config.d_ff, bias=False)
        self.wo = nn.Linear(config.d_ff, config.d_model, bias=False)
        self.dropout = nn.Dropout(config.dropout_rate)

    def forward(self, x):
        gate = F.gelu(self.wi_0(x), approximate="tanh")
        return self.wo(self.dropout(gate * self.wi_1(x)))


class T5LayerFF(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.DenseReluDense = T5DenseGatedActDense(config) if config.is_gated_act \
            else T5DenseActDense(config)
        self.layer_norm = T5LayerNorm(config.d_model, config.layer_norm_epsilon)
        self.dropout = nn.Dropout(config.dropout_rate)

    def forward(self, hidden_states):
        return hidden_states + self.dropout(self.DenseReluDense(self.layer_norm(hidden_states)))


class T5Attention(nn.Module):
    """Self- or cross-attention on ``[B, S, H, D]`` views; ``rel_table`` is the
    stack's ``[buckets, H_local]`` relative-position table (or None)."""

    traceable = False

    def __init__(self, config, has_relative_attention_bias=False, causal=False):
        super().__init__()
        self.n_heads = config.num_heads
        self.d_kv = config.d_kv
        inner = config.num_heads * config.d_kv
        self.q = nn.Linear(config.d_model, inner, bias=False)
        self.k = nn.Linear(config.d_model, inner, bias=False)
        self.v = nn.Linear(config.d_model, inner, bias=False)
        self.o = nn.Linear(inner, config.d_model, bias=False)
        self.causal = causal
        self.dropout = config.dropout_rate
        self.num_buckets = config.relative_attention_num_buckets
        self.max_distance = config.relative_attention_max_distance
        self.attn_op_name = config.attn_op_name
        if has_relative_attention_bias:
            self.relative_attention_bias = nn.Embedding(self.num_buckets, self.n_heads)

    def forward(self, hidden_states, key_value_states=None, key_bias=None, rel_table=None):
        kv_in = hidden_states if key_value_states is None else key_value_states
        shape = lambda t: t.view(t.shape[:-1] + (-1, self.d_kv))  # noqa: E731
        q, k, v = shape(self.q(hidden_states)), shape(self.k(kv_in)), shape(self.v(kv_in))
        kwargs = dict(key_padding_bias=key_bias, causal=self.causal, scale=1.0,
                      dropout_p=self.dropout, training=self.training, rel_bias_table=rel_table,
                      rel_bidirectional=not self.causal, rel_max_distance=self.max_distance)
        if self.attn_op_name == "reference":
            ctx = NF.attention_reference(q, k, v, **kwargs)
        else:
            ctx = NF.flash_attention(q, k, v, **kwargs)
        return self.o(ctx.reshape(ctx.shape[:-2] + (-1,)))


class T5FusedAttention(nn.Module):
    """:class:`T5Attention` with its projections fused: self-attention computes q, k and v
    with ONE GEMM (``qkv``), cross-attention k and v of the encoder output with one (``kv``)
    next to ``q``.  Weight rows are ordered ``[head][q | k | v][d_kv]`` (``[head][k | v][d_kv]``),
    so slicing axis 0 by the tensor-parallel size hands each rank whole heads, and the
    projection output is read in place as strided ``[B, S, H, D]`` views - the packed
    flash-attention path takes them without a copy.

    Parity: the horizontal ``replace`` of q/k/v by ``FusedQKV`` and of cross-attention k/v by
    ``FusedKV`` + ``ShardableQ`` (slapo/model_schedule/t5.py:95-143, 168-200 of the reference)."""

    traceable = False

    def __init__(self, attn: "T5Attention", cross: bool):
        super().__init__()
        self.n_heads, self.d_kv, self.cross = attn.n_heads, attn.d_kv, cross
        self.causal, self.dropout = attn.causal, attn.dropout
        self.num_buckets, self.max_distance = attn.num_buckets, attn.max_distance
        self.attn_op_name = attn.attn_op_name
        d_model = attn.q.weight.shape[1]
        inner = self.n_heads * self.d_kv
        meta = attn.q.weight.is_meta
        kw = dict(bias=False, device=attn.q.weight.device, dtype=attn.q.weight.dtype)

        def pack(*mats):
            parts = [m.reshape(self.n_heads, self.d_kv, d_model) for m in mats]
            return torch.cat(parts, dim=1).reshape(-1, d_model)

        if cross:
            self.q = attn.q
            self.kv = nn.Linear(d_model, 2 * inner, **kw)
            if not meta:
                self.kv.weight = nn.Parameter(pack(attn.k.weight.data, attn.v.weight.data))
        else:
            self.qkv = nn.Linear(d_model, 3 * inner, **kw)
            if not meta:
                self.qkv.weight = nn.Parameter(pack(attn.q.weight.data, attn.k.weight.data,
                                                    attn.v.weight.data))
        self.o = attn.o
        if hasattr(attn, "relative_attention_bias"):
            self.relative_attention_bias = attn.relative_attention_bias

    def forward(self, hidden_states, key_value_states=None, key_bias=None, rel_table=None):
        d = self.d_kv
        if self.cross:
            q = self.q(hidden_states)
            q = q.view(q.shape[:-1] + (-1, d))
            kv = self.kv(key_value_states)
            kv = kv.view(kv.shape[:-1] + (-1, 2, d))        # -1 absorbs a split of the heads
            k, v = kv[..., 0, :], kv[..., 1, :]
        else:
            qkv = self.qkv(hidden_states)
            qkv = qkv.view(qkv.shape[:-1] + (-1, 3, d))
            q, k, v = qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :]
        kwargs = dict(key_padding_bias=key_bias, causal=self.causal, scale=1.0,
                      dropout_p=self.dropout, training=self.training, rel_bias_table=rel_table,
                      rel_bidirectional=not self.causal, rel_max_distance=self.max_distance)
        if self.attn_op_name == "reference":
            ctx = NF.attention_reference(q, k, v, **kwargs)
        else:
            ctx = NF.flash_attention(q, k, v, **kwargs)
        return self.o(ctx.reshape(ctx.shape[:-2] + (-1,)))


class T5LayerSelfAttention(nn.Module):
    def __init__(self, config, has_relative_attention_bias, causal):
        super().__init__()
        self.SelfAttention = T5Attention(config, has_relative_attention_bias, causal)
        self.layer_norm = T5LayerNorm(config.d_model, config.layer_norm_epsilon)
        self.dropout = nn.Dropout(config.dropout_rate)

    def forward(self, hidden_states, key_bias=None, rel_table=None):
        out = self.SelfAttention(self.layer_norm(hidden_states), None, key_bias, rel_table)
        return hidden_states + self.dropout(out)


class T5LayerCrossAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.EncDecAttention = T5Attention(config, False, False)
        self.layer_norm = T5LayerNorm(config.d_model, config.layer_norm_epsilon)
        self.dropout = nn.Dropout(config.dropout_rate)

    def forward(self, hidden_states, encoder_hidden_states, enc_key_bias=None):
        out = self.EncDecAttention(self.layer_norm(hidden_states), encoder_hidden_states,
                                   enc_key_bias, None)
        return hidden_states + self.dropout(out)


class T5Block(nn.Module):
    def __init__(self, config, is_decoder, has_relative_attention_bias):
        super().__init__()
        self.is_decoder = is_decoder
        layers = [T5LayerSelfAttention(config, has_relative_attention_bias, is_decoder)]
        if is_decoder:
            layers.append(T5LayerCrossAttention(config))
        layers.append(T5LayerFF(config))
        self.layer = nn.ModuleList(layers)

    def forward(self, hidden_states, key_bias=None, rel_table=None, encoder_hidden_states=None,
                enc_key_bias=None):
        hidden_states = self.layer[0](hidden_states, key_bias, rel_table)
        if self.is_decoder:
            hidden_states = self.layer[1](hidden_states, encoder_hidden_states, enc_key_bias)
        return self.layer[-1](hidden_states)


class T5Stack(nn.Module):
    def __init__(self, config, embed_tokens, is_decoder):
        super().__init__()
        self.is_decoder = is_decoder
        self.embed_tokens = embed_tokens
        n = config.num_decoder_layers if is_decoder else config.num_layers
        self.block = nn.ModuleList([T5Block(config, is_decoder, i == 0) for i in range(n)])
        self.final_layer_norm = T5LayerNorm(config.d_model, config.layer_norm_epsilon)
        self.dropout = nn.Dropout(config.dropout_rate)

    def _rel_table(self):
        # looked up by name: block 0 may be wrapped (checkpointing) or have had its
        # attention replaced by a scheduled variant
        for name, mod in self.block[0].named_modules():
            if name.endswith("relative_attention_bias"):
                return mod.weight
        raise AttributeError("block 0 owns no relative_attention_bias")

    def forward(self, input_ids, attention_mask=None, encoder_hidden_states=None,
                encoder_attention_mask=None):
        hidden = self.dropout(self.embed_tokens(input_ids))
        key_bias = None if attention_mask is None else (1.0 - attention_mask.float()) * -10000.0
        enc_bias = None if encoder_attention_mask is None else \
            (1.0 - encoder_attention_mask.float()) * -10000.0
        rel_table = self._rel_table()
        for blk in self.block:
            hidden = blk(hidden, key_bias, rel_table, encoder_hidden_states, enc_bias)
        return self.dropout(self.final_layer_norm(hidden))


class T5ForConditionalGeneration(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.shared = nn.Embedding(config.vocab_size, config.d_model)
        self.encoder = T5Stack(config, self.shared, False)
        self.decoder = T5Stack(config, self.shared, True)
        self.lm_head = nn.Linear(config.d_model, config.vocab_size, bias=False)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.shared.weight

    def _init_weights(self, module):
        f = self.config.initializer_factor
        d = self.config.d_model
        if isinstance(module, T5LayerNorm):
            module.weight.data.fill_(f)
        elif isinstance(module, nn.Embedding):
            module.weight.data.normal_(mean=0.0, std=f)
        elif isinstance(module, nn.Linear):
            module.weight.data.normal_(mean=0.0, std=f * (module.in_features ** -0.5))
            if module.bias is not None:
                module.bias.data.zero_()
        del d

    def init_weights(self):
        self.apply(self._init_weights)
        return self

    def forward(self, input_ids, decoder_input_ids, attention_mask=None,
                decoder_attention_mask=None, labels=None):
        enc = self.encoder(input_ids, attention_mask)
        dec = self.decoder(decoder_input_ids, decoder_attention_mask, enc, attention_mask)
        if self.config.tie_word_embeddings:
            dec = dec * (self.config.d_model ** -0.5)
        logits = self.lm_head(dec)
        if labels is None:
            return {"logits": logits}
        return {"loss": seq2seq_loss(logits, labels), "logits": logits}


def seq2seq_loss(logits, labels, tp_group=None, vocab_parallel=False):
    from ..ops.cross_entropy import LOCAL, vocab_parallel_cross_entropy

    per_tok = vocab_parallel_cross_entropy(logits.contiguous(), labels,
                                           tp_group if vocab_parallel else LOCAL)
    n_valid = (labels != -100).sum().clamp(min=1)
    return per_tok.float().sum() / n_valid
