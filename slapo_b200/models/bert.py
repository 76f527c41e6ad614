"""BERT / RoBERTa encoder family with Hugging Face parameter names.

The module tree and parameter names match ``transformers``' BERT
(``bert.encoder.layer.N.attention.self.query`` ...), so path-based schedules
and checkpoints written against HF models apply unchanged; the
implementation is independent, free of data-dependent control flow and
therefore traceable level by level with ``torch.fx``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    hidden_act: str = "gelu"
    hidden_dropout_prob: float = 0.1
    attention_probs_dropout_prob: float = 0.1
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-12
    pad_token_id: int = 0
    position_offset: int = 0  # RoBERTa: pad_token_id + 1
    model_type: str = "bert"

    @classmethod
    def large(cls, **kw):
        return cls(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16,
                   intermediate_size=4096, **kw)

    @classmethod
    def base(cls, **kw):
        return cls(**kw)


def _act(name):
    if name == "gelu":
        return nn.GELU()
    if name in ("gelu_new", "gelu_tanh", "gelu_pytorch_tanh"):
        return nn.GELU(approximate="tanh")
    if name == "relu":
        return nn.ReLU()
    raise ValueError(f"unsupported activation {name}")


class BertEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.word_embeddings = nn.Embedding(config.vocab_size, config.hidden_size,
                                            padding_idx=config.pad_token_id)
        self.position_embeddings = nn.Embedding(
            config.max_position_embeddings + config.position_offset, config.hidden_size)
        self.token_type_embeddings = nn.Embedding(config.type_vocab_size, config.hidden_size)
        self.LayerNorm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)
        self.position_offset = config.position_offset
        self.register_buffer(
            "position_ids",
            torch.arange(config.max_position_embeddings).unsqueeze(0) + config.position_offset,
            persistent=False)

    def forward(self, input_ids, token_type_ids=None, position_ids=None):
        seq_len = input_ids.size(1)
        if position_ids is None:
            position_ids = self.position_ids[:, :seq_len]
        emb = self.word_embeddings(input_ids) + self.position_embeddings(position_ids)
        if token_type_ids is None:
            emb = emb + self.token_type_embeddings.weight[0]
        else:
            emb = emb + self.token_type_embeddings(token_type_ids)
        return self.dropout(self.LayerNorm(emb))


class BertSelfAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.num_attention_heads = config.num_attention_heads
        self.attention_head_size = config.hidden_size // config.num_attention_heads
        self.all_head_size = config.hidden_size
        self.query = nn.Linear(config.hidden_size, config.hidden_size)
        self.key = nn.Linear(config.hidden_size, config.hidden_size)
        self.value = nn.Linear(config.hidden_size, config.hidden_size)
        self.dropout = nn.Dropout(config.attention_probs_dropout_prob)

    def transpose_for_scores(self, x):
        new_shape = x.size()[:-1] + (-1, self.attention_head_size)
        return x.view(new_shape).permute(0, 2, 1, 3)

    def forward(self, hidden_states, attention_mask=None):
        q = self.transpose_for_scores(self.query(hidden_states))
        k = self.transpose_for_scores(self.key(hidden_states))
        v = self.transpose_for_scores(self.value(hidden_states))
        scores = torch.matmul(q, k.transpose(-1, -2)) / (self.attention_head_size ** 0.5)
        if attention_mask is not None:
            scores = scores + attention_mask
        probs = self.dropout(F.softmax(scores, dim=-1))
        ctx = torch.matmul(probs, v).permute(0, 2, 1, 3).contiguous()
        ctx = ctx.view(ctx.size()[:-2] + (-1,))
        return (ctx, None)


class BertSelfOutput(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = nn.Linear(config.hidden_size, config.hidden_size)
        self.LayerNorm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)

    def forward(self, hidden_states, input_tensor):
        hidden_states = self.dropout(self.dense(hidden_states))
        return self.LayerNorm(hidden_states + input_tensor)


class BertAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.self = BertSelfAttention(config)
        self.output = BertSelfOutput(config)

    def forward(self, hidden_states, attention_mask=None):
        self_out = self.self(hidden_states, attention_mask)
        return self.output(self_out[0], hidden_states)


class BertIntermediate(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = nn.Linear(config.hidden_size, config.intermediate_size)
        self.intermediate_act_fn = _act(config.hidden_act)

    def forward(self, hidden_states):
        return self.intermediate_act_fn(self.dense(hidden_states))


class BertOutput(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = nn.Linear(config.intermediate_size, config.hidden_size)
        self.LayerNorm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)

    def forward(self, hidden_states, input_tensor):
        hidden_states = self.dropout(self.dense(hidden_states))
        return self.LayerNorm(hidden_states + input_tensor)


class BertLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.attention = BertAttention(config)
        self.intermediate = BertIntermediate(config)
        self.output = BertOutput(config)

    def forward(self, hidden_states, attention_mask=None):
        attn = self.attention(hidden_states, attention_mask)
        return self.output(self.intermediate(attn), attn)


class BertEncoder(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layer = nn.ModuleList([BertLayer(config) for _ in range(config.num_hidden_layers)])

    def forward(self, hidden_states, attention_mask=None):
        for layer in self.layer:
            hidden_states = layer(hidden_states, attention_mask)
        return hidden_states


class BertPooler(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = nn.Linear(config.hidden_size, config.hidden_size)
        self.activation = nn.Tanh()

    def forward(self, hidden_states):
        return self.activation(self.dense(hidden_states[:, 0]))


class BertPreTrainedModel(nn.Module):
    def _init_weights(self, module):
        std = self.config.initializer_range
        if isinstance(module, nn.Linear):
            module.weight.data.normal_(mean=0.0, std=std)
            if module.bias is not None:
                module.bias.data.zero_()
        elif isinstance(module, nn.Embedding):
            module.weight.data.normal_(mean=0.0, std=std)
            if module.padding_idx is not None and module.padding_idx < module.weight.shape[0]:
                module.weight.data[module.padding_idx].zero_()
        elif isinstance(module, nn.LayerNorm):
            module.bias.data.zero_()
            module.weight.data.fill_(1.0)
        elif isinstance(module, (BertLMPredictionHead, RobertaLMHead)):
            module.bias.data.zero_()

    def init_weights(self):
        self.apply(self._init_weights)
        return self


class BertModel(BertPreTrainedModel):
    def __init__(self, config, add_pooling_layer=True):
        super().__init__()
        self.config = config
        self.embeddings = BertEmbeddings(config)
        self.encoder = BertEncoder(config)
        self.pooler = BertPooler(config) if add_pooling_layer else None

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None):
        ext_mask = None
        if attention_mask is not None:
            ext_mask = (1.0 - attention_mask[:, None, None, :].to(
                self.embeddings.LayerNorm.weight.dtype)) * -10000.0
        hidden = self.embeddings(input_ids, token_type_ids, position_ids)
        hidden = self.encoder(hidden, ext_mask)
        pooled = self.pooler(hidden) if self.pooler is not None else None
        return {"last_hidden_state": hidden, "pooler_output": pooled}


class BertPredictionHeadTransform(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = nn.Linear(config.hidden_size, config.hidden_size)
        self.transform_act_fn = _act(config.hidden_act)
        self.LayerNorm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)

    def forward(self, hidden_states):
        return self.LayerNorm(self.transform_act_fn(self.dense(hidden_states)))


class BertLMPredictionHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.transform = BertPredictionHeadTransform(config)
        self.decoder = nn.Linear(config.hidden_size, config.vocab_size, bias=True)
        self.bias = nn.Parameter(torch.zeros(config.vocab_size))
        # one bias under two names, like Hugging Face: the GEMM adds it
        self.decoder.bias = self.bias

    def forward(self, hidden_states):
        return self.decoder(self.transform(hidden_states))


class BertOnlyMLMHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.predictions = BertLMPredictionHead(config)

    def forward(self, sequence_output):
        return self.predictions(sequence_output)


class BertForMaskedLM(BertPreTrainedModel):
    """BERT with the masked-LM head; the decoder weight is tied to the word
    embedding.  ``forward`` returns ``{"logits"}`` or, given ``labels``
    (``-100`` = ignore), ``{"loss", "logits"}``."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.bert = BertModel(config, add_pooling_layer=False)
        self.cls = BertOnlyMLMHead(config)
        self.tie_weights()

    def tie_weights(self):
        self.cls.predictions.decoder.weight = self.bert.embeddings.word_embeddings.weight

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None,
                labels=None):
        hidden = self.bert(input_ids, attention_mask, token_type_ids, position_ids)[
            "last_hidden_state"]
        logits = self.cls(hidden)
        if labels is None:
            return {"logits": logits}
        loss = mlm_loss(logits, labels)
        return {"loss": loss, "logits": logits}


def mlm_loss(logits, labels, tp_group=None, vocab_parallel=False):
    """Mean cross entropy over the positions with ``labels != -100``.

    ``vocab_parallel``: ``logits`` hold this rank's vocabulary slice."""
    from ..ops.cross_entropy import LOCAL, vocab_parallel_cross_entropy

    per_tok = vocab_parallel_cross_entropy(logits, labels, tp_group if vocab_parallel else LOCAL)
    n_valid = (labels != -100).sum().clamp(min=1)
    return per_tok.float().sum() / n_valid


RobertaConfig = BertConfig


def roberta_config(**kw):
    kw.setdefault("vocab_size", 50265)
    kw.setdefault("pad_token_id", 1)
    kw.setdefault("position_offset", 2)
    kw.setdefault("type_vocab_size", 1)
    kw.setdefault("layer_norm_eps", 1e-5)
    return BertConfig(model_type="roberta", **kw)


class RobertaModel(BertModel):
    """RoBERTa = BERT with position ids that count the non-padding tokens (starting at
    ``pad_token_id + 1``; padding positions keep ``pad_token_id``) and a different vocabulary."""

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None):
        if position_ids is None:
            pad = self.config.pad_token_id
            keep = (input_ids != pad).to(torch.long)
            position_ids = torch.cumsum(keep, dim=1) * keep + pad
        return super().forward(input_ids, attention_mask, token_type_ids, position_ids)


class RobertaLMHead(nn.Module):
    """dense -> GeLU -> LayerNorm -> decoder (tied to the word embedding), Hugging Face names."""

    def __init__(self, config):
        super().__init__()
        self.dense = nn.Linear(config.hidden_size, config.hidden_size)
        self.layer_norm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.decoder = nn.Linear(config.hidden_size, config.vocab_size, bias=True)
        self.bias = nn.Parameter(torch.zeros(config.vocab_size))
        self.decoder.bias = self.bias       # one bias under two names, like Hugging Face
        self.act = _act("gelu")

    def forward(self, features):
        return self.decoder(self.layer_norm(self.act(self.dense(features))))


class RobertaForMaskedLM(BertPreTrainedModel):
    """RoBERTa with the masked-LM head, parameter names as in Hugging Face
    (``roberta.*``, ``lm_head.{dense,layer_norm,decoder,bias}``)."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.roberta = RobertaModel(config, add_pooling_layer=False)
        self.lm_head = RobertaLMHead(config)
        self.tie_weights()

    def tie_weights(self):
        self.lm_head.decoder.weight = self.roberta.embeddings.word_embeddings.weight

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, position_ids=None,
                labels=None):
        hidden = self.roberta(input_ids, attention_mask, token_type_ids, position_ids)[
            "last_hidden_state"]
        logits = self.lm_head(hidden)
        if labels is None:
            return {"logits": logits}
        return {"loss": mlm_loss(logits, labels), "logits": logits}
