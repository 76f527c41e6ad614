"""ALBERT: a BERT-shaped encoder whose transformer layer is shared by all
depths and whose embeddings are factorised (``embedding_size`` < hidden).
Hugging Face parameter names (``albert.encoder.albert_layer_groups.0.
albert_layers.0.attention.query`` ...)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from .bert import _act, mlm_loss  # noqa: F401


@dataclass
class AlbertConfig:
    vocab_size: int = 30000
    embedding_size: int = 128
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_hidden_groups: int = 1
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    inner_group_num: int = 1
    hidden_act: str = "gelu_new"
    hidden_dropout_prob: float = 0.0
    attention_probs_dropout_prob: float = 0.0
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-12
    pad_token_id: int = 0
    model_type: str = "albert"


class AlbertEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        e = config.embedding_size
        self.word_embeddings = nn.Embedding(config.vocab_size, e, padding_idx=config.pad_token_id)
        self.position_embeddings = nn.Embedding(config.max_position_embeddings, e)
        self.token_type_embeddings = nn.Embedding(config.type_vocab_size, e)
        self.LayerNorm = nn.LayerNorm(e, eps=config.layer_norm_eps)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)
        self.register_buffer("position_ids",
                             torch.arange(config.max_position_embeddings).unsqueeze(0),
                             persistent=False)

    def forward(self, input_ids, token_type_ids=None):
        pos = self.position_ids.narrow(1, 0, input_ids.size(1))
        emb = self.word_embeddings(input_ids) + self.position_embeddings(pos)
        emb = emb + (self.token_type_embeddings.weight[0] if token_type_ids is None
                     else self.token_type_embeddings(token_type_ids))
        return self.dropout(self.LayerNorm(emb))


class AlbertAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        h = config.hidden_size
        self.num_attention_heads = config.num_attention_heads
        self.attention_head_size = h // config.num_attention_heads
        self.query = nn.Linear(h, h)
        self.key = nn.Linear(h, h)
        self.value = nn.Linear(h, h)
        self.attention_dropout = nn.Dropout(config.attention_probs_dropout_prob)
        self.output_dropout = nn.Dropout(config.hidden_dropout_prob)
        self.dense = nn.Linear(h, h)
        self.LayerNorm = nn.LayerNorm(h, eps=config.layer_norm_eps)

    def _heads(self, x):
        return x.view(x.size()[:-1] + (-1, self.attention_head_size)).permute(0, 2, 1, 3)

    def forward(self, hidden_states, attention_mask=None):
        q, k, v = (self._heads(m(hidden_states)) for m in (self.query, self.key, self.value))
        scores = torch.matmul(q, k.transpose(-1, -2)) / (self.attention_head_size ** 0.5)
        if attention_mask is not None:
            scores = scores + attention_mask
        probs = self.attention_dropout(F.softmax(scores, dim=-1))
        ctx = torch.matmul(probs, v).permute(0, 2, 1, 3).contiguous()
        ctx = ctx.view(ctx.size()[:-2] + (-1,))
        return self.LayerNorm(hidden_states + self.output_dropout(self.dense(ctx)))


class AlbertLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.attention = AlbertAttention(config)
        self.ffn = nn.Linear(config.hidden_size, config.intermediate_size)
        self.ffn_output = nn.Linear(config.intermediate_size, config.hidden_size)
        self.activation = _act(config.hidden_act)
        self.full_layer_layer_norm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)

    def forward(self, hidden_states, attention_mask=None):
        attn = self.attention(hidden_states, attention_mask)
        ffn = self.dropout(self.ffn_output(self.activation(self.ffn(attn))))
        return self.full_layer_layer_norm(ffn + attn)


class AlbertLayerGroup(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.albert_layers = nn.ModuleList([AlbertLayer(config)
                                            for _ in range(config.inner_group_num)])

    def forward(self, hidden_states, attention_mask=None):
        for layer in self.albert_layers:
            hidden_states = layer(hidden_states, attention_mask)
        return hidden_states


class AlbertTransformer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.num_hidden_layers = config.num_hidden_layers
        self.num_hidden_groups = config.num_hidden_groups
        self.embedding_hidden_mapping_in = nn.Linear(config.embedding_size, config.hidden_size)
        self.albert_layer_groups = nn.ModuleList([AlbertLayerGroup(config)
                                                  for _ in range(config.num_hidden_groups)])

    def forward(self, hidden_states, attention_mask=None):
        hidden_states = self.embedding_hidden_mapping_in(hidden_states)
        per_group = self.num_hidden_layers // self.num_hidden_groups
        for i in range(self.num_hidden_layers):
            hidden_states = self.albert_layer_groups[i // per_group](hidden_states, attention_mask)
        return hidden_states


class AlbertModel(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.embeddings = AlbertEmbeddings(config)
        self.encoder = AlbertTransformer(config)

    def forward(self, input_ids, attention_mask=None, token_type_ids=None):
        ext = None
        if attention_mask is not None:
            ext = (1.0 - attention_mask[:, None, None, :].to(
                self.embeddings.LayerNorm.weight.dtype)) * -10000.0
        return self.encoder(self.embeddings(input_ids, token_type_ids), ext)


class AlbertMLMHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.LayerNorm = nn.LayerNorm(config.embedding_size, eps=config.layer_norm_eps)
        self.bias = nn.Parameter(torch.zeros(config.vocab_size))
        self.dense = nn.Linear(config.hidden_size, config.embedding_size)
        self.decoder = nn.Linear(config.embedding_size, config.vocab_size)
        self.activation = _act(config.hidden_act)
        self.decoder.bias = self.bias

    def forward(self, hidden_states):
        return self.decoder(self.LayerNorm(self.activation(self.dense(hidden_states))))


class AlbertForMaskedLM(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.albert = AlbertModel(config)
        self.predictions = AlbertMLMHead(config)
        self.predictions.decoder.weight = self.albert.embeddings.word_embeddings.weight

    def _init_weights(self, module):
        std = self.config.initializer_range
        if isinstance(module, nn.Linear):
            module.weight.data.normal_(mean=0.0, std=std)
            if module.bias is not None:
                module.bias.data.zero_()
        elif isinstance(module, nn.Embedding):
            module.weight.data.normal_(mean=0.0, std=std)
        elif isinstance(module, nn.LayerNorm):
            module.bias.data.zero_()
            module.weight.data.fill_(1.0)

    def init_weights(self):
        self.apply(self._init_weights)
        return self

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, labels=None):
        logits = self.predictions(self.albert(input_ids, attention_mask, token_type_ids))
        if labels is None:
            return {"logits": logits}
        return {"loss": mlm_loss(logits, labels), "logits": logits}
