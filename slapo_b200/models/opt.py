"""OPT decoder-only language model with Hugging Face parameter names
(``model.decoder.layers.N.self_attn.q_proj`` ...): pre-LayerNorm blocks, ReLU
FFN, learned positions with the usual offset of 2."""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from .gpt import _GPTBase, _act, _causal_attention, causal_lm_loss  # noqa: F401


@dataclass
class OPTConfig:
    vocab_size: int = 50272
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    ffn_dim: int = 3072
    max_position_embeddings: int = 2048
    activation_function: str = "relu"
    dropout: float = 0.1
    attention_dropout: float = 0.0
    do_layer_norm_before: bool = True
    initializer_range: float = 0.02
    layer_norm_epsilon: float = 1e-5
    pad_token_id: int = 1
    model_type: str = "opt"

    @property
    def init_std(self):
        return self.initializer_range

    @classmethod
    def opt_2_7b(cls, **kw):
        return cls(hidden_size=2560, num_hidden_layers=32, num_attention_heads=32, ffn_dim=10240,
                   **kw)

    @classmethod
    def opt_350m(cls, **kw):
        return cls(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, ffn_dim=4096,
                   **kw)


class OPTLearnedPositionalEmbedding(nn.Embedding):
    def __init__(self, num_embeddings, embedding_dim):
        self.offset = 2
        super().__init__(num_embeddings + self.offset, embedding_dim)

    def forward(self, position_ids):
        return super().forward(position_ids + self.offset)


class OPTAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        h = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = h // self.num_heads
        self.k_proj = nn.Linear(h, h)
        self.v_proj = nn.Linear(h, h)
        self.q_proj = nn.Linear(h, h)
        self.out_proj = nn.Linear(h, h)
        self.attn_dropout = nn.Dropout(config.attention_dropout)

    def _heads(self, x):
        return x.view(x.size()[:-1] + (-1, self.head_dim)).permute(0, 2, 1, 3)

    def forward(self, hidden_states, attention_mask=None):
        q = self._heads(self.q_proj(hidden_states))
        k = self._heads(self.k_proj(hidden_states))
        v = self._heads(self.v_proj(hidden_states))
        ctx = _causal_attention(q, k, v, attention_mask, self.attn_dropout, self.head_dim ** -0.5)
        ctx = ctx.permute(0, 2, 1, 3).contiguous()
        ctx = ctx.view(ctx.size()[:-2] + (-1,))
        return (self.out_proj(ctx), None)


class OPTDecoderLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        h = config.hidden_size
        self.self_attn = OPTAttention(config)
        self.self_attn_layer_norm = nn.LayerNorm(h, eps=config.layer_norm_epsilon)
        self.fc1 = nn.Linear(h, config.ffn_dim)
        self.fc2 = nn.Linear(config.ffn_dim, h)
        self.activation_fn = _act(config.activation_function)
        self.final_layer_norm = nn.LayerNorm(h, eps=config.layer_norm_epsilon)
        self.dropout = nn.Dropout(config.dropout)

    def forward(self, hidden_states, attention_mask=None):
        residual = hidden_states
        hidden_states = self.self_attn(self.self_attn_layer_norm(hidden_states), attention_mask)[0]
        hidden_states = residual + self.dropout(hidden_states)
        residual = hidden_states
        hidden_states = self.fc2(self.activation_fn(self.fc1(self.final_layer_norm(hidden_states))))
        return residual + self.dropout(hidden_states)


class OPTDecoder(_GPTBase):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.embed_positions = OPTLearnedPositionalEmbedding(config.max_position_embeddings,
                                                             config.hidden_size)
        self.layers = nn.ModuleList([OPTDecoderLayer(config)
                                     for _ in range(config.num_hidden_layers)])
        self.final_layer_norm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.register_buffer("position_ids",
                             torch.arange(config.max_position_embeddings).unsqueeze(0),
                             persistent=False)

    def forward(self, input_ids, attention_mask=None):
        positions = self.position_ids.narrow(1, 0, input_ids.size(1))
        ext_mask = None
        if attention_mask is not None:
            ext_mask = (1.0 - attention_mask[:, None, None, :].to(
                self.final_layer_norm.weight.dtype)) * -10000.0
        hidden = self.embed_tokens(input_ids) + self.embed_positions(positions)
        for layer in self.layers:
            hidden = layer(hidden, ext_mask)
        return self.final_layer_norm(hidden)


class OPTModel(_GPTBase):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.decoder = OPTDecoder(config)

    def forward(self, input_ids, attention_mask=None):
        return self.decoder(input_ids, attention_mask)


class OPTForCausalLM(_GPTBase):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.model = OPTModel(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.lm_head.weight = self.model.decoder.embed_tokens.weight

    def forward(self, input_ids, attention_mask=None, labels=None):
        logits = self.lm_head(self.model(input_ids, attention_mask))
        if labels is None:
            return {"logits": logits}
        return {"loss": causal_lm_loss(logits, labels), "logits": logits}
