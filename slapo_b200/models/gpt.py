"""Decoder-only language models with Hugging Face parameter names:
GPT-2 (``Conv1D`` projections, fused ``c_attn``) and GPT-Neo (separate
bias-free q/k/v projections, no 1/sqrt(d) scaling).  Free of data-dependent
control flow, so every level traces with ``torch.fx``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn


class Conv1D(nn.Module):
    """GPT-2's linear layer: ``y = x @ weight + bias`` with ``weight`` stored
    ``[in_features, out_features]`` (``nf`` = out features)."""

    def __init__(self, nf, nx, device=None, dtype=None):
        super().__init__()
        self.nf = nf
        self.nx = nx
        self.weight = nn.Parameter(torch.empty(nx, nf, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(nf, device=device, dtype=dtype))
        if not self.weight.is_meta:
            nn.init.normal_(self.weight, std=0.02)

    def forward(self, x):
        from ..ops import functional as NF

        return NF.linear_t(x, self.weight, self.bias)


@dataclass
class GPTConfig:
    vocab_size: int = 50257
    n_positions: int = 1024
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    intermediate_size: int = None
    activation_function: str = "gelu_new"
    resid_dropout: float = 0.1
    embed_dropout: float = 0.1
    attention_dropout: float = 0.1
    layer_norm_epsilon: float = 1e-5
    initializer_range: float = 0.02
    model_type: str = "gpt2"

    def __post_init__(self):
        if self.intermediate_size is None:
            self.intermediate_size = 4 * self.hidden_size

    # HF aliases used by schedules written against transformers configs
    @property
    def n_embd(self):
        return self.hidden_size

    @property
    def n_head(self):
        return self.num_heads

    @property
    def n_layer(self):
        return self.num_layers

    @property
    def num_hidden_layers(self):
        return self.num_layers

    @property
    def num_attention_heads(self):
        return self.num_heads

    @property
    def max_position_embeddings(self):
        return self.n_positions

    @classmethod
    def gpt_neo_125m(cls, **kw):
        return cls(hidden_size=768, num_layers=12, num_heads=12, n_positions=2048,
                   model_type="gpt_neo", **kw)

    @classmethod
    def gpt_neo_1_3b(cls, **kw):
        return cls(hidden_size=2048, num_layers=24, num_heads=16, n_positions=2048,
                   model_type="gpt_neo", **kw)

    @classmethod
    def gpt_neo_2_7b(cls, **kw):
        return cls(hidden_size=2560, num_layers=32, num_heads=20, n_positions=2048,
                   model_type="gpt_neo", **kw)


def _act(name):
    if name in ("gelu_new", "gelu_tanh", "gelu_pytorch_tanh"):
        return nn.GELU(approximate="tanh")
    if name == "gelu":
        return nn.GELU()
    if name == "relu":
        return nn.ReLU()
    raise ValueError(f"unsupported activation {name}")


def _causal_attention(q, k, v, attention_mask, dropout, scale):
    """q, k, v: [B, H, S, D]; additive mask [B, 1, 1, S] or None."""
    s = q.size(-2)
    scores = torch.matmul(q, k.transpose(-1, -2))
    if scale is not None:
        scores = scores * scale
    causal = torch.ones(s, s, dtype=torch.bool, device=q.device).tril()
    scores = scores.masked_fill(~causal, torch.finfo(scores.dtype).min)
    if attention_mask is not None:
        scores = scores + attention_mask
    probs = dropout(F.softmax(scores, dim=-1))
    return torch.matmul(probs, v)


# ---------------------------------------------------------------------- #
class GPT2Attention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.num_heads = config.num_heads
        self.head_dim = config.hidden_size // config.num_heads
        self.c_attn = Conv1D(3 * config.hidden_size, config.hidden_size)
        self.c_proj = Conv1D(config.hidden_size, config.hidden_size)
        self.attn_dropout = nn.Dropout(config.attention_dropout)
        self.resid_dropout = nn.Dropout(config.resid_dropout)

    def _heads(self, x):
        return x.view(x.size()[:-1] + (-1, self.head_dim)).permute(0, 2, 1, 3)

    def forward(self, hidden_states, attention_mask=None):
        qkv = self.c_attn(hidden_states)
        q, k, v = qkv.chunk(3, dim=-1)
        ctx = _causal_attention(self._heads(q), self._heads(k), self._heads(v), attention_mask,
                                self.attn_dropout, self.head_dim ** -0.5)
        ctx = ctx.permute(0, 2, 1, 3).contiguous()
        ctx = ctx.view(ctx.size()[:-2] + (-1,))
        return (self.resid_dropout(self.c_proj(ctx)), None)


class GPT2MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.c_fc = Conv1D(config.intermediate_size, config.hidden_size)
        self.c_proj = Conv1D(config.hidden_size, config.intermediate_size)
        self.act = _act(config.activation_function)
        self.dropout = nn.Dropout(config.resid_dropout)

    def forward(self, hidden_states):
        return self.dropout(self.c_proj(self.act(self.c_fc(hidden_states))))


class GPT2Block(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.ln_1 = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.attn = GPT2Attention(config)
        self.ln_2 = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.mlp = GPT2MLP(config)

    def forward(self, hidden_states, attention_mask=None):
        hidden_states = hidden_states + self.attn(self.ln_1(hidden_states), attention_mask)[0]
        return hidden_states + self.mlp(self.ln_2(hidden_states))


# ---------------------------------------------------------------------- #
class GPTNeoSelfAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        h = config.hidden_size
        self.num_heads = config.num_heads
        self.head_dim = h // config.num_heads
        self.k_proj = nn.Linear(h, h, bias=False)
        self.v_proj = nn.Linear(h, h, bias=False)
        self.q_proj = nn.Linear(h, h, bias=False)
        self.out_proj = nn.Linear(h, h, bias=True)
        self.attn_dropout = nn.Dropout(config.attention_dropout)
        self.resid_dropout = nn.Dropout(config.resid_dropout)

    def _heads(self, x):
        return x.view(x.size()[:-1] + (-1, self.head_dim)).permute(0, 2, 1, 3)

    def forward(self, hidden_states, attention_mask=None):
        q = self._heads(self.q_proj(hidden_states))
        k = self._heads(self.k_proj(hidden_states))
        v = self._heads(self.v_proj(hidden_states))
        ctx = _causal_attention(q, k, v, attention_mask, self.attn_dropout, None)
        ctx = ctx.permute(0, 2, 1, 3).contiguous()
        ctx = ctx.view(ctx.size()[:-2] + (-1,))
        return (self.resid_dropout(self.out_proj(ctx)), None)


class GPTNeoAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.attention = GPTNeoSelfAttention(config)

    def forward(self, hidden_states, attention_mask=None):
        return self.attention(hidden_states, attention_mask)


class GPTNeoMLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.c_fc = nn.Linear(config.hidden_size, config.intermediate_size)
        self.c_proj = nn.Linear(config.intermediate_size, config.hidden_size)
        self.act = _act(config.activation_function)
        self.dropout = nn.Dropout(config.resid_dropout)

    def forward(self, hidden_states):
        return self.dropout(self.c_proj(self.act(self.c_fc(hidden_states))))


class GPTNeoBlock(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.ln_1 = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.attn = GPTNeoAttention(config)
        self.ln_2 = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.mlp = GPTNeoMLP(config)

    def forward(self, hidden_states, attention_mask=None):
        hidden_states = hidden_states + self.attn(self.ln_1(hidden_states), attention_mask)[0]
        return hidden_states + self.mlp(self.ln_2(hidden_states))


# ---------------------------------------------------------------------- #
class _GPTBase(nn.Module):
    def _init_weights(self, module):
        std = self.config.initializer_range
        if isinstance(module, (nn.Linear, Conv1D)):
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


class GPTTransformer(_GPTBase):
    """``transformer`` trunk shared by GPT-2 and GPT-Neo."""

    def __init__(self, config, block_cls):
        super().__init__()
        self.config = config
        self.wte = nn.Embedding(config.vocab_size, config.hidden_size)
        self.wpe = nn.Embedding(config.n_positions, config.hidden_size)
        self.drop = nn.Dropout(config.embed_dropout)
        self.h = nn.ModuleList([block_cls(config) for _ in range(config.num_layers)])
        self.ln_f = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.register_buffer("position_ids", torch.arange(config.n_positions).unsqueeze(0),
                             persistent=False)

    def forward(self, input_ids, attention_mask=None, position_ids=None):
        if position_ids is None:
            position_ids = self.position_ids.narrow(1, 0, input_ids.size(1))
        ext_mask = None
        if attention_mask is not None:
            ext_mask = (1.0 - attention_mask[:, None, None, :].to(self.ln_f.weight.dtype)) * -10000.0
        hidden = self.drop(self.wte(input_ids) + self.wpe(position_ids))
        for block in self.h:
            hidden = block(hidden, ext_mask)
        return self.ln_f(hidden)


class _GPTLMHead(_GPTBase):
    block_cls = None

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.transformer = GPTTransformer(config, self.block_cls)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.lm_head.weight = self.transformer.wte.weight

    def forward(self, input_ids, attention_mask=None, position_ids=None, labels=None):
        hidden = self.transformer(input_ids, attention_mask, position_ids)
        logits = self.lm_head(hidden)
        if labels is None:
            return {"logits": logits}
        return {"loss": causal_lm_loss(logits, labels), "logits": logits}


class GPT2LMHeadModel(_GPTLMHead):
    block_cls = GPT2Block


class GPTNeoForCausalLM(_GPTLMHead):
    block_cls = GPTNeoBlock


def causal_lm_loss(logits, labels, tp_group=None, vocab_parallel=False):
    """Next-token cross entropy: position t predicts ``labels[t + 1]``."""
    from ..ops.cross_entropy import LOCAL, vocab_parallel_cross_entropy

    shift_logits = logits[:, :-1].contiguous()
    shift_labels = labels[:, 1:].contiguous()
    per_tok = vocab_parallel_cross_entropy(shift_logits, shift_labels,
                                           tp_group if vocab_parallel else LOCAL)
    n_valid = (shift_labels != -100).sum().clamp(min=1)
    return per_tok.float().sum() / n_valid
