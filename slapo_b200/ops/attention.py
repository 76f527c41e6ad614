"""Self-attention module and op that schedules swap in for a model's own
attention.

``FlashAttentionOp`` adapts ``forward(q, k, v, attention_mask, p)`` on
``[B, S, H, D]`` tensors to the tcgen05 flash-attention kernels (CUDA,
bf16/fp16) or to the PyTorch reference (everything else).  An HF-style
additive mask ``[B, 1, 1, Sk]`` is honoured on every path (the reference's
``cuda`` path silently drops it, slapo/op/attention.py:318-323); a bias per
head or per (query, key) pair runs the PyTorch reference, with a warning.

``FlashAttention`` is a complete self-attention block: fused or separate
q/k/v projections, the op, optional output projection + dropout.  The fused
QKV weight is laid out ``[head][q|k|v][head_dim]`` along its output axis so
that ``shard("weight", 0)`` gives every tensor-parallel rank whole heads.

Parity: slapo/op/attention.py:245-522 of the reference.
"""
from __future__ import annotations

import torch
from torch import nn

from . import functional as NF

_REFERENCE_NAMES = ("reference", "native_xformers", "native_flash_attn", "eager")


_GENERAL_BIAS_SEEN = set()


def _warn_general_bias(bias):
    key = tuple(bias.shape[1:3])
    if key in _GENERAL_BIAS_SEEN:
        return
    _GENERAL_BIAS_SEEN.add(key)
    import logging

    logging.getLogger("slapo_b200.ops").warning(
        "attention bias of shape %s is not a key-padding mask: this call runs the PyTorch "
        "reference with a materialised score matrix (kernels take [B, Sk] / [B, 1, 1, Sk] masks, "
        "causal=True and T5 relative-position tables)", tuple(bias.shape))


class FlashAttentionOp(nn.Module):
    traceable = False

    def __init__(self, attn_op_name="auto", apply_causal_mask=False, scale=None,
                 rel_bias_table=None, rel_bidirectional=True, rel_max_distance=128):
        super().__init__()
        self.attn_op_name = attn_op_name
        self.apply_causal_mask = apply_causal_mask
        self.scale = scale
        self.rel_bias_table = rel_bias_table  # nn.Parameter [buckets, H] owned by the caller
        self.rel_bidirectional = rel_bidirectional
        self.rel_max_distance = rel_max_distance

    def forward(self, query_layer, key_layer, value_layer, attention_mask=None, p=0.0,
                rel_bias_table=None):
        table = rel_bias_table if rel_bias_table is not None else self.rel_bias_table
        if self._is_general_bias(attention_mask):
            # a bias per head or per (query, key) pair: no kernel takes one, the PyTorch
            # reference does (the path the reference library calls "native_xformers" with a
            # tensor bias, slapo/op/attention.py:339-365)
            _warn_general_bias(attention_mask)
            if attention_mask.dtype == torch.bool:
                attention_mask = torch.zeros_like(
                    attention_mask, dtype=torch.float32).masked_fill(~attention_mask, -10000.0)
            return NF.attention_reference(
                query_layer, key_layer, value_layer, None, self.apply_causal_mask, self.scale, p,
                self.training, table, self.rel_bidirectional, self.rel_max_distance,
                attn_bias=attention_mask)
        key_bias = self._key_bias(attention_mask, key_layer.shape[0], key_layer.shape[1])
        args = (query_layer, key_layer, value_layer, key_bias, self.apply_causal_mask,
                self.scale, p, self.training, table, self.rel_bidirectional,
                self.rel_max_distance)
        if self.attn_op_name in _REFERENCE_NAMES:
            return NF.attention_reference(*args)
        return NF.flash_attention(*args)

    def _is_general_bias(self, attention_mask):
        """True for a 4-D bias that is not a key-padding mask (nor, for causal attention, the
        causal + padding mask whose last row is one)."""
        if attention_mask is None or attention_mask.dim() != 4:
            return False
        return attention_mask.shape[1] != 1 or (attention_mask.shape[2] != 1
                                                and not self.apply_causal_mask)

    def _key_bias(self, attention_mask, b, sk):
        """Additive per-key bias ``[B, Sk]`` from the mask a model passes.

        Accepted: ``[B, Sk]`` / ``[B, 1, 1, Sk]`` key-padding masks, and - for causal attention
        - the combined ``[B, 1, Sq, Sk]`` causal + padding mask that Hugging Face models build:
        its last query row is exactly the key-padding part (the triangular part is applied by
        the kernel).  Boolean masks (``True`` = attend) become ``0 / -10000``."""
        if attention_mask is None:
            return None
        if attention_mask.dim() == 4:
            if attention_mask.shape[1] != 1 or (attention_mask.shape[2] != 1
                                                and not self.apply_causal_mask):
                raise NotImplementedError(
                    "only key-padding masks [B,1,1,Sk] are supported (or [B,1,Sq,Sk] causal + "
                    "padding masks with causal=True); use causal=True for the triangular part")
            attention_mask = attention_mask[:, :, -1, :]
        if attention_mask.dtype == torch.bool:
            attention_mask = torch.zeros_like(attention_mask, dtype=torch.float32).masked_fill(
                ~attention_mask, -10000.0)
        return attention_mask.reshape(-1, sk).expand(b, sk)

    def forward_packed(self, qkv, attention_mask=None, p=0.0):
        """Attention on a packed ``[B, S, H, 3, D]`` tensor, or None when the
        packed kernel path does not apply (the caller then slices q/k/v)."""
        from .flash_attn import flash_attention_qkvpacked, packed_supported

        if self.attn_op_name in _REFERENCE_NAMES or not packed_supported(qkv) \
                or self._is_general_bias(attention_mask):
            return None
        key_bias = self._key_bias(attention_mask, qkv.shape[0], qkv.shape[1])
        return flash_attention_qkvpacked(
            qkv, key_bias, self.apply_causal_mask, self.scale, p if self.training else 0.0,
            self.rel_bias_table, self.rel_bidirectional, self.rel_max_distance)

    def extra_repr(self):
        return f"op={self.attn_op_name}, causal={self.apply_causal_mask}, scale={self.scale}"


class FlashAttention(nn.Module):
    """Self-attention block ``hidden -> (context, present)``.

    ``causal=None`` keeps the reference's convention (causal iff the block has
    an output projection, slapo/op/attention.py:428); pass it explicitly for
    anything else."""

    def __init__(self, hidden_size, num_attention_heads, attn_pdrop=0.0, resid_pdrop=0.0,
                 attn_op_name="auto", bias=True, output_proj=True, fused_qkv=False,
                 causal=None, scale=None, device=None, dtype=None):
        super().__init__()
        if hidden_size % num_attention_heads != 0:
            raise ValueError(f"hidden size {hidden_size} is not a multiple of "
                             f"{num_attention_heads} heads")
        kw = dict(device=device, dtype=dtype)
        self.num_attention_heads = num_attention_heads
        self.head_size = hidden_size // num_attention_heads
        self.all_head_size = hidden_size
        self.fused_qkv = fused_qkv
        if fused_qkv:
            self.qkv = nn.Linear(hidden_size, 3 * hidden_size, bias=bias, **kw)
        else:
            self.query = nn.Linear(hidden_size, hidden_size, bias=bias, **kw)
            self.key = nn.Linear(hidden_size, hidden_size, bias=bias, **kw)
            self.value = nn.Linear(hidden_size, hidden_size, bias=bias, **kw)
        self.output_proj = output_proj
        if output_proj:
            self.out_proj = nn.Linear(hidden_size, hidden_size, **kw)
            self.resid_dropout = nn.Dropout(resid_pdrop)
        self.attn_pdrop = attn_pdrop
        causal = output_proj if causal is None else causal
        self.attn_op = FlashAttentionOp(attn_op_name, causal, scale)

    @staticmethod
    def layout_qkv_from_separate(q, k, v, num_heads):
        """Pack separate ``[h, in]`` q/k/v weights (or ``[h]`` biases) into the
        head-interleaved fused layout."""
        parts = [t.reshape(num_heads, -1, *t.shape[1:]) for t in (q, k, v)]
        return torch.cat(parts, dim=1).reshape(-1, *q.shape[1:])

    def reshape_for_scores(self, x):
        # -1 absorbs a tensor-parallel split of the head dimension
        return x.view(x.shape[:-1] + (-1, self.head_size))

    def forward(self, hidden_states, attention_mask=None, layer_past=None, head_mask=None,
                encoder_hidden_states=None, encoder_attention_mask=None, use_cache=False,
                output_attentions=False, past_key_value=None, **_ignored):
        if encoder_hidden_states is not None:
            raise NotImplementedError("cross attention is not supported by FlashAttention")
        if head_mask is not None or output_attentions:
            raise NotImplementedError("head_mask / output_attentions are not supported")
        past = layer_past if layer_past is not None else past_key_value
        if self.fused_qkv:
            qkv = self.qkv(hidden_states)
            qkv = qkv.view(qkv.shape[:-1] + (-1, 3, self.head_size))
            if past is None and not use_cache:
                packed = self.attn_op.forward_packed(
                    qkv, attention_mask, self.attn_pdrop if self.training else 0.0)
                if packed is not None:
                    ctx = packed.reshape(packed.shape[:-2] + (-1,))
                    if self.output_proj:
                        ctx = self.resid_dropout(self.out_proj(ctx))
                    return ctx, None
            q, k, v = qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :]
        else:
            q = self.reshape_for_scores(self.query(hidden_states))
            k = self.reshape_for_scores(self.key(hidden_states))
            v = self.reshape_for_scores(self.value(hidden_states))
        if past is not None:
            k = torch.cat((past[0], k), dim=1)
            v = torch.cat((past[1], v), dim=1)
        present = (k, v) if use_cache else None
        ctx = self.attn_op(q, k, v, attention_mask, self.attn_pdrop if self.training else 0.0)
        ctx = ctx.reshape(ctx.shape[:-2] + (-1,))
        if self.output_proj:
            ctx = self.resid_dropout(self.out_proj(ctx))
        return ctx, present
