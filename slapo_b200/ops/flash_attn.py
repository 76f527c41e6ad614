"""Python binding of the tcgen05 flash-attention kernels."""
from __future__ import annotations

import math

import torch

from . import native

_HEAD_DIMS = (64, 128)


def native_supported(q, k, v) -> bool:
    if not (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16)):
        return False
    if q.shape[-1] not in _HEAD_DIMS or q.stride(-1) != 1 or k.stride(-1) != 1 or v.stride(-1) != 1:
        return False
    return native.available() and hasattr(torch.ops.slapo_b200, "flash_attn_fwd")


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, key_bias, causal, scale, p, rel_table, rel_bidir, rel_maxd):
        from .functional import _philox_reserve

        b, sq, h, d = q.shape
        rng = _philox_reserve(b * h * sq * k.shape[1]) if p > 0 else None
        out, lse = native.ops().flash_attn_fwd(
            q, k, v, key_bias, rel_table, causal, scale, p, rng, rel_bidir, rel_maxd)
        ctx.save_for_backward(q, k, v, out, lse, key_bias, rel_table)
        ctx.cfg = (causal, scale, p, rng, rel_bidir, rel_maxd)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, key_bias, rel_table = ctx.saved_tensors
        causal, scale, p, rng, rel_bidir, rel_maxd = ctx.cfg
        dq, dk, dv, dtable = native.ops().flash_attn_bwd(
            dout.contiguous(), q, k, v, out, lse, key_bias, rel_table, causal, scale, p, rng,
            rel_bidir, rel_maxd)
        return dq, dk, dv, None, None, None, None, (dtable if rel_table is not None else None), None, None


def flash_attention_native(q, k, v, key_bias, causal, scale, p, rel_table, rel_bidir, rel_maxd):
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if key_bias is not None:
        key_bias = key_bias.float().contiguous()
    if rel_table is not None:
        rel_table = rel_table.float()
    return _FlashAttnFn.apply(q, k, v, key_bias, causal, scale, p, rel_table, rel_bidir, rel_maxd)
