"""Python binding of the tcgen05 flash-attention kernels.

``flash_attention_native`` is differentiable in q, k, v and in the T5
relative-position table.  The table ``[num_buckets, H]`` is expanded with
plain (differentiable) torch indexing into a per-distance bias ``[H, Sq + Sk -
1]`` - entry ``(key - query) + Sq - 1`` - which the kernels add in-line, so the
``[H, Sq, Sk]`` bias matrix is never materialised and the table gradient flows
back through that small gather.
"""
from __future__ import annotations

import math

import torch

from . import native

def head_dim_supported(d: int) -> bool:
    """Head dimensions the kernels take: multiples of 8 up to 128 (OPT-2.7B's 80 included);
    tiles are 64 or 128 wide and TMA zero-fills the columns beyond ``d``."""
    return 8 <= d <= 128 and d % 8 == 0


def native_supported(q, k, v) -> bool:
    if not (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16)):
        return False
    if q.dim() != 4 or not head_dim_supported(q.shape[-1]):
        return False
    for t in (q, k, v):
        if t.stride(-1) != 1 or any(s % 8 for s in t.stride()[:3]) or t.data_ptr() % 16:
            return False
    return native.available()


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, key_bias, rel, causal, scale, p):
        rng = native.ops().philox_reserve(q.shape[0] * q.shape[2] * q.shape[1] * k.shape[1]) \
            if p > 0 else None
        out, lse = native.ops().flash_attn_fwd(q, k, v, key_bias, rel, causal, scale, p, rng)
        ctx.save_for_backward(q, k, v, out, lse, key_bias, rel)
        ctx.cfg = (causal, scale, p, rng)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, key_bias, rel = ctx.saved_tensors
        causal, scale, p, rng = ctx.cfg
        dq, dk, dv, drel = native.ops().flash_attn_bwd(
            dout.contiguous(), q, k, v, out, lse, key_bias, rel, causal, scale, p, rng, False)
        return dq, dk, dv, None, (drel if rel is not None else None), None, None, None


class _FlashAttnPackedFn(torch.autograd.Function):
    """Same kernels on a packed projection output ``[B, S, H, 3, D]``: q, k, v
    are read in place through strided views and the three gradients are
    written into one tensor of the packed layout (no slicing copies, no
    concatenation in autograd)."""

    @staticmethod
    def forward(ctx, qkv, key_bias, rel, causal, scale, p):
        q, k, v = qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :]
        rng = native.ops().philox_reserve(q.shape[0] * q.shape[2] * q.shape[1] * k.shape[1]) \
            if p > 0 else None
        out, lse = native.ops().flash_attn_fwd(q, k, v, key_bias, rel, causal, scale, p, rng)
        ctx.save_for_backward(qkv, out, lse, key_bias, rel)
        ctx.cfg = (causal, scale, p, rng)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, key_bias, rel = ctx.saved_tensors
        causal, scale, p, rng = ctx.cfg
        q, k, v = qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :]
        dqkv, _, _, drel = native.ops().flash_attn_bwd(
            dout.contiguous(), q, k, v, out, lse, key_bias, rel, causal, scale, p, rng, True)
        return dqkv, None, (drel if rel is not None else None), None, None, None


def relative_bias_by_distance(table, sq, sk, bidirectional, max_distance):
    """``[num_buckets, H]`` table -> ``[H, sq + sk - 1]`` bias per (key - query)."""
    from .functional import t5_relative_position_bucket

    # query i sits at absolute position i + (sk - sq); distance = key - that
    dist = torch.arange(-(sq - 1), sk, device=table.device) - (sk - sq)
    buckets = t5_relative_position_bucket(dist, bidirectional, table.shape[0], max_distance)
    return table.float()[buckets].t().contiguous()


def flash_attention_native(q, k, v, key_bias, causal, scale, p, rel_table, rel_bidir, rel_maxd):
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if key_bias is not None:
        key_bias = key_bias.float().contiguous()
    rel = None
    if rel_table is not None:
        rel = relative_bias_by_distance(rel_table, q.shape[1], k.shape[1], rel_bidir, rel_maxd)
    return _FlashAttnFn.apply(q, k, v, key_bias, rel, bool(causal), float(scale), float(p))


def flash_attention_qkvpacked(qkv, key_bias=None, causal=False, scale=None, p=0.0,
                              rel_table=None, rel_bidir=True, rel_maxd=128):
    """Attention on a packed ``[B, S, H, 3, D]`` projection output."""
    scale = 1.0 / math.sqrt(qkv.shape[-1]) if scale is None else scale
    if key_bias is not None:
        key_bias = key_bias.float().contiguous()
    rel = None
    if rel_table is not None:
        rel = relative_bias_by_distance(rel_table, qkv.shape[1], qkv.shape[1], rel_bidir, rel_maxd)
    return _FlashAttnPackedFn.apply(qkv, key_bias, rel, bool(causal), float(scale), float(p))


def packed_supported(qkv) -> bool:
    return (torch.is_tensor(qkv) and qkv.is_cuda and qkv.dim() == 5 and qkv.shape[3] == 3
            and qkv.is_contiguous() and qkv.dtype in (torch.bfloat16, torch.float16)
            and head_dim_supported(qkv.shape[-1]) and native.available())


def effective_dropout_p(p: float) -> float:
    """See :func:`slapo_b200.ops.functional.effective_dropout_p`."""
    from .functional import effective_dropout_p as impl

    return impl(p)


def dropout_keep_mask(b, h, sq, sk, p):
    """The keep mask the next flash-attention call with dropout ``p`` would
    draw, WITHOUT advancing the generator (testing aid)."""
    gen = torch.cuda.default_generators[torch.cuda.current_device()]
    state = gen.get_state()
    rng = native.ops().philox_reserve(b * h * sq * sk)
    mask = native.ops().flash_attn_dropout_mask(b, h, sq, sk, p, rng)
    gen.set_state(state)
    return mask.bool()
