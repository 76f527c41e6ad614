"""Functional front ends of the fused element-wise / normalisation ops.

Every function has two implementations with identical semantics:

* CUDA tensors run the hand-written sm_100a kernels of the ``_C`` extension
  (one pass over HBM for the forward, one for the backward, dropout masks
  regenerated from a Philox ``(seed, offset)`` pair instead of being stored);
* anything else (CPU tensors, meta tensors, fx proxies) runs plain PyTorch,
  which is also the numerical oracle of the kernel tests.

A CUDA tensor with the extension missing is an error unless the environment
variable ``SLAPO_B200_ALLOW_FALLBACK=1`` is set: a silent eager fallback on a
GPU would hide a broken build.
"""
from __future__ import annotations

import math
import os

import torch
import torch.nn.functional as F

from . import native

_TANH_ACTS = ("gelu_new", "gelu_tanh", "gelu_pytorch_tanh")


def _native_ok(*tensors) -> bool:
    t = next((x for x in tensors if torch.is_tensor(x)), None)
    if t is None or not isinstance(t, torch.Tensor) or not t.is_cuda:
        return False
    if t.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        return False
    if native.available():
        return True
    if os.environ.get("SLAPO_B200_ALLOW_FALLBACK", "0") == "1":
        return False
    raise RuntimeError(
        "slapo_b200 native extension is not built/loaded but a CUDA tensor was given; "
        "run `python -c 'import __graft_entry__ as g; g.build()'` or set "
        "SLAPO_B200_ALLOW_FALLBACK=1 to accept the eager PyTorch path")


# ---------------------------------------------------------------------- #
# activations
def _act_ref(x, act):
    if act == "gelu":
        return F.gelu(x)
    if act in _TANH_ACTS:
        return F.gelu(x, approximate="tanh")
    if act == "relu":
        return F.relu(x)
    raise NotImplementedError(act)


def _act_code(act):
    return {"gelu": 0, "relu": 2}.get(act, 1)


class _BiasActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, act):
        ctx.act = act
        ctx.has_bias = bias is not None
        ctx.save_for_backward(x, bias)
        return native.ops().bias_act_fwd(x.contiguous(), bias, _act_code(act))

    @staticmethod
    def backward(ctx, grad):
        x, bias = ctx.saved_tensors
        dx, dbias = native.ops().bias_act_bwd(grad.contiguous(), x.contiguous(), bias,
                                              _act_code(ctx.act))
        return dx, (dbias if ctx.has_bias else None), None


def bias_act(x, bias, act: str = "gelu"):
    """``act(x + bias)``; act in gelu (erf) / gelu_new (tanh) / relu."""
    if _native_ok(x) and x.shape[-1] % 8 == 0:
        return _BiasActFn.apply(x, bias, act)
    return _act_ref(x + bias if bias is not None else x, act)


def bias_gelu(x, bias, approximate: str = "none"):
    return bias_act(x, bias, "gelu" if approximate == "none" else "gelu_new")


# ---------------------------------------------------------------------- #
# linear layers on the tcgen05 GEMM
def gemm_supported(x, weight) -> bool:
    """CUDA 16-bit operands whose dimensions TMA can address (multiples of 8 elements)."""
    if not (torch.is_tensor(x) and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16)):
        return False
    if weight.dtype != x.dtype or weight.dim() != 2 or weight.stride(1) != 1:
        return False
    if os.environ.get("SLAPO_B200_LIBRARY_GEMM", "0") == "1":   # A/B switch for measurements
        return False
    return (x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0 and weight.stride(0) % 8 == 0
            and x.numel() > 0 and _native_ok(x))


def _rows(t):
    """``t`` as a 2-D matrix with contiguous rows whose stride TMA accepts."""
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(1) != 1 or t2.stride(0) % 8 or t2.data_ptr() % 16:
        t2 = t2.contiguous()
    return t2


def gemm(a, b, bias=None, act=-1, a_mn=False, b_mn=False, out=None, pre_act=None, split_k=False):
    """``act(A B^T + bias)`` on this library's tcgen05 kernels (CTA pairs where the problem
    has a pair tile).  ``a_mn`` / ``b_mn``: the operand is stored ``[K, M]`` / ``[K, N]``."""
    return native.ops().gemm_out(a, b, bias, act, a_mn, b_mn, out, pre_act, 0, split_k)


_RELU = 2


class _LinearFn(torch.autograd.Function):
    """``y = x W^T + b`` (optionally ``relu`` of it): three GEMMs of this library, none of them
    transposing an operand in memory.  The bias rides in the forward GEMM's epilogue and so
    does ReLU, whose derivative the backward reads off the output (``y > 0``).  GeLU is NOT
    fused: the four epilogue warps of a tcgen05 GEMM have a fraction of the SM's FP32 issue
    rate, and an erf per element made the GEMM 2.5 x slower than running
    :func:`bias_act` over the output afterwards."""

    @staticmethod
    def forward(ctx, x, weight, bias, act):
        x2 = _rows(x)
        y = gemm(x2, weight, bias, act)
        ctx.act, ctx.has_bias = act, bias is not None
        ctx.save_for_backward(x2, weight, y if act >= 0 else None)
        ctx.x_shape = x.shape
        return y.view(tuple(x.shape[:-1]) + (weight.shape[0],))

    @staticmethod
    def backward(ctx, dy):
        x2, weight, y = ctx.saved_tensors
        dy2 = _rows(dy)
        dbias = None
        if ctx.act >= 0:
            # relu'(z) = (y > 0): the saved output stands in for the pre-activation
            dy2, dbias = native.ops().act_bwd_colsum(dy2.contiguous(), y, ctx.act)
        elif ctx.has_bias and ctx.needs_input_grad[2]:
            dbias = native.ops().colsum(dy2)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dX = dZ W:  B = W [N, K] read N-major (its rows are the contraction)
            dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            # dW = dZ^T X:  A = dZ [T, N] read M-major, B = X [T, K] read N-major; few tiles and a
            # long contraction, hence split-K
            dw = gemm(dy2, x2, a_mn=True, b_mn=True, split_k=True)
        return dx, dw, (dbias if ctx.has_bias else None), None


class _LinearTFn(torch.autograd.Function):
    """``y = x W + b`` with ``W`` stored ``[in, out]`` (GPT-2's ``Conv1D``): the same three
    GEMMs with the operand roles read the other way round, again without a transpose in memory."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = _rows(x)
        y = gemm(x2, weight, bias, b_mn=True)            # B = W [K, N] read N-major
        ctx.has_bias = bias is not None
        ctx.save_for_backward(x2, weight)
        ctx.x_shape = x.shape
        return y.view(tuple(x.shape[:-1]) + (weight.shape[1],))

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = _rows(dy)
        dbias = native.ops().colsum(dy2) if ctx.has_bias and ctx.needs_input_grad[2] else None
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight).view(ctx.x_shape)      # dX = dY W^T: B = W [in, out] K-major
        if ctx.needs_input_grad[1]:
            dw = gemm(x2, dy2, a_mn=True, b_mn=True, split_k=True)    # dW = X^T dY
        return dx, dw, dbias


def linear_t(x, weight, bias=None):
    """``x @ weight + bias`` for a weight stored ``[in_features, out_features]``."""
    if (torch.is_tensor(x) and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16)
            and weight.dtype == x.dtype and weight.dim() == 2 and weight.stride(1) == 1
            and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0 and weight.stride(0) % 8 == 0
            and x.numel() > 0 and os.environ.get("SLAPO_B200_LIBRARY_GEMM", "0") != "1"
            and _native_ok(x)):
        return _LinearTFn.apply(x, weight, bias)
    out = torch.matmul(x, weight)
    return out if bias is None else out + bias


def linear(x, weight, bias=None, act=None):
    """``act(x @ weight.T + bias)``; ``act`` in None / "gelu" / "gelu_new" / "relu".  CUDA
    16-bit tensors run this library's GEMM (bias and activation in its epilogue), anything
    else PyTorch."""
    if gemm_supported(x, weight):
        if act is None or act == "relu":
            return _LinearFn.apply(x, weight, bias, -1 if act is None else _RELU)
        return bias_act(_LinearFn.apply(x, weight, None, -1), bias, act)
    out = F.linear(x, weight, bias)
    return out if act is None else _act_ref(out, act)


# ---------------------------------------------------------------------- #
# dropout family
def effective_dropout_p(p: float) -> float:
    """Dropout probability the CUDA kernels actually apply.  They draw 7-bit
    random numbers (16 decisions per Philox call), so ``p`` is rounded to a
    multiple of 1/128 (0.1 -> 13/128 = 0.1016); kept values are rescaled by
    ``1 / (1 - effective p)``, which keeps the expectation exact."""
    return min(max(int(p * 128.0 + 0.5), 0), 127) / 128.0


def _philox_reserve(numel):
    """Reserve Philox offsets on the current CUDA generator (so masks follow
    torch's RNG state: manual_seed, fork_rng, checkpoint replay).  Returns the
    opaque CPU int64[4] state the kernels take; valid under graph capture."""
    return native.ops().philox_reserve(int(numel))


class _BiasDropoutAddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, residual, p):
        rng = _philox_reserve(x.numel())
        ctx.p, ctx.rng = p, rng
        ctx.has_bias, ctx.has_res = bias is not None, residual is not None
        return native.ops().bias_dropout_add_fwd(
            x.contiguous(), bias, residual.contiguous() if residual is not None else None,
            p, rng)

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous()
        dx, dbias = native.ops().bias_dropout_add_bwd(grad, ctx.p, ctx.rng, ctx.has_bias)
        return dx, (dbias if ctx.has_bias else None), (grad if ctx.has_res else None), None


def bias_dropout_add(x, bias, residual, p: float, training: bool = True):
    """``dropout(x + bias, p) + residual`` (bias / residual may be None)."""
    if _native_ok(x) and training and p > 0.0 and x.shape[-1] % 8 == 0:
        return _BiasDropoutAddFn.apply(x, bias, residual, p)
    out = x + bias if bias is not None else x
    out = F.dropout(out, p, training)
    return out + residual if residual is not None else out


def bias_dropout(x, bias, p: float, training: bool = True):
    return bias_dropout_add(x, bias, None, p, training)


# ---------------------------------------------------------------------- #
# normalisation
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms):
        shape = x.shape
        x2 = x.contiguous().view(-1, shape[-1])
        y, mean, rstd = native.ops().layer_norm_fwd(x2, weight, bias, eps, rms)
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.rms, ctx.has_bias, ctx.shape = rms, bias is not None, shape
        return y.view(shape)

    @staticmethod
    def backward(ctx, grad):
        x2, weight, mean, rstd = ctx.saved_tensors
        g2 = grad.contiguous().view(-1, ctx.shape[-1])
        dx, dw, db = native.ops().layer_norm_bwd(g2, x2, weight, mean, rstd, ctx.rms)
        return dx.view(ctx.shape), dw, (db if ctx.has_bias else None), None, None


def layer_norm(x, weight, bias, eps: float = 1e-5):
    if _native_ok(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        return _LayerNormFn.apply(x, weight, bias, eps, False)
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


def rms_norm(x, weight, eps: float = 1e-6):
    """T5-style RMS norm: no mean subtraction, no bias, fp32 statistics."""
    if _native_ok(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        return _LayerNormFn.apply(x, weight, None, eps, True)
    var = x.float().pow(2).mean(-1, keepdim=True)
    return (x.float() * torch.rsqrt(var + eps)).to(x.dtype) * weight


class _DropoutAddLayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, residual, weight, ln_bias, p, eps, training):
        shape = x.shape
        cols = shape[-1]
        x2 = x.contiguous().view(-1, cols)
        r2 = residual.contiguous().view(-1, cols)
        p_eff = p if training else 0.0
        rng = _philox_reserve(x.numel()) if p_eff > 0 else None
        y, z, mean, rstd = native.ops().dropout_add_ln_fwd(
            x2, bias, r2, weight, ln_bias, p_eff, eps, rng)
        ctx.save_for_backward(z, weight, mean, rstd)
        ctx.p, ctx.rng = p_eff, rng
        ctx.has_bias, ctx.shape = bias is not None, shape
        return y.view(shape), z.view(shape)

    @staticmethod
    def backward(ctx, gy, gz):
        z, weight, mean, rstd = ctx.saved_tensors
        cols = ctx.shape[-1]
        gy2 = gy.contiguous().view(-1, cols)
        gz2 = gz.contiguous().view(-1, cols) if gz is not None else None
        dx, dres, dw, db, dbias = native.ops().dropout_add_ln_bwd(
            gy2, gz2, z, weight, mean, rstd, ctx.p, ctx.rng, ctx.has_bias)
        return (dx.view(ctx.shape), (dbias if ctx.has_bias else None), dres.view(ctx.shape),
                dw, db, None, None, None)


def dropout_add_layer_norm(x, bias, residual, weight, ln_bias, p: float, eps: float,
                           training: bool = True):
    """``z = dropout(x + bias) + residual; y = LayerNorm(z)``; returns ``(y, z)``.

    ``z`` is returned because a pre-LN block needs it as the next residual; a
    post-LN block (BERT) just drops it."""
    if _native_ok(x) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        return _DropoutAddLayerNormFn.apply(x, bias, residual, weight, ln_bias, p, eps, training)
    z = x + bias if bias is not None else x
    z = F.dropout(z, p, training) + residual
    return F.layer_norm(z, (z.shape[-1],), weight, ln_bias, eps), z


# ---------------------------------------------------------------------- #
# attention
def t5_relative_position_bucket(relative_position, bidirectional=True, num_buckets=32,
                                max_distance=128):
    """T5 bucket index of ``relative_position = key_pos - query_pos``."""
    ret = torch.zeros_like(relative_position)
    n = num_buckets
    if bidirectional:
        n //= 2
        ret = ret + (relative_position > 0).to(torch.long) * n
        rp = relative_position.abs()
    else:
        rp = -torch.min(relative_position, torch.zeros_like(relative_position))
    max_exact = n // 2
    is_small = rp < max_exact
    large = max_exact + (
        torch.log(rp.float().clamp(min=1) / max_exact) / math.log(max_distance / max_exact)
        * (n - max_exact)).to(torch.long)
    large = torch.min(large, torch.full_like(large, n - 1))
    return ret + torch.where(is_small, rp, large)


def attention_reference(q, k, v, key_padding_bias=None, causal=False, scale=None,
                        dropout_p=0.0, training=False, rel_bias_table=None,
                        rel_bidirectional=True, rel_max_distance=128, dropout_mask=None,
                        attn_bias=None):
    """Plain-PyTorch attention on ``[B, S, H, D]`` tensors (the oracle).

    ``key_padding_bias`` is an additive ``[B, Sk]`` bias (0 / large negative);
    ``rel_bias_table`` a ``[num_buckets, H]`` T5 relative-position table; ``attn_bias`` any
    additive bias that broadcasts to ``[B, H, Sq, Sk]`` (only this function takes one)."""
    b, sq, h, d = q.shape
    sk = k.shape[1]
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    qf, kf, vf = (t.transpose(1, 2).float() for t in (q, k, v))
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if rel_bias_table is not None:
        ctx_pos = torch.arange(sq, device=q.device)[:, None] + (sk - sq)
        mem_pos = torch.arange(sk, device=q.device)[None, :]
        buckets = t5_relative_position_bucket(
            mem_pos - ctx_pos, rel_bidirectional, rel_bias_table.shape[0], rel_max_distance)
        scores = scores + rel_bias_table.float()[buckets].permute(2, 0, 1)[None]
    if key_padding_bias is not None:
        scores = scores + key_padding_bias.float().view(b, 1, 1, sk)
    if attn_bias is not None:
        scores = scores + attn_bias.float()
    if causal:
        keep = torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril(diagonal=sk - sq)
        scores = scores.masked_fill(~keep, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    if dropout_mask is not None:
        probs = probs * dropout_mask / (1.0 - dropout_p)
    elif dropout_p > 0.0 and training:
        probs = F.dropout(probs, dropout_p, True)
    out = torch.matmul(probs, vf)
    return out.transpose(1, 2).to(q.dtype)


_FALLBACK_SEEN = set()


def _warn_attention_fallback(q, k):
    """One WARNING per (dtype, head dim, layout problem): a CUDA attention call that the
    tcgen05 kernels do not take runs the fp32 reference with a materialised [B, H, Sq, Sk]
    score matrix - correct, but many times slower and memory-hungry."""
    why = []
    if q.dtype not in (torch.bfloat16, torch.float16):
        why.append(f"dtype {q.dtype} (kernels: bf16 / fp16)")
    d = q.shape[-1]
    if not (8 <= d <= 128 and d % 8 == 0):
        why.append(f"head dim {d} (kernels: multiples of 8 up to 128)")
    if q.dim() != 4:
        why.append(f"{q.dim()}-D input (kernels: [B, S, H, D])")
    if not why:
        why.append("strides or alignment (D contiguous, other strides multiples of 8 "
                   "elements, 16-byte aligned data)")
    key = (q.dtype, d, tuple(why))
    if key in _FALLBACK_SEEN:
        return
    _FALLBACK_SEEN.add(key)
    import logging

    logging.getLogger("slapo_b200.ops").warning(
        "flash_attention falls back to the PyTorch reference for q %s / k %s: %s",
        tuple(q.shape), tuple(k.shape), "; ".join(why))


def flash_attention(q, k, v, key_padding_bias=None, causal=False, scale=None, dropout_p=0.0,
                    training=True, rel_bias_table=None, rel_bidirectional=True,
                    rel_max_distance=128):
    """Attention on ``[B, S, H, D]`` tensors (any strides on B/S/H, D
    contiguous).  CUDA bf16/fp16 inputs run the tcgen05 flash kernels."""
    from .flash_attn import flash_attention_native, native_supported

    if torch.is_tensor(q) and q.is_cuda and native_supported(q, k, v):
        _native_ok(q)
        return flash_attention_native(q, k, v, key_padding_bias, causal, scale,
                                      dropout_p if training else 0.0, rel_bias_table,
                                      rel_bidirectional, rel_max_distance)
    if torch.is_tensor(q) and q.is_cuda:
        _warn_attention_fallback(q, k)
    return attention_reference(q, k, v, key_padding_bias, causal, scale, dropout_p, training,
                               rel_bias_table, rel_bidirectional, rel_max_distance)
