"""Linear-layer variants that schedules swap in.

* ``LinearWithSeparateBias`` - matmul then an explicit ``+ bias`` (what
  ``decompose`` produces).
* ``LinearWithSyncFunc`` - matmul -> collective -> ``+ bias`` for
  row-parallel layers whose output is a partial sum.
* ``LinearWithAct`` - matmul -> collective -> fused bias + activation.
* ``LinearWithDropout`` - matmul -> collective -> fused bias + dropout.
* ``FusedQKV`` - one projection producing q, k, v for the local heads.

On CUDA the bias/activation/dropout tails run as single sm_100a kernels (see
:mod:`slapo_b200.ops.functional`); on CPU they are plain PyTorch.

Parity: slapo/op/linear.py:20-264 of the reference.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from . import functional as NF


class Linear(nn.Linear):
    """``nn.Linear`` whose products run on this library's tcgen05 GEMM (forward, input
    gradient and weight gradient) when the tensors are CUDA 16-bit; same parameters, same
    state dict, same behaviour elsewhere."""

    def forward(self, x):
        return NF.linear(x, self.weight, self.bias)


def adopt_native_linears(model: nn.Module) -> int:
    """Give every plain ``nn.Linear`` below ``model`` the forward of :class:`Linear`.

    The module objects stay what they are - parameters, hooks, schedule-tree references and
    ``isinstance(m, nn.Linear)`` all survive - only their class changes.  The native dialect
    calls this when it builds an engine on CUDA, so that no contraction of the step is left to
    a library GEMM.  Returns the number of modules changed."""
    n = 0
    for mod in model.modules():
        if type(mod) is nn.Linear:
            mod.__class__ = Linear
            n += 1
    return n


class LinearWithSeparateBias(nn.Linear):
    def forward(self, x):
        out = NF.linear(x, self.weight, None)
        return out + self.bias if self.bias is not None else out


class LinearWithSyncFunc(nn.Linear):
    """``F.linear(x, W) -> sync_fn -> + bias``.

    After :func:`slapo_b200.parallel.lowering.lower_fused_tp` the module carries
    a *fused plan*: ``fused_pre = ("ag", ctx)`` (its input is all-gathered
    inside the GEMM), ``fused_post = ("rs" | "ar", ctx)`` (its partial output is
    reduce-scattered / all-reduced by the GEMM's epilogue) or ``fused_bwd =
    ("ar", ctx)`` (its input gradient is all-reduced by the dgrad GEMM); CUDA
    16-bit inputs then run the single-kernel paths, everything else the
    unfused one above."""

    traceable = False

    def __init__(self, in_features, out_features, bias=True, device=None, dtype=None,
                 sync_fn=None):
        super().__init__(in_features, out_features, bias, device, dtype)
        self.sync_fn = sync_fn
        self.fused_pre = None
        self.fused_post = None
        self.fused_bwd = None

    def matmul_sync(self, x, epilogue_bias=None):
        """matmul and the collectives around it, without the module's own bias
        handling; ``epilogue_bias`` is added inside the GEMM when that is legal
        (i.e. no reduction follows)."""
        if self.fused_pre or self.fused_post or self.fused_bwd:
            from ..parallel import fused_tp

            if fused_tp.supported(x):
                if self.fused_pre is not None:
                    return fused_tp.ag_linear(x, self.weight, epilogue_bias, self.fused_pre[1])
                if self.fused_post is not None:
                    kind, ctx = self.fused_post
                    fn = fused_tp.rs_linear if kind == "rs" else fused_tp.ar_linear
                    out = fn(x, self.weight, None, ctx)
                    return out if epilogue_bias is None else out + epilogue_bias
                return fused_tp.col_linear_ar_bwd(x, self.weight, epilogue_bias, self.fused_bwd[1])
            return self._unfused_fallback(x, epilogue_bias)
        if self.sync_fn is None:
            return NF.linear(x, self.weight, epilogue_bias)     # bias in the GEMM epilogue
        out = self.sync_fn(NF.linear(x, self.weight, None))
        return out if epilogue_bias is None else out + epilogue_bias

    def _unfused_fallback(self, x, epilogue_bias):
        """The plan's collectives through torch.distributed (CPU tensors, fp32)."""
        from ..parallel import sync_ops as so

        if self.fused_pre is not None:
            x = so.all_gather_forward_output(x, 0, self.fused_pre[1].group)
        elif self.fused_bwd is not None:
            x = so.reduce_backward_grad(x, self.fused_bwd[1].group)
        out = F.linear(x, self.weight, None)
        if self.fused_post is not None:
            kind, ctx = self.fused_post
            out = (so.reduce_scatter_forward_output(out, 0, ctx.group) if kind == "rs"
                   else so.reduce_forward_output(out, ctx.group))
        return out if epilogue_bias is None else out + epilogue_bias

    def forward(self, x, skip_bias: bool = False):
        """``skip_bias=True`` leaves the bias to the caller, which fuses it
        into the kernel that follows (dropout / residual / LayerNorm)."""
        return self.matmul_sync(x, None if (skip_bias or self.bias is None) else self.bias)

    @classmethod
    def from_linear(cls, linear: nn.Linear, **kwargs):
        """Same parameters (shared objects), new forward."""
        new = cls(linear.in_features, linear.out_features, bias=linear.bias is not None,
                  device="meta", **kwargs)
        new.weight = linear.weight
        if linear.bias is not None:
            new.bias = linear.bias
        return new

    def _sync_repr(self):
        fn = self.sync_fn
        if fn is None:
            return "None"
        op = getattr(fn, "sync_op", None)
        if op is not None:
            kw = ", ".join(f"{k}={v}" for k, v in getattr(fn, "sync_kwargs", {}).items())
            return f"{op}({kw})"
        inner = getattr(fn, "func", fn)
        text = getattr(inner, "__name__", repr(inner))
        kws = getattr(fn, "keywords", None)
        if kws:
            text += "(" + ", ".join(f"{k}={v}" for k, v in kws.items() if k != "group") + ")"
        return text

    def extra_repr(self):
        text = f"{super().extra_repr()}, sync_fn={self._sync_repr()}"
        for name in ("fused_pre", "fused_post", "fused_bwd"):
            plan = getattr(self, name, None)
            if plan is not None:
                text += f", {name}={plan[0]}"
        return text


class Conv1DWithSyncFunc(nn.Module):
    """GPT-2 ``Conv1D`` (weight ``[in, out]``) as ``x @ W -> sync_fn -> + bias``."""

    traceable = False

    def __init__(self, nf, nx, device=None, dtype=None, sync_fn=None):
        super().__init__()
        self.nf, self.nx = nf, nx
        self.weight = nn.Parameter(torch.empty(nx, nf, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(nf, device=device, dtype=dtype))
        self.sync_fn = sync_fn

    def forward(self, x):
        if self.sync_fn is None:
            return NF.linear_t(x, self.weight, self.bias)
        return self.sync_fn(NF.linear_t(x, self.weight, None)) + self.bias

    def extra_repr(self):
        return f"nx={self.nx}, nf={self.nf}, sync_fn={self.sync_fn}"


_ACTS = ("gelu", "gelu_new", "gelu_tanh", "gelu_pytorch_tanh", "relu")


class LinearWithAct(LinearWithSyncFunc):
    """Linear whose bias add and activation run as one kernel."""

    def __init__(self, in_features, out_features, bias=True, act_fn="gelu", device=None,
                 dtype=None, sync_fn=None):
        super().__init__(in_features, out_features, bias, device, dtype, sync_fn)
        if act_fn not in _ACTS:
            raise NotImplementedError(f"unsupported activation {act_fn}")
        self.act_fn = act_fn

    def forward(self, x):
        if (self.sync_fn is None and not (self.fused_pre or self.fused_post or self.fused_bwd)
                and NF.gemm_supported(x, self.weight)):
            # local product: bias and activation ride in the GEMM's epilogue
            return NF.linear(x, self.weight, self.bias, self.act_fn)
        return NF.bias_act(self.matmul_sync(x), self.bias, self.act_fn)

    def extra_repr(self):
        return f"{super().extra_repr()}, act_fn={self.act_fn}"


class LinearWithDropout(LinearWithSyncFunc):
    """Linear whose bias add and dropout run as one kernel."""

    def __init__(self, in_features, out_features, bias=True, p=0.5, inplace=False,
                 device=None, dtype=None, sync_fn=None):
        super().__init__(in_features, out_features, bias, device, dtype, sync_fn)
        self.p = p

    def forward(self, x):
        return NF.bias_dropout(self.matmul_sync(x), self.bias, self.p, self.training)

    def extra_repr(self):
        return f"{super().extra_repr()}, p={self.p}"


class FusedQKV(nn.Module):
    """Fused q/k/v projection for ``num_heads // world_size`` local heads.

    The weight rows are ordered ``[head][q|k|v][head_dim]``, so slicing axis 0
    by the tensor-parallel size hands each rank whole heads."""

    def __init__(self, hidden_size, num_heads, world_size=1, bias=True, device=None, dtype=None):
        super().__init__()
        if hidden_size % num_heads != 0 or num_heads % world_size != 0:
            raise ValueError("hidden_size % num_heads and num_heads % world_size must be 0")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.head_size = hidden_size // num_heads
        self.world_size = world_size
        self.fused_linear = nn.Linear(hidden_size, 3 * num_heads // world_size * self.head_size,
                                      bias=bias, device=device, dtype=dtype)

    def forward(self, hidden_states):
        qkv = self.fused_linear(hidden_states)
        new_shape = qkv.shape[:-1] + (self.num_heads // self.world_size, 3, self.head_size)
        qkv = qkv.view(new_shape)
        return qkv[..., 0, :], qkv[..., 1, :], qkv[..., 2, :]
