"""Differentiable collectives used by ``sync``.

Each op is an autograd function pairing a forward collective with the
collective its gradient needs:

=========================  =====================  ==============================
op                         forward                backward
=========================  =====================  ==============================
all_gather_forward_output  all-gather along dim   reduce-scatter (or local slice
                                                  when the consumer is replicated)
reduce_scatter_forward_…   reduce-scatter         all-gather
scatter_forward_output     keep the local slice   all-gather
reduce_forward_output      all-reduce             identity
reduce_backward_grad       identity               all-reduce
=========================  =====================  ==============================

They run on any backend: NCCL on GPUs, gloo on CPU ranks (the oracle and the
host-side test path).  With a world size of one every op is the identity.
The along-dim helpers gather into / scatter from a rank-major staging tensor
and touch the payload once when ``dim != 0``.

Parity: slapo/sharding/sync_ops.py:13-327 of the reference.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _world(group):
    if not (dist.is_available() and dist.is_initialized()):
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def _norm_dim(dim, ndim):
    return dim if dim >= 0 else dim + ndim


def all_gather_along_dim(inp: torch.Tensor, dim: int, world_size: int, group=None):
    """Concatenate every rank's ``inp`` along ``dim``."""
    if world_size == 1:
        return inp
    dim = _norm_dim(dim, inp.dim())
    src = inp.contiguous()
    if src.dim() == 0:
        src = src.view(1)
    flat = torch.empty((world_size * src.shape[0],) + tuple(src.shape[1:]), dtype=src.dtype,
                       device=src.device)
    dist.all_gather_into_tensor(flat, src, group=group)
    if dim == 0:
        return flat
    staging = flat.view((world_size,) + tuple(src.shape))
    return torch.cat(staging.unbind(0), dim=dim)


def reduce_scatter_along_dim(inp: torch.Tensor, dim: int, world_size: int, group=None):
    """Sum over ranks, keep this rank's slice of ``dim``."""
    if world_size == 1:
        return inp
    dim = _norm_dim(dim, inp.dim())
    if inp.shape[dim] % world_size != 0:
        raise ValueError(f"dim {dim} of size {inp.shape[dim]} is not divisible by {world_size}")
    if dim == 0:
        staging = inp.contiguous()
    else:
        staging = torch.cat(inp.chunk(world_size, dim=dim), dim=0)  # rank-major
    out_shape = list(inp.shape)
    out_shape[dim] //= world_size
    out = torch.empty(out_shape, dtype=inp.dtype, device=inp.device)
    dist.reduce_scatter_tensor(out, staging, group=group)
    return out


def scatter_along_dim(inp: torch.Tensor, dim: int, world_size: int, group=None):
    """This rank's slice of ``dim`` (no communication)."""
    if world_size == 1:
        return inp
    rank = dist.get_rank(group)
    if inp.shape[dim] % world_size != 0:
        raise ValueError(f"dim {dim} of size {inp.shape[dim]} is not divisible by {world_size}")
    return inp.chunk(world_size, dim=dim)[rank].contiguous()


class _AllGatherForwardOutput(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, dim, group, tensor_parallel_output_grad=True):
        ctx.dim, ctx.group = dim, group
        ctx.tp_grad = tensor_parallel_output_grad
        ctx.world = _world(group)[0]
        return all_gather_along_dim(inp, dim, ctx.world, group)

    @staticmethod
    def backward(ctx, grad):
        if ctx.tp_grad:
            g = reduce_scatter_along_dim(grad, ctx.dim, ctx.world, ctx.group)
        else:
            g = scatter_along_dim(grad, ctx.dim, ctx.world, ctx.group)
        return g, None, None, None


class _ReduceScatterForwardOutput(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, dim, group):
        ctx.dim, ctx.group = dim, group
        ctx.world = _world(group)[0]
        return reduce_scatter_along_dim(inp, dim, ctx.world, group)

    @staticmethod
    def backward(ctx, grad):
        return all_gather_along_dim(grad, ctx.dim, ctx.world, ctx.group), None, None


class _ScatterForwardOutput(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, dim, group):
        ctx.dim, ctx.group = dim, group
        ctx.world = _world(group)[0]
        return scatter_along_dim(inp, dim, ctx.world, group)

    @staticmethod
    def backward(ctx, grad):
        return all_gather_along_dim(grad, ctx.dim, ctx.world, ctx.group), None, None


class _ReduceForwardOutput(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, group):
        if _world(group)[0] == 1:
            return inp
        out = inp.contiguous().clone()
        dist.all_reduce(out, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class _ReduceBackwardGradient(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, group):
        ctx.group = group
        return inp.view_as(inp)

    @staticmethod
    def backward(ctx, grad):
        if _world(ctx.group)[0] == 1:
            return grad, None
        grad = grad.contiguous().clone()
        dist.all_reduce(grad, group=ctx.group)
        return grad, None


def all_gather_forward_output(inp, dim, group=None, tensor_parallel_output_grad=True):
    """All-gather ``inp`` along ``dim``; the gradient is reduce-scattered
    (``tensor_parallel_output_grad=True``: each rank's consumer differs) or
    sliced (False: the consumers are replicas)."""
    return _AllGatherForwardOutput.apply(inp, dim, group, tensor_parallel_output_grad)


def reduce_scatter_forward_output(inp, dim, group=None):
    return _ReduceScatterForwardOutput.apply(inp, dim, group)


def scatter_forward_output(inp, dim, group=None):
    return _ScatterForwardOutput.apply(inp, dim, group)


def reduce_forward_output(inp, group=None):
    return _ReduceForwardOutput.apply(inp, group)


def reduce_backward_grad(inp, group=None):
    return _ReduceBackwardGradient.apply(inp, group)
