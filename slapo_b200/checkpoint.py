"""Activation checkpointing with exact RNG replay.

``checkpoint(fn, *args)`` runs ``fn`` without keeping its intermediates and
recomputes them in backward.  Once ``set_random_seed`` has armed the RNG
tracker the recomputation restores the CPU generator, the device generator
and every named tracker stream to what they were at the first run, so dropout
masks - inside and outside ``fork()`` regions - are bit-identical.  Without a
seeded tracker it defers to ``torch.utils.checkpoint``.

Parity: slapo/checkpoint.py:15-124 of the reference.
"""
from __future__ import annotations

import torch
from torch.utils.checkpoint import checkpoint as torch_checkpoint

from .random import _get_state, _set_state, get_cuda_rng_tracker, is_random_seed_set


class _CheckpointWithRNGReplay(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_fn, n_args, *args):
        ctx.run_fn = run_fn
        ctx.cpu_state = torch.get_rng_state()
        ctx.dev_state = _get_state()
        ctx.tracker_states = get_cuda_rng_tracker().get_states()
        ctx.autocast = torch.is_autocast_enabled()
        with torch.no_grad():
            outputs = run_fn(*args)
        tensors, ctx.non_tensor = [], {}
        for i, a in enumerate(args):
            if torch.is_tensor(a):
                tensors.append(a)
            else:
                ctx.non_tensor[i] = a
        ctx.n_args = len(args)
        ctx.save_for_backward(*tensors)
        return outputs

    @staticmethod
    def backward(ctx, *grads):
        saved = list(ctx.saved_tensors)
        args = []
        for i in range(ctx.n_args):
            if i in ctx.non_tensor:
                args.append(ctx.non_tensor[i])
            else:
                t = saved.pop(0)
                d = t.detach()
                d.requires_grad_(t.requires_grad)
                args.append(d)
        # replay under the states of the first run, then put the live ones back
        live_cpu, live_dev = torch.get_rng_state(), _get_state()
        tracker = get_cuda_rng_tracker()
        live_tracker = tracker.get_states()
        torch.set_rng_state(ctx.cpu_state)
        _set_state(ctx.dev_state)
        tracker.set_states(ctx.tracker_states)
        try:
            with torch.enable_grad():
                outputs = ctx.run_fn(*args)
        finally:
            torch.set_rng_state(live_cpu)
            _set_state(live_dev)
            tracker.set_states(live_tracker)
        if torch.is_tensor(outputs):
            outputs = (outputs,)
        outs, gs = [], []
        for out, g in zip(outputs, grads):
            if torch.is_tensor(out) and out.requires_grad and g is not None:
                outs.append(out)
                gs.append(g)
        if outs:
            torch.autograd.backward(outs, gs)
        in_grads = tuple(a.grad if torch.is_tensor(a) else None for a in args)
        return (None, None) + in_grads


def checkpoint(function, *args, use_reentrant=True, **kwargs):
    """Checkpoint ``function(*args)``; see the module docstring."""
    if is_random_seed_set():
        if kwargs:
            raise ValueError("keyword arguments are not supported with RNG replay; "
                             "pass them positionally")
        return _CheckpointWithRNGReplay.apply(function, len(args), *args)
    return torch_checkpoint(function, *args, use_reentrant=use_reentrant, **kwargs)
