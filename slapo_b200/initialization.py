"""Delayed (meta-device) initialisation.

Under ``init_empty_weights()`` every parameter registered on any module lands
on the ``meta`` device, so a model of any size can be constructed, scheduled
and sharded without memory; ``build`` materialises only this rank's slices.

Parity: slapo/initialization.py:14-109 of the reference.
"""
from __future__ import annotations

import contextlib

import torch
from torch import nn


@contextlib.contextmanager
def init_on_device(device, include_buffers: bool = False):
    """Place every newly registered parameter (and buffer) on ``device``."""
    device = torch.device(device)
    old_register_parameter = nn.Module.register_parameter
    old_register_buffer = nn.Module.register_buffer

    def register_parameter(module, name, param):
        old_register_parameter(module, name, param)
        if param is not None and param.device != device:
            cls = type(module._parameters[name])
            extra = {k: v for k, v in vars(module._parameters[name]).items()}
            new = cls(module._parameters[name].to(device), requires_grad=param.requires_grad)
            for k, v in extra.items():
                try:
                    setattr(new, k, v)
                except Exception:  # pragma: no cover
                    pass
            module._parameters[name] = new

    def register_buffer(module, name, tensor, persistent=True):
        old_register_buffer(module, name, tensor, persistent=persistent)
        if tensor is not None and tensor.device != device:
            module._buffers[name] = module._buffers[name].to(device)

    factories = {}
    if include_buffers:
        for fname in ("empty", "zeros", "ones", "full"):
            orig = getattr(torch, fname)
            factories[fname] = orig

            def patched(*args, __orig=orig, **kwargs):
                kwargs["device"] = device
                return __orig(*args, **kwargs)

            setattr(torch, fname, patched)
    nn.Module.register_parameter = register_parameter
    if include_buffers:
        nn.Module.register_buffer = register_buffer
    try:
        yield
    finally:
        nn.Module.register_parameter = old_register_parameter
        nn.Module.register_buffer = old_register_buffer
        for fname, orig in factories.items():
            setattr(torch, fname, orig)


@contextlib.contextmanager
def init_empty_weights(enable: bool = True, include_buffers: bool = False):
    """Context manager: modules created inside get their parameters (and, on request, buffers)
    on the meta device - shapes only, no memory - until ``build`` materialises each rank's
    shards."""
    if not enable:
        yield
        return
    with init_on_device("meta", include_buffers=include_buffers):
        yield
