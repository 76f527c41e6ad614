"""``Verify``: check that a scheduled model still computes what the original did.

Used as a context manager around scheduling code::

    with Verify(sch, example_inputs, device="cuda"):
        sch["fc1"].shard("weight", 0)
        sch["fc2"].shard("weight", 1)
        sch["fc2"].sync("fwd_post", "all_reduce")

On entry it snapshots the unscheduled module.  On exit it materialises the
snapshot, broadcasts inputs and weights from rank 0, runs it, then builds a
copy of the scheduled module whose parameters are the matching slices of the
*same* weights, runs that, and compares the outputs - and, unlike the
reference (forward only, slapo/verify.py:58), the **gradients**: full
gradients of the original are sliced along each parameter's shard axis and
compared with the scheduled model's local gradients.  A missing or wrong
``sync`` therefore fails either check.  Works on CPU (gloo) and CUDA (NCCL).

Parity: slapo/verify.py:21-125 of the reference.
"""
from __future__ import annotations

import copy
from contextlib import ContextDecorator

import torch
import torch.distributed as dist

from .logger import get_logger
from .random import set_random_seed

logger = get_logger("verify")


def _first_tensor(out):
    if torch.is_tensor(out):
        return out
    if isinstance(out, dict):
        for v in out.values():
            t = _first_tensor(v)
            if t is not None:
                return t
        return None
    if isinstance(out, (tuple, list)):
        for v in out:
            t = _first_tensor(v)
            if t is not None:
                return t
    return None


def _slice_like(full, local_shape, rank, world):
    diff = [i for i, (a, b) in enumerate(zip(full.shape, local_shape)) if a != b]
    if not diff:
        return full
    return full.chunk(world, dim=diff[0])[rank]


class Verify(ContextDecorator):
    """Context manager around a block of scheduling primitives: on exit the scheduled model is
    run against a copy taken on entry - forward outputs and, with ``check_grads``, parameter and
    input gradients (sharded parameters are gathered first) - and a mismatch raises.  Works on
    CPU (gloo ranks) and on GPUs; ``enable=False`` turns it into a no-op."""

    def __init__(self, sch, example_inputs, example_outputs=None, loss_fn=None, device=None,
                 eval_mode=True, enable=True, check_grads=True, init_weights=True,
                 rtol=None, atol=None, **_compat):
        if not isinstance(example_inputs, (list, tuple)):
            example_inputs = [example_inputs]
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.sch = sch
        self.device = torch.device(device)
        self.example_inputs = list(example_inputs)
        self.loss_fn = loss_fn
        self.eval_mode = eval_mode
        self.enable = enable
        self.check_grads = check_grads
        self.init_weights = init_weights
        self.rtol, self.atol = rtol, atol
        self.original_sch = None

    def __enter__(self):
        if self.enable:
            from .schedule import create_schedule

            self.original_sch = create_schedule(copy.deepcopy(self.sch.mod), group=None)
        return self

    # ------------------------------------------------------------------ #
    def _run(self, model, inputs):
        model.train(not self.eval_mode)
        for p in model.parameters():
            p.grad = None
        set_random_seed(2023)
        if self.check_grads:
            # floating-point inputs become leaves, so that a missing backward collective
            # in front of the first sharded layer shows up as a wrong input gradient
            inputs = [x.detach().clone().requires_grad_(True)
                      if torch.is_tensor(x) and x.is_floating_point() else x for x in inputs]
        out = _first_tensor(model(*inputs))
        grads = {}
        if self.check_grads and out is not None and out.requires_grad:
            loss = self.loss_fn(out) if self.loss_fn is not None else out.float().pow(2).mean()
            loss.backward()
            grads = {n: p.grad.detach().clone() for n, p in model.named_parameters()
                     if p.grad is not None}
            for i, x in enumerate(inputs):
                if torch.is_tensor(x) and x.grad is not None:
                    grads[f"<input {i}>"] = x.grad.detach().clone()
        return out.detach() if out is not None else None, grads

    def __exit__(self, exc_type, exc, tb):
        if exc_type is not None or not self.enable:
            return False
        from .build import build
        from .schedule import create_schedule

        sch, dev = self.sch, self.device
        world = sch.world_size
        distributed = dist.is_available() and dist.is_initialized()
        # 1. original model, identical on all ranks
        orig_model, _ = build(self.original_sch, init_weights=self.init_weights, device=dev)
        orig_model.to(dev)
        inputs = [x.to(dev) if torch.is_tensor(x) else x for x in self.example_inputs]
        if distributed:
            for t in inputs:
                if torch.is_tensor(t):
                    dist.broadcast(t, src=0)
            for t in list(orig_model.state_dict().values()):
                if torch.is_tensor(t) and not t.is_meta:
                    dist.broadcast(t, src=0)
        full_state = {k: v.detach().clone() for k, v in orig_model.state_dict().items()}
        ref_out, ref_grads = self._run(orig_model, inputs)

        # 2. scheduled copy with the matching slices of the same weights
        new_sch = create_schedule(copy.deepcopy(sch.mod), group=sch.group_arg)
        new_sch.metadata = copy.copy(sch.metadata)
        rank = sch.rank

        def inject(mod, path):
            for name, tensor in list(mod._parameters.items()) + list(mod._buffers.items()):
                if tensor is None:
                    continue
                key = f"{path}.{name}" if path else name
                if key not in full_state:
                    raise KeyError(
                        f"Verify cannot map '{key}' to the original model; parameters of "
                        "replaced modules must keep their names or be verified separately")
                src = full_state[key]
                tensor.data.copy_(src.to(tensor.dtype))

        scheduled_model, _ = build(new_sch, init_weights=inject, device=dev)
        scheduled_model.to(dev)
        # parameters that were already materialised keep their values in
        # build(); load the reference weights into them as well
        named = dict(scheduled_model.named_parameters())
        named.update(dict(scheduled_model.named_buffers()))
        for key, tensor in named.items():
            if key in full_state:
                src = _slice_like(full_state[key], tensor.shape, rank, world)
                if src.shape == tensor.shape:
                    tensor.data.copy_(src.to(tensor.dtype))
        new_out, new_grads = self._run(scheduled_model, inputs)

        # 3. compare
        kw = {}
        if self.rtol is not None:
            kw = {"rtol": self.rtol, "atol": self.atol if self.atol is not None else 1e-5}
        elif ref_out is not None and ref_out.dtype in (torch.float16, torch.bfloat16):
            kw = {"rtol": 5e-2, "atol": 5e-2}
        else:
            kw = {"rtol": 1e-4, "atol": 1e-4}
        if ref_out is not None:
            torch.testing.assert_close(new_out, ref_out, **kw)
        if self.check_grads:
            checked = 0
            for key, g_new in new_grads.items():
                if key not in ref_grads:
                    continue
                g_ref = _slice_like(ref_grads[key], g_new.shape, rank, world)
                if g_ref.shape != g_new.shape:
                    continue
                torch.testing.assert_close(g_new, g_ref, **kw, msg=lambda m, k=key: f"grad of {k}: {m}")
                checked += 1
            logger.info("verified output and %d parameter gradients", checked, ranks=0)
        else:
            logger.info("verified output", ranks=0)
        if distributed:
            dist.barrier()
        return False
