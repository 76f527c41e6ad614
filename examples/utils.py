"""Helpers shared by the example scripts, under the names that scripts written against the
reference use: a DeepSpeed-layout configuration (``build(target="deepspeed")`` translates it for
the native engine), the process-group layout for pipeline x tensor parallelism, even pipeline
cuts and two plain training loops.

Parity: examples/utils.py of the reference (``get_ds_config``, ``create_dist_group_for_pipeline``,
``generate_pipeline_cuts``, ``train_with_torch``, ``train_with_deepspeed_engine``).
"""
from __future__ import annotations

import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from slapo_b200.logger import get_logger  # noqa: E402
from slapo_b200.parallel.mesh import DeviceMesh, generate_pipeline_cuts  # noqa: E402,F401

logger = get_logger("examples")


def get_ds_config(batch_size, micro_batch_size_per_gpu, fp16=True, zero_stage=0, desc="", bf16=False,
                  sequence_parallel=False):
    """Configuration dict in DeepSpeed's layout: AdamW at 1e-4, clipping at 1.0, the batch
    sizes, and a ZeRO block when ``zero_stage > 0``."""
    config = {
        "help": desc,
        "steps_per_print": 10,
        "train_batch_size": batch_size,
        "train_micro_batch_size_per_gpu": micro_batch_size_per_gpu,
        "optimizer": {"type": "AdamW", "params": {"lr": 1e-4}},
        "gradient_clipping": 1.0,
        "fp16": {"enabled": bool(fp16), "initial_scale_power": 12},
        "bf16": {"enabled": bool(bf16)},
        "pipeline": {"sequence_parallel": bool(sequence_parallel)},
        "wall_clock_breakdown": False,
    }
    if zero_stage > 0:
        config["zero_optimization"] = {"stage": int(zero_stage), "overlap_comm": True,
                                       "reduce_scatter": True, "contiguous_gradients": False,
                                       "prefetch_bucket_size": 5e8}
        config["zero_allow_untested_optimizer"] = True
    return config


def create_dist_group_for_pipeline(num_pp, num_mp):
    """``(topology, tensor_parallel_group)`` for ``num_pp`` pipeline stages of ``num_mp``-way
    tensor parallelism; the rest of the world is data parallel.  The topology is this
    framework's :class:`DeviceMesh` (``build(..., topology=mesh)`` and ``mesh=mesh`` both take it)."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world % (num_pp * num_mp):
        raise ValueError(f"{world} ranks do not split into {num_pp} stages x {num_mp}-way TP")
    mesh = DeviceMesh(pp=num_pp, dp=world // (num_pp * num_mp), tp=num_mp)
    return mesh, mesh.tp_group


def _loss_of(model, inputs, labels, loss_fn):
    if loss_fn is None:
        out = model(*inputs, labels=labels)
        return out["loss"] if isinstance(out, dict) else out.loss
    out = model(*inputs)
    return loss_fn(out["logits"] if isinstance(out, dict) else out.logits, labels)


def train_with_torch(model, dataloader, optimizer, loss_fn=None, preproc=None, postproc=None,
                     steps=40):
    """Plain PyTorch loop (no data parallelism, no gradient accumulation); returns the losses."""
    losses = []
    for step, batch in enumerate(dataloader):
        inputs, labels = preproc(step, batch) if preproc is not None else batch
        optimizer.zero_grad(set_to_none=True)
        loss = _loss_of(model, inputs, labels, loss_fn)
        loss.backward()
        optimizer.step()
        loss = postproc(step, loss) if postproc is not None else loss
        losses.append(float(loss))
        if step % 10 == 0:
            logger.info("step %d loss: %.4f", step, losses[-1], ranks=0)
        if step + 1 >= steps:
            break
    return losses


def train_with_engine(engine, dataloader, preproc=None, postproc=None, steps=40, device=None):
    """Loop over ``engine.train_batch`` (the engine that ``build(target="native")`` - or the
    ``"deepspeed"`` target - returns); logs samples / s after a short warm-up and returns the
    losses."""
    device = device if device is not None else next(engine.model.parameters()).device
    losses, seen, t0 = [], 0, None
    for step, batch in enumerate(dataloader):
        inputs, labels = preproc(step, batch) if preproc is not None else batch
        if isinstance(inputs, dict):        # named inputs (encoder-decoder models)
            inputs = {k: t.to(device) if torch.is_tensor(t) else t for k, t in inputs.items()}
            loss = engine.train_batch(**inputs, labels=labels.to(device))
        else:
            inputs = [t.to(device) if torch.is_tensor(t) else t for t in inputs]
            loss = engine.train_batch(*inputs, labels=labels.to(device))
        loss = postproc(step, loss) if postproc is not None else loss
        losses.append(float(loss))
        if step == 2:
            t0, seen = time.time(), 0
        seen += labels.shape[0]
        if step % 10 == 0:
            logger.info("step %d loss: %.4f", step, losses[-1], ranks=0)
        if step + 1 >= steps:
            break
    if t0 is not None and time.time() > t0:
        logger.info("%.1f samples/s", (seen - labels.shape[0]) / (time.time() - t0), ranks=0)
    return losses


train_with_deepspeed_engine = train_with_engine


# the name the reference's scripts call (examples/utils.py:134 there); the engine that
# ``build(target="deepspeed")`` returns here is this framework's own
train_with_deepspeed_engine = train_with_engine
