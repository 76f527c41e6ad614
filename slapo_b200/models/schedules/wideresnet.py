"""Scheduling recipe for bottleneck Wide ResNets.

Tensor parallelism per bottleneck: ``conv1`` splits its output channels
(``bn1`` follows the split, statistics are per channel so nothing crosses
ranks), ``conv2`` splits its input channels and all-reduces the partial
sums, ``conv3`` splits its output channels and all-gathers them along the
channel axis before ``bn3``.  Checkpointing takes the first
``int(depth * ratio)`` blocks of each of the four groups; pipeline cuts are
given per group (``[[], [3], [10, 30], []]``).

Parity: slapo/model_schedule/wideresnet.py:16-247 of the reference.
"""
from __future__ import annotations

from ... import create_schedule
from ...model_schedule.registry import register_schedule
from .common import broadcast_input, cast_dtype, logger


def _cfg_get(cfg, key):
    return cfg[key] if isinstance(cfg, dict) else getattr(cfg, key)


def shard_bottlenecks(sch, depths):
    if sch.world_size == 1:
        return 0
    n = 0
    for gi, depth in enumerate(depths):
        for bi in range(depth):
            blk = sch[f"layer{gi + 1}"][str(bi)]
            blk["conv1"].shard("weight", axis=0)
            blk["conv1"].sync("bwd_post", "all_reduce")
            for name in ("weight", "bias", "running_mean", "running_var"):
                blk["bn1"].shard(name, axis=0)
            blk["conv2"].shard("weight", axis=1)
            blk["conv2"].sync("fwd_post", "all_reduce")
            blk["conv3"].shard("weight", axis=0)
            blk["conv3"].sync("fwd_post", "all_gather", axis=1,
                              tensor_parallel_output_grad=False)
            blk["conv3"].sync("bwd_post", "all_reduce")
            n += 1
    return n


def checkpoint_bottlenecks(sch, depths, ratio):
    total = 0
    for gi, depth in enumerate(depths):
        for bi in range(int(depth * ratio)):
            sch[f"layer{gi + 1}"][str(bi)].checkpoint()
            total += 1
    return total


@register_schedule("wideresnet")
def schedule_wideresnet(model, model_config=None, prefix="model", fp16=False, bf16=False,
                        group=None, ckpt_ratio=0.0, checkpoint_method="uniform",
                        bcast_input=False, pipeline_cuts=None, channels_last=False, **_unused):
    if model_config is None:
        raise ValueError("model_config is required")
    if checkpoint_method != "uniform":
        raise NotImplementedError(f"checkpoint method {checkpoint_method}")
    _, depths = _cfg_get(model_config, "block_size")
    cast_dtype(model, fp16, bf16)
    if channels_last:
        import torch
        model.to(memory_format=torch.channels_last)
    sch = create_schedule(model, group=group)
    trunk = sch[prefix] if prefix else sch
    n_shard = shard_bottlenecks(trunk, depths)
    if bcast_input:
        broadcast_input(sch)
    n_ckpt = checkpoint_bottlenecks(trunk, depths, ckpt_ratio) if ckpt_ratio > 0 else 0
    if pipeline_cuts:
        if len(pipeline_cuts) != 4:
            raise ValueError("pipeline_cuts needs one list per residual group (4)")
        dot = f"{prefix}." if prefix else ""
        leaves = [f"{dot}layer{i + 1}" for i in range(4) if pipeline_cuts[i]]
        # the stages compute the logits; the loss (and its labels) stays with the engine's
        # loss function, so a wrapper's optional ``labels`` input is frozen at None
        import inspect

        frozen = {"labels": None} if "labels" in inspect.signature(model.forward).parameters \
            else {}
        sch.trace_until(leaves, tracer="pytorch", concrete_args=frozen)
        for i, cuts in enumerate(pipeline_cuts):
            for cut in cuts:
                sch[f"{dot}layer{i + 1}"][str(cut)].cut_pipeline_stage()
    logger.info("wideresnet schedule: %d bottlenecks sharded, %d checkpointed", n_shard, n_ckpt,
                ranks=0)
    return sch
