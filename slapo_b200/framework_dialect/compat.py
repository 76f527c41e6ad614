"""``target="deepspeed"`` and ``target="megatron"`` for code written against the reference.

The reference hands a scheduled model to DeepSpeed (``build(sch, target="deepspeed",
config=ds_config, topology=topology, loss_fn=...)``) or wraps it for Megatron-LM.  Neither
runtime is needed here: both targets resolve to this framework's own engines, after the call's
arguments have been translated -

* ``config``: a DeepSpeed configuration dict (``optimizer.params``, ``gradient_clipping``,
  ``train_batch_size`` / ``train_micro_batch_size_per_gpu`` / ``gradient_accumulation_steps``,
  ``zero_optimization.stage``) becomes an :class:`~slapo_b200.runtime.engine.EngineConfig`;
* ``topology``: a DeepSpeed ``ProcessTopology`` (anything with ``get_dim(axis)`` for the axes
  ``pipe`` / ``data`` / ``model``), a ``{"pp", "dp", "tp"}`` dict or a ``DeviceMesh`` becomes
  the mesh.

Parity: slapo/framework_dialect/deepspeed/engine.py:11-49 and pipeline.py:357-490 of the
reference (the runtime side of those files is ``runtime/engine.py`` and
``runtime/pipeline_engine.py`` here).
"""
from __future__ import annotations

from ..logger import get_logger
from .registry import get_dialect_cls, register_framework_dialect

logger = get_logger("dialect")


def mesh_from_topology(topology):
    """``DeviceMesh`` for a DeepSpeed-style topology, a ``{"pp","dp","tp"}`` dict or a mesh."""
    from ..parallel.mesh import DeviceMesh

    if topology is None or isinstance(topology, DeviceMesh):
        return topology
    if isinstance(topology, dict):
        dims = {k: int(topology.get(k, 1)) for k in ("pp", "dp", "tp")}
    elif hasattr(topology, "get_dim"):
        def dim(*names):
            for name in names:
                try:
                    return int(topology.get_dim(name))
                except Exception:   # an axis this topology does not have
                    continue
            return 1

        dims = {"pp": dim("pipe", "pp"), "dp": dim("data", "dp"), "tp": dim("model", "tensor", "tp")}
    else:
        raise TypeError(f"cannot read a (pp, dp, tp) layout from {type(topology).__name__}")
    import torch.distributed as dist

    if dims["pp"] * dims["dp"] * dims["tp"] == 1 and not dist.is_initialized():
        return None         # a single process needs no mesh
    return DeviceMesh(**dims)


def translate_ds_config(config, dp_size=1):
    """Engine configuration dict from a DeepSpeed configuration dict (unknown keys are kept
    under their own names: the engine ignores what it does not know)."""
    if config is None or not isinstance(config, dict):
        return config
    cfg = dict(config)
    out = {}
    opt = cfg.pop("optimizer", None)
    if isinstance(opt, dict):
        if str(opt.get("type", "AdamW")).lower() not in ("adamw", "adam", "fusedadam"):
            logger.warning("optimizer type %s is not available; AdamW runs instead", opt.get("type"))
        for key, val in (opt.get("params") or {}).items():
            if key in ("lr", "eps", "weight_decay"):
                out[key] = val
            elif key == "betas":
                out["betas"] = tuple(val)
    if "gradient_clipping" in cfg:
        out["clip_grad"] = cfg.pop("gradient_clipping")
    micro = cfg.get("train_micro_batch_size_per_gpu")
    total = cfg.get("train_batch_size")
    if "gradient_accumulation_steps" in cfg:
        out["grad_accum_steps"] = int(cfg.pop("gradient_accumulation_steps"))
    elif micro and total:
        out["grad_accum_steps"] = max(1, int(total) // (int(micro) * max(1, dp_size)))
    zero = cfg.pop("zero_optimization", None)
    if isinstance(zero, dict):
        stage = int(zero.get("stage", 0))
        out["zero"] = stage >= 1
        if stage >= 2:
            logger.info("ZeRO stage %d requested: optimizer state is sharded (stage 1); gradients "
                        "are reduce-scattered and parameters all-gathered by the fused kernels", stage)
        if "overlap_comm" in zero:
            out["overlap_comm"] = bool(zero["overlap_comm"])
    else:
        out["zero"] = False
    fp16 = cfg.get("fp16") or {}
    if isinstance(fp16, dict) and fp16.get("enabled"):
        logger.info("fp16 is enabled in the configuration: the model's own dtype decides here "
                    "(pass fp16=True / bf16=True to the schedule recipe); the engine's loss "
                    "scaler takes the block's initial_scale_power / loss_scale / window")
    for key, val in cfg.items():
        out.setdefault(key, val)
    return out


def _with_native(kind):
    return get_dialect_cls(kind, "native")


def _compat_engine(label):
    def init_engine(sch, model, config=None, topology=None, mesh=None, loss_fn=None, **kwargs):
        mesh = mesh if mesh is not None else mesh_from_topology(topology)
        dp = mesh.dp_size if mesh is not None else 1
        logger.info("target %r runs on this framework's native engine", label, ranks=0)
        return _with_native("runtime_engine")(sch, model, config=translate_ds_config(config, dp),
                                              mesh=mesh, loss_fn=loss_fn, **kwargs)

    return init_engine


for _target in ("deepspeed", "megatron"):
    register_framework_dialect(_target, "runtime_engine")(_compat_engine(_target))
    register_framework_dialect(_target, "pipeline_stage")(
        lambda *a, **k: _with_native("pipeline_stage")(*a, **k))
    register_framework_dialect(_target, "pipeline_engine")(
        lambda *a, **k: _with_native("pipeline_engine")(*a, **k))
