"""The ``"native"`` target: this framework's own runtime.

``build(sch, target="native", config=..., mesh=..., loss_fn=...)`` returns
``(TrainEngine, engine)`` - the engine plays both the model and the optimizer
role (``engine.train_batch``); with pipeline cuts it returns a
``PipelineEngine`` running the 1F1B schedule over NCCL p2p.
"""
from __future__ import annotations

from .registry import register_framework_dialect


@register_framework_dialect("native", "runtime_engine")
def init_native_engine(sch, model, config=None, mesh=None, loss_fn=None, dp_group=None,
                       **kwargs):
    from ..runtime.engine import TrainEngine
    from ..runtime.pipeline_engine import PipelineEngine, PipelineModel

    fused = kwargs.pop("fused_tp", True)
    ctx = None
    import torch as _torch

    if _torch.cuda.is_available():
        # every remaining plain nn.Linear runs its three GEMMs on this library's kernels
        from ..ops.linear import adopt_native_linears

        adopt_native_linears(sch.mod)
        if isinstance(model, _torch.nn.Module):
            adopt_native_linears(model)
    if fused and sch.world_size > 1:
        import torch

        if torch.cuda.is_available():
            from ..parallel.lowering import lower_fused_tp
            from ..parallel.symm import SymmContext

            # structural only (plans on the Linear modules); inside a pipeline the stage
            # modules are the very objects the schedule tree points at
            ctx = SymmContext(sch.group)
            lower_fused_tp(sch, ctx)
    if isinstance(model, PipelineModel):
        engine = PipelineEngine(model, config=config, mesh=mesh, loss_fn=loss_fn,
                                tp_group=sch.group, **kwargs)
        engine.symm_ctx = ctx
        return engine, engine
    if ctx is not None:
        model = sch.mod
    engine = TrainEngine(model, config=config, mesh=mesh, tp_group=sch.group,
                         dp_group=dp_group, loss_fn=loss_fn)
    engine.symm_ctx = ctx
    return engine, engine


@register_framework_dialect("native", "pipeline_stage")
def native_pipeline_stage(*args, **kwargs):
    from ..runtime.pipeline_engine import PipelineStage

    return PipelineStage(*args, **kwargs)


@register_framework_dialect("native", "pipeline_engine")
def native_pipeline_engine(*args, **kwargs):
    from ..runtime.pipeline_engine import PipelineModel

    return PipelineModel(*args, **kwargs)
