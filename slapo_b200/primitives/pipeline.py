"""``cut_pipeline_stage``: mark the end of a pipeline stage.

``sch["encoder.layer.11"].cut_pipeline_stage()`` says "a stage ends after
this module".  The parent must already be traced (``trace_until``): the cut
is recorded on the ``call_module`` node of this child as
``node.meta["partition"] = True`` and the parent's path is appended to the
ordered cut list of the top schedule; ``build`` later splits the graphs.

Parity: slapo/primitives/pipeline.py:13-63 of the reference.
"""
from __future__ import annotations

from torch import fx

from .base import Primitive, register_primitive


@register_primitive()
class PipelineCutPrimitive(Primitive):
    @staticmethod
    def name():
        return "cut_pipeline_stage"

    @staticmethod
    def init_metadata():
        return []

    @staticmethod
    def apply(sch):
        parent = sch.parent
        if parent is None:
            raise ValueError("the top module cannot be a pipeline cut")
        if not isinstance(parent.mod, fx.GraphModule):
            raise RuntimeError(
                f"parent of {sch.path} is not traced; call trace_until('{parent.path}') first")
        target = sch.name
        node = next((n for n in parent.mod.graph.nodes
                     if n.op == "call_module" and n.target == target), None)
        if node is None:
            raise RuntimeError(f"no call of '{target}' in the traced graph of '{parent.path}'")
        node.meta["partition"] = True
        top = sch.get_top_schedule()
        cuts = top.metadata.primitives.get("cut_pipeline_stage")
        if cuts is None:
            cuts = top.metadata.primitives["cut_pipeline_stage"] = []
        if parent.path not in cuts:
            cuts.append(parent.path)
