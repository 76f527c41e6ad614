"""``cut_pipeline_stage``: mark the end of a pipeline stage.

``sch["encoder.layer.11"].cut_pipeline_stage()`` says "a stage ends after
this module".  The parent must already be traced (``trace_until``): the cut
is recorded on the ``call_module`` node of this child as
``node.meta["partition"] = True`` and the parent's path is appended to the
ordered cut list of the top schedule; ``build`` later splits the graphs.

A module that its parent calls several times (ALBERT's shared layer group)
takes ``cut_pipeline_stage(call_index=k)``: the stage ends after the k-th
call (0-based).  The stages on both sides then hold the same parameters,
which the pipeline engine keeps tied (values from the first stage, gradients
summed over the stages).

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
    def apply(sch, call_index=0):
        parent = sch.parent
        if parent is None:
            raise ValueError("the top module cannot be a pipeline cut")
        if not isinstance(parent.mod, fx.GraphModule):
            raise RuntimeError(
                f"parent of {sch.path} is not traced; call trace_until('{parent.path}') first")
        target = sch.name
        calls = [n for n in parent.mod.graph.nodes
                 if n.op == "call_module" and n.target == target]
        if not calls:
            raise RuntimeError(f"no call of '{target}' in the traced graph of '{parent.path}'")
        if not 0 <= call_index < len(calls):
            raise IndexError(f"'{target}' is called {len(calls)} time(s) in '{parent.path}'; "
                             f"call_index {call_index} is out of range")
        node = calls[call_index]
        node.meta["partition"] = True
        top = sch.get_top_schedule()
        cuts = top.metadata.primitives.get("cut_pipeline_stage")
        if cuts is None:
            cuts = top.metadata.primitives["cut_pipeline_stage"] = []
        if parent.path not in cuts:
            cuts.append(parent.path)
