"""Alias of :mod:`slapo_b200.graph.tracer` under the reference's module name."""
from .graph.tracer import HierTracer, trace, trace_module  # noqa: F401
