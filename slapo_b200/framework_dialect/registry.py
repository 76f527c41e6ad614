"""Registry of runtime adapters ("dialects").

A dialect binds the schedule language to a training runtime.  Four kinds of
adapter exist: ``pipeline_stage`` (wraps one stage module), ``pipeline_engine``
(assembles the stages), ``runtime_engine`` (returns ``(model, optimizer)``)
and ``log_parser`` (extracts throughput / memory from a training log for the
auto-tuner).  Built-in targets: ``None`` (no runtime: ``(model, None)``) and
``"native"`` (this framework's own engines).  ``"deepspeed"`` and ``"megatron"`` resolve to
the native engines after their arguments have been translated (``compat.py``), and log
parsers are provided for logs of those tools.

Parity: slapo/framework_dialect/registry.py:5-50 of the reference.
"""
from __future__ import annotations

DIALECT_KINDS = ("pipeline_stage", "pipeline_engine", "runtime_engine", "log_parser")

DIALECTS: dict[str, dict] = {kind: {} for kind in DIALECT_KINDS}
DIALECTS["runtime_engine"][None] = lambda sch, model, **kwargs: (model, None)


def register_framework_dialect(target, cls_type, override: bool = False):
    if cls_type not in DIALECTS:
        raise ValueError(f"unknown dialect kind '{cls_type}'; expected one of {DIALECT_KINDS}")

    def decorator(obj):
        if target in DIALECTS[cls_type] and not override:
            raise ValueError(f"{cls_type} of target '{target}' is already registered")
        DIALECTS[cls_type][target] = obj
        return obj

    return decorator


def get_all_dialects(cls_type):
    if cls_type not in DIALECTS:
        raise ValueError(f"unknown dialect kind '{cls_type}'")
    return DIALECTS[cls_type]


def get_dialect_cls(cls_type, target, allow_none: bool = False):
    table = get_all_dialects(cls_type)
    if target not in table:
        if allow_none and None in table:
            return table[None]
        raise ValueError(f"target '{target}' has no {cls_type}; known: {list(table)}")
    return table[target]
