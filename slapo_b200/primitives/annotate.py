"""``annotate``: attach a tag to a parameter that survives re-sharding.

Parity: slapo/primitives/annotate.py:9-37 of the reference.
"""
from .base import Primitive, register_primitive


@register_primitive()
class AnnotateParamPrimitive(Primitive):
    """``sch.annotate(param_name, key, value)`` sets ``param.<key> = value``
    and registers ``key`` as a tag that ``shard`` and ``build`` copy to every
    replacement of the parameter."""

    @staticmethod
    def name():
        return "annotate"

    @staticmethod
    def apply(sch, param_name, key, value):
        param = getattr(sch.mod, param_name, None)
        if param is None:
            raise KeyError(f"{sch.path or '<root>'} has no parameter '{param_name}'")
        setattr(param, key, value)
        sch.get_top_schedule().metadata.param_tags.add(key)
