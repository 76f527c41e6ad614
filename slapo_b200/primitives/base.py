"""Primitive registry.

A primitive is a class with a unique ``name()`` and a static ``apply(sch, ...)``;
``@register_primitive()`` makes it callable as ``sch.<name>(...)`` on every
schedule node.

Parity: slapo/primitives/base.py:7-48 of the reference.
"""
from __future__ import annotations

PRIMITIVES: dict[str, type] = {}


class Primitive:
    """Base class of all schedule primitives."""

    @staticmethod
    def name() -> str:
        raise NotImplementedError

    @staticmethod
    def is_verifiable() -> bool:
        """Whether ``Verify`` should re-check numerics after this primitive."""
        return False

    @staticmethod
    def init_metadata():
        """Initial value of ``sch.metadata.primitives[name]`` (or None)."""
        return None

    @staticmethod
    def apply(sch, *args, **kwargs):
        raise NotImplementedError


def register_primitive(override: bool = False):
    def decorator(cls):
        if not (isinstance(cls, type) and issubclass(cls, Primitive)):
            raise ValueError(f"{cls} must subclass Primitive")
        pname = cls.name()
        if pname in PRIMITIVES and not override:
            raise ValueError(f"primitive {pname} is already registered")
        PRIMITIVES[pname] = cls
        return cls

    return decorator
