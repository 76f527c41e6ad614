"""Registry of per-model scheduling recipes (parity: slapo/model_schedule/registry.py:7-28)."""
from __future__ import annotations

SCHEDULE_METHODS: dict[str, callable] = {}


def register_schedule(name: str | None = None, override: bool = False):
    def decorator(fn):
        key = name or fn.__module__.rsplit(".", 1)[-1]
        if key in SCHEDULE_METHODS and not override:
            raise ValueError(f"schedule '{key}' is already registered")
        SCHEDULE_METHODS[key] = fn
        return fn

    return decorator


def get_schedule(name: str):
    if name not in SCHEDULE_METHODS:
        raise ValueError(f"no schedule registered for '{name}'; known: {sorted(SCHEDULE_METHODS)}")
    return SCHEDULE_METHODS[name]
