"""``apply_schedule(model, key, **config)`` (parity: slapo/model_schedule/api.py:7-16)."""
from .registry import get_schedule


def apply_schedule(model, schedule_key, **sch_config):
    """Run the registered recipe for ``schedule_key`` (e.g. ``"bert"``) on
    ``model`` and return the resulting schedule (pass it to ``build``)."""
    return get_schedule(schedule_key)(model, **sch_config)
