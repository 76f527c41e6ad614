"""Pipeline partitioning of a traced schedule (see :mod:`.parallel.pipeline_partition`)
and tied-weight analysis.

Parity: slapo/pipeline.py:17-440 of the reference.
"""
from __future__ import annotations

from torch import nn

from .parallel.pipeline_partition import (analyze_pipeline_module,  # noqa: F401
                                          build_pipeline_model,
                                          generate_pipeline_partition,
                                          propagate_partition)


def analyze_tie_weights(top_mod: nn.Module, is_pipeline_partitioned: bool = False):
    """Find Parameters reachable under more than one name.

    Returns ``{param: [(name, stage_id), ...]}`` for every shared Parameter.
    ``named_parameters()`` hides aliases, so the walk is explicit.  With
    ``is_pipeline_partitioned`` the top level is a sequence of stage modules
    ``submod_<i>``: names drop that prefix and carry the stage index; without
    it every stage id is 0."""
    seen: dict = {}

    def walk(mod, prefix, stage, visited):
        if id(mod) in visited:
            return
        visited.add(id(mod))
        for pname, param in mod._parameters.items():
            if param is None:
                continue
            full = f"{prefix}.{pname}" if prefix else pname
            seen.setdefault(param, []).append((full, stage))
        for cname, child in mod._modules.items():
            if child is None:
                continue
            walk(child, f"{prefix}.{cname}" if prefix else cname, stage, visited)

    if is_pipeline_partitioned:
        stage = 0
        for cname, child in top_mod._modules.items():
            if child is None:
                continue
            if cname.startswith("submod_"):
                walk(child, "", stage, set())
                stage += 1
            else:
                walk(child, cname, max(stage - 1, 0), set())
        for pname, param in top_mod._parameters.items():
            if param is not None:
                seen.setdefault(param, []).append((pname, 0))
    else:
        walk(top_mod, "", 0, set())
    return {p: names for p, names in seen.items() if len(names) > 1}
