"""Hook plumbing and small helpers shared by the primitives.

Parity: slapo/utils/common.py:11-172 of the reference.
"""
from __future__ import annotations

import importlib
from collections import OrderedDict
from types import FunctionType

from torch import fx, nn

HOOK_TYPE_TO_ATTR = {
    "fwd_pre": "_forward_pre_hooks",
    "fwd_post": "_forward_hooks",
    "bwd_post": "_backward_hooks",
}
# dictionaries that travel with the hook dictionaries in recent torch versions
_HOOK_SIDE_ATTRS = {
    "_forward_pre_hooks": ["_forward_pre_hooks_with_kwargs"],
    "_forward_hooks": ["_forward_hooks_with_kwargs", "_forward_hooks_always_called"],
    "_backward_hooks": [],
}


def get_hooks(mod: nn.Module) -> dict:
    """All hooks of ``mod`` as ``{"fwd_pre": [...], "fwd_post": [...], "bwd_post": [...]}``."""
    return {
        kind: list(getattr(mod, attr, OrderedDict()).values())
        for kind, attr in HOOK_TYPE_TO_ATTR.items()
    }


def has_hook(mod: nn.Module, hook_type: str) -> bool:
    if hook_type not in HOOK_TYPE_TO_ATTR:
        raise ValueError(f"unknown hook type {hook_type}")
    return len(getattr(mod, HOOK_TYPE_TO_ATTR[hook_type], ())) > 0


def transfer_hooks(old_mod: nn.Module, new_mod: nn.Module, hook_types=None):
    """Move (not copy) the hooks of the given kinds from old_mod to new_mod."""
    if hook_types is None:
        hook_types = list(HOOK_TYPE_TO_ATTR)
    for kind in hook_types:
        attr = HOOK_TYPE_TO_ATTR[kind]
        src = getattr(old_mod, attr, None)
        if not src:
            continue
        dst = getattr(new_mod, attr)
        for key, hook in src.items():
            dst[key] = hook
        for side in _HOOK_SIDE_ATTRS[attr]:
            if hasattr(old_mod, side) and hasattr(new_mod, side):
                getattr(new_mod, side).update(getattr(old_mod, side))
        if attr == "_backward_hooks" and getattr(old_mod, "_is_full_backward_hook", None) is not None:
            new_mod._is_full_backward_hook = old_mod._is_full_backward_hook
        setattr(old_mod, attr, OrderedDict())


def transfer_hooks_for_fusion(sch, subgraphs, new_mod: nn.Module):
    """Carry hooks across a subgraph replacement.

    For a vertical fusion the first module of the chain may own forward-pre
    and backward hooks and the last one forward-post hooks; they move to the
    fused module.  A hook anywhere else (or any hook under horizontal fusion)
    cannot keep its meaning and raises.
    """
    named = dict(sch.mod.named_modules())

    def module_of(path, node):
        if node.op != "call_module":
            return None
        full = f"{path}.{node.target}" if path else node.target
        return named.get(full)

    if len(subgraphs) > 1:
        for sub in subgraphs:
            for path, node in sub:
                mod = module_of(path, node)
                if mod is not None and any(get_hooks(mod).values()):
                    raise RuntimeError(
                        f"module {node.target} has hooks; hooks cannot be kept "
                        "under horizontal fusion"
                    )
        return
    ops = subgraphs[0]
    for idx, (path, node) in enumerate(ops):
        mod = module_of(path, node)
        if mod is None:
            continue
        hooks = get_hooks(mod)
        first, last = idx == 0, idx == len(ops) - 1
        for kind, items in hooks.items():
            if not items:
                continue
            legal = (kind in ("fwd_pre", "bwd_post") and first) or (kind == "fwd_post" and last)
            if not legal:
                raise RuntimeError(
                    f"{kind} hook on {node.target} sits in the middle of the fused "
                    "region and cannot be transferred"
                )
            transfer_hooks(mod, new_mod, [kind])


def transfor_param_tags(sch, param, new_param):
    """Copy the registered parameter tags (``annotate``) onto a new parameter."""
    for tag in sch.get_top_schedule().metadata.param_tags:
        if hasattr(param, tag):
            setattr(new_param, tag, getattr(param, tag))


transfer_param_tags = transfor_param_tags


def is_lambda_function(obj) -> bool:
    return isinstance(obj, FunctionType) and obj.__name__ == "<lambda>"


def is_module_list(mod) -> bool:
    """True for ``nn.ModuleList`` and for what a ModuleList becomes after
    tracing: a GraphModule-like container that is never called directly and
    whose children are named ``0..n-1``."""
    if isinstance(mod, nn.Sequential):
        return False
    if isinstance(mod, nn.ModuleList):
        return True
    if isinstance(mod, fx.GraphModule):
        return False
    children = [name for name, _ in mod.named_children()]
    if not children or type(mod) is not nn.Module:
        return False
    return children == [str(i) for i in range(len(children))]


def importlib_or_none(name: str):
    try:
        return importlib.import_module(name)
    except Exception:  # ImportError or a broken optional package
        return None
