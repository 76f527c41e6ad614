"""Version comparison helpers (parity: slapo/utils/versions.py:30-62)."""
import importlib
import operator

from packaging import version as _v

_OPS = {
    "<": operator.lt, "<=": operator.le, "==": operator.eq,
    "!=": operator.ne, ">=": operator.ge, ">": operator.gt,
}


def compare_versions(lib_or_version, op: str, requirement: str) -> bool:
    if op not in _OPS:
        raise ValueError(f"operation must be one of {list(_OPS)}, got {op}")
    # a string is a library name (its __version__ is compared) unless it already looks
    # like a version number
    if isinstance(lib_or_version, str) and not lib_or_version[:1].isdigit():
        lib_or_version = importlib.import_module(lib_or_version).__version__
    return _OPS[op](_v.parse(str(lib_or_version)), _v.parse(requirement))


def is_torch_version(op: str, requirement: str) -> bool:
    import torch

    return compare_versions(torch.__version__.split("+")[0], op, requirement)
