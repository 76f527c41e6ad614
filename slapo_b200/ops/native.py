"""Loader of the in-tree ``_C`` extension (hand-written sm_100a kernels).

The shared object is built by ``slapo_b200.csrc.build`` into the package
directory and registers its entry points as ``torch.ops.slapo_b200.*``.
"""
from __future__ import annotations

import os

import torch

_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C.so")
_STATE = {"tried": False, "ok": False, "error": None}


def lib_path() -> str:
    return _LIB


def available() -> bool:
    if not _STATE["tried"]:
        _STATE["tried"] = True
        if os.path.exists(_LIB):
            try:
                torch.ops.load_library(_LIB)
                _STATE["ok"] = True
            except Exception as err:  # pragma: no cover - depends on the build
                _STATE["error"] = str(err)
        else:
            _STATE["error"] = f"{_LIB} does not exist"
    return _STATE["ok"]


def load_error():
    available()
    return _STATE["error"]


def ops():
    if not available():
        raise RuntimeError(f"slapo_b200 native extension unavailable: {_STATE['error']}")
    return torch.ops.slapo_b200


def reset():
    """Forget a failed load (used after building in the same process)."""
    _STATE.update(tried=False, ok=False, error=None)


def launch_count() -> int:
    """Kernels launched by the extension since it was loaded (host counter;
    a CUDA-graph replay re-runs captured launches without counting them)."""
    return int(ops().launch_count()) if available() else 0
