"""Host-side arithmetic of the allocation-free entry point: how much of its static scratch a
shape needs.  Needs no GPU (148 SMs are assumed when no device can be queried)."""
import ctypes

import pytest

from slapo_b200.ops import native

SCRATCH_FLOATS = 327680   # SLAPO_NOALLOC_SCRATCH_FLOATS of csrc/no_alloc.h
MAX_COLS = 16384


def _need():
    if not native.available():
        pytest.skip(f"extension not built: {native.load_error()}")
    fn = ctypes.CDLL(native.lib_path()).slapo_bias_act_bwd_noalloc_scratch_floats
    fn.restype = ctypes.c_long
    fn.argtypes = [ctypes.c_int, ctypes.c_int]
    return fn


def test_scratch_need_formula_and_bound():
    import torch

    need = _need()
    sms = torch.cuda.get_device_properties(0).multi_processor_count if torch.cuda.is_available() \
        else 148
    for rows, cols in [(1, 8), (37, 264), (4096, 4096), (1 << 20, 256), (1 << 20, 8), (1 << 20, MAX_COLS),
                       (1000, 1024), (65536, 1032)]:
        slabs = (cols + 255) // 256
        chunks = max(1, min((sms * 8 + slabs - 1) // slabs, (rows + 7) // 8))
        assert need(rows, cols) == chunks * cols
    assert need(0, 1024) == 0
    if sms <= 148:
        # every width the entry point accepts fits, however tall the matrix
        worst = max(need(1 << 24, cols) for cols in range(8, MAX_COLS + 1, 8))
        assert worst <= SCRATCH_FLOATS
