"""Random-number state management for model parallelism.

Two families of random streams are needed in tensor-parallel training:

* the *default* stream - equal on all TP ranks, used where activations are
  replicated (dropout on a replicated tensor must pick the same mask on
  every rank);
* the *tensor-parallel* stream ``"model-parallel-rng"`` - seeded with
  ``seed + 2718 + tp_rank``, used inside ``fork()`` where activations are
  sharded so each rank needs its own mask.

``RNGStatesTracker`` stores named generator states for the current device
type: CUDA generator states on a GPU, CPU generator states otherwise, so
that the same schedules (and the tests that pin their behaviour) run on
gloo/CPU ranks.

Parity: slapo/random.py:18-228 of the reference (CUDA only there).
"""
from __future__ import annotations

import contextlib
import random as _py_random

import numpy as np
import torch

_MODEL_PARALLEL_RNG = "model-parallel-rng"
_SEED_SET = False


def _use_cuda() -> bool:
    return torch.cuda.is_available()


def _capturing() -> bool:
    return _use_cuda() and torch.cuda.is_current_stream_capturing()


def _get_state():
    """State of the device generator (CPU generator without CUDA).  While a CUDA graph is
    being captured the ordinary state cannot be read; the graph-safe handle (which carries the
    offset inside the graph) is returned instead and ``_set_state`` accepts it back."""
    if not _use_cuda():
        return torch.get_rng_state()
    if _capturing():
        return torch.cuda.default_generators[torch.cuda.current_device()].graphsafe_get_state()
    return torch.cuda.get_rng_state()


def _set_state(state):
    if not _use_cuda():
        torch.set_rng_state(state)
    elif isinstance(state, torch.Generator):
        torch.cuda.default_generators[torch.cuda.current_device()].graphsafe_set_state(state)
    else:
        torch.cuda.set_rng_state(state)


def _manual_seed(seed):
    if _use_cuda():
        torch.cuda.manual_seed(seed)
    else:
        torch.manual_seed(seed)


class RNGStatesTracker:
    """Named RNG states; ``fork(name)`` runs a block under one of them and
    stores the advanced state back, leaving the default stream untouched."""

    def __init__(self):
        self.states_ = {}
        self.seeds_ = set()

    def reset(self):
        self.states_ = {}
        self.seeds_ = set()

    def get_states(self):
        return dict(self.states_)

    def set_states(self, states):
        self.states_ = dict(states)

    def add(self, name, seed):
        if seed in self.seeds_:
            raise RuntimeError(f"seed {seed} already exists")
        if name in self.states_:
            raise RuntimeError(f"rng state {name} already exists")
        self.seeds_.add(seed)
        saved = _get_state()
        _manual_seed(seed)
        self.states_[name] = _get_state()
        _set_state(saved)

    @contextlib.contextmanager
    def fork(self, name=_MODEL_PARALLEL_RNG):
        if name not in self.states_:
            raise RuntimeError(f"rng state {name} is not added; call set_random_seed first")
        saved = _get_state()
        _set_state(self.states_[name])
        try:
            yield
        finally:
            self.states_[name] = _get_state()
            _set_state(saved)


# the reference's class name
CudaRNGStatesTracker = RNGStatesTracker

_TRACKER = RNGStatesTracker()


def get_cuda_rng_tracker() -> RNGStatesTracker:
    """The process-wide tracker of named RNG states (``fork_rng`` regions draw from the
    tensor-parallel state so that dropout differs across the ranks of a group)."""
    return _TRACKER


def model_parallel_cuda_manual_seed(seed, tp_rank, always_enable_tp_seed):
    """Seed the default stream with ``seed`` (or, for sequence parallelism
    where every activation is sharded, with the TP seed) and register the TP
    stream ``seed + 2718 + tp_rank``."""
    tp_seed = seed + 2718 + tp_rank
    _TRACKER.reset()
    _manual_seed(tp_seed if always_enable_tp_seed else seed)
    _TRACKER.add(_MODEL_PARALLEL_RNG, tp_seed)
    return tp_seed


def is_random_seed_set() -> bool:
    return _SEED_SET


def set_random_seed(seed=2013, dp_rank=None, pp_rank=None, tp_rank=None,
                    always_enable_tp_seed=False) -> int:
    """Seed python, numpy and torch for this rank.

    Pipeline stages and data-parallel replicas get different base seeds
    (``+100*pp_rank + 10*dp_rank``); TP ranks share the base seed and differ
    only in the tensor-parallel stream.  Returns the base seed."""
    global _SEED_SET
    if pp_rank is not None:
        seed += 100 * pp_rank
    if dp_rank is not None:
        seed += 10 * dp_rank
    _py_random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if tp_rank is not None or _use_cuda():
        model_parallel_cuda_manual_seed(seed, tp_rank or 0, always_enable_tp_seed)
    _SEED_SET = True
    return seed
