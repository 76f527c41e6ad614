"""Sharded checkpoints: save / load / consolidate / reshard / resume.

The reference has no checkpoint code of its own - saving and resuming is left
to DeepSpeed or Megatron (slapo/build.py:234-272 hands the model to them).
Here the native engine owns the optimizer, so it owns the checkpoint too.

Layout of a checkpoint directory::

    manifest.json                 mesh, step, per-parameter table (local shape, full
                                  ``orig_shape``, sharded axis, pipeline stage, dtype)
    model_pp{P}_tp{T}.pt          {name: local shard}       written by DP rank 0
    optim_pp{P}_tp{T}.pt          {"step", "state": {name: {master, exp_avg, exp_avg_sq}}}
                                  per parameter, in the parameter's local shape: no
                                  trace of buckets, ZeRO slices or the DP size
    rng_rank{R}.pt                python / numpy / torch / CUDA / tensor-parallel RNG state
    extra.pt                      user payload (rank 0)

Because optimizer state is stored per parameter, a checkpoint written by a
``dp8`` ZeRO run resumes on ``dp2`` unchanged, and :func:`reshard_checkpoint`
re-splits both weights and optimizer moments for another TP size by
concatenating along the recorded axis and slicing again.
"""
from .io import (consolidate_checkpoint, load_checkpoint, read_manifest,  # noqa: F401
                 reshard_checkpoint, save_checkpoint)
