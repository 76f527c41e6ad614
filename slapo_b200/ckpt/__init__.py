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

Tensors are stored under the names of the unpartitioned model, whatever the pipeline
layout: the partitioner records them on every stage module (``original_tensor_names``),
and the other names of a tied tensor travel in the manifest (``aliases``), because a
stage may hold ``lm_head.weight`` without ``wte.weight``.  A checkpoint written by
2 stages x 2-way tensor parallelism therefore loads - weights and optimizer state - into
a tensor-parallel-only job or a single process, and the other way round; ``save_checkpoint``
and ``load_checkpoint`` accept a pipeline engine in place of ``(stage module, stage engine)``.
"""
from .io import (consolidate_checkpoint, load_checkpoint, read_manifest,  # noqa: F401
                 reshard_checkpoint, save_checkpoint)
