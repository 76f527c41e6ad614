"""Process bootstrap helpers for tutorials and tests.

``setup`` joins a single-node world over 127.0.0.1, ``cleanup`` leaves it and
``execute`` spawns ``world_size`` processes running ``fn(rank, *args)``.

Parity: slapo/env.py:10-30 of the reference (which is NCCL only; here the
backend defaults to NCCL when CUDA is present and gloo otherwise).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def setup(rank: int, world_size: int, backend: str | None = None, port: int = 12355):
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(port))
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(rank % max(torch.cuda.device_count(), 1))
    dist.init_process_group(backend, rank=rank, world_size=world_size)


def cleanup():
    if dist.is_initialized():
        dist.destroy_process_group()


def execute(fn, args=(), world_size: int | None = None):
    if world_size is None:
        world_size = max(torch.cuda.device_count(), 1)
    mp.spawn(fn, args=tuple(args), nprocs=world_size, join=True)
