"""Run a function on N CPU ranks (gloo) in child processes.

``run_distributed(fn, world_size, *args)`` starts ``world_size`` processes,
initialises a gloo group over a temporary file store (no sockets to resolve),
calls ``fn(rank, world_size, *args)`` on each and re-raises the first failure.
``fn`` must be defined at module level (it is pickled by name).  CPU ranks come
from a fork server with torch preloaded (``SLAPO_B200_TEST_SPAWN=1`` spawns them
from scratch instead); NCCL ranks are always spawned.
"""
import multiprocessing
import os
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world_size, store_path, fn, args, backend):
    os.environ.setdefault("OMP_NUM_THREADS", "2")
    torch.set_num_threads(2)
    if backend == "nccl":
        torch.cuda.set_device(rank)
    dist.init_process_group(backend, init_method=f"file://{store_path}", rank=rank,
                            world_size=world_size)
    try:
        torch.manual_seed(9999)
        fn(rank, world_size, *args)
        dist.barrier()
    except Exception:
        traceback.print_exc()
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


_PRELOAD = ["torch", "torch.distributed", "torch.fx", "torch.fx.experimental.meta_tracer", "numpy",
            "slapo_b200", "slapo_b200.models", "transformers"] + [
    f"transformers.models.{m}.modeling_{m}"      # a missing module is skipped by the server
    for m in ("bert", "roberta", "albert", "gpt2", "gpt_neo", "opt", "t5")]


def _start_method(backend):
    """CPU ranks are forked from a fork server that has imported torch and this package once
    (a clean process: no threads, no process group), which takes the import time out of
    every rank of every test; NCCL ranks are spawned from scratch."""
    if backend != "gloo" or os.environ.get("SLAPO_B200_TEST_SPAWN") == "1":
        return "spawn"
    try:
        multiprocessing.set_forkserver_preload(_PRELOAD)
    except Exception:  # pragma: no cover - platforms without a fork server
        return "spawn"
    return "forkserver"


def run_distributed(fn, world_size=2, *args, backend="gloo"):
    fd, store_path = tempfile.mkstemp(prefix="slapo_b200_store_")
    os.close(fd)
    os.unlink(store_path)
    try:
        mp.start_processes(_worker, args=(world_size, store_path, fn, args, backend),
                           nprocs=world_size, join=True, start_method=_start_method(backend))
    finally:
        if os.path.exists(store_path):
            os.unlink(store_path)
