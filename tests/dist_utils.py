"""Run a function on N CPU ranks (gloo) in child processes.

``run_distributed(fn, world_size, *args)`` spawns ``world_size`` processes,
initialises a gloo group over a temporary file store (no sockets to resolve),
calls ``fn(rank, world_size, *args)`` on each and re-raises the first failure.
``fn`` must be defined at module level (it is pickled by name).
"""
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


def run_distributed(fn, world_size=2, *args, backend="gloo"):
    fd, store_path = tempfile.mkstemp(prefix="slapo_b200_store_")
    os.close(fd)
    os.unlink(store_path)
    try:
        mp.start_processes(_worker, args=(world_size, store_path, fn, args, backend),
                           nprocs=world_size, join=True, start_method="spawn")
    finally:
        if os.path.exists(store_path):
            os.unlink(store_path)
