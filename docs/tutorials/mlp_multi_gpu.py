"""Tensor-parallel MLP on several devices
========================================

    python docs/tutorials/mlp_multi_gpu.py          # two CPU ranks over gloo
    python docs/tutorials/mlp_multi_gpu.py 2 cuda   # two GPUs over NCCL + peer memory

The MLP of a transformer, ``linear2(gelu(linear1(x)))``, is split Megatron-style: the first
weight by output columns, the second by input rows, so that the activation between them
stays sharded and ONE all-reduce after ``linear2`` restores the result.  With the schedule
language that is four lines: two ``shard`` calls per layer and the two ``sync`` points (the
forward all-reduce, and the all-reduce of the input gradient in backward).  ``Verify`` runs
the original and the scheduled module on every rank and compares outputs and gradients - a
forgotten ``sync`` fails right here instead of as a diverging loss days later.

On GPUs ``build(..., target="native")`` lowers those ``shard`` + ``sync`` pairs to kernels that
do the GEMM and the collective together over NVLink peer memory; on CPU ranks the same
schedule runs ``torch.distributed`` collectives, which is how this tutorial runs anywhere.
"""
import copy
import os
import sys

import torch
import torch.distributed as dist
from torch import nn

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import slapo_b200 as slapo  # noqa: E402


class MLP(nn.Module):
    def __init__(self, hidden):
        super().__init__()
        self.linear1 = nn.Linear(hidden, 4 * hidden)
        self.activation = nn.GELU()
        self.linear2 = nn.Linear(4 * hidden, hidden)

    def forward(self, data):
        return self.linear2(self.activation(self.linear1(data)))


def worker(rank, world, device):
    slapo.env.setup(rank, world, backend="nccl" if device == "cuda" else "gloo", port=12377)
    dev = torch.device(device, rank) if device == "cuda" else torch.device("cpu")
    torch.manual_seed(0)                       # the same model on every rank
    model = MLP(64).to(dev)
    x = torch.randn(8, 64, device=dev)

    sch = slapo.create_schedule(copy.deepcopy(model))
    print(f"[rank {rank}] schedule over {sch.world_size} ranks") if rank == 0 else None
    with slapo.Verify(sch, [x], device=str(dev)):
        # column-parallel: rank r keeps rows [r * n/p, (r+1) * n/p) of the weight (and bias)
        sch["linear1"].shard("weight", axis=0)
        sch["linear1"].shard("bias", axis=0)
        # its input is replicated, so the input gradient is a partial sum
        sch["linear1"].sync(mode="bwd_post", sync_op_or_fn="all_reduce")
        # row-parallel: the contraction dimension is split, the output is a partial sum
        sch["linear2"].shard("weight", axis=1)
        sch["linear2"].sync(mode="fwd_post", sync_op_or_fn="all_reduce")
    built, _ = slapo.build(sch, init_weights=False)
    if rank == 0:
        print(built)
        print("local shapes:", tuple(built.linear1.weight.shape), tuple(built.linear2.weight.shape))
    assert built.linear1.weight.shape[0] == 4 * 64 // world
    torch.testing.assert_close(built(x), model(x), rtol=1e-4, atol=1e-4)

    # what happens without the forward sync?  Verify says so.
    sch2 = slapo.create_schedule(copy.deepcopy(model))
    try:
        with slapo.Verify(sch2, [x], device=str(dev)):
            sch2["linear1"].shard("weight", axis=0)
            sch2["linear1"].shard("bias", axis=0)
            sch2["linear1"].sync(mode="bwd_post", sync_op_or_fn="all_reduce")
            sch2["linear2"].shard("weight", axis=1)       # ... and no all-reduce after it
    except Exception as err:
        if rank == 0:
            print("Verify caught the missing all-reduce:", str(err).splitlines()[0][:90])
    else:
        raise AssertionError("a missing sync must not verify")
    dist.barrier()
    slapo.env.cleanup()
    if rank == 0:
        print("multi-device tutorial finished")


if __name__ == "__main__":
    n = int(sys.argv[1]) if len(sys.argv) > 1 else 2
    where = sys.argv[2] if len(sys.argv) > 2 else "cpu"
    slapo.env.execute(worker, args=(n, where), world_size=n)
