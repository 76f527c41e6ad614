"""Data parallelism over NVLink peer memory: gradient reduce-scatter and
AdamW + parameter all-gather as two fused kernels per bucket.

``FusedDP`` owns the symmetric flat gradient / parameter buffers of one
data-parallel group and wraps the kernels of ``csrc/dp_comm.cu``:

* ``grad_rs(bucket, epoch, lo, out, dup_mask)`` - handshake with the peers (a
  one-CTA launch, so a slow peer costs no SMs), then pull this rank's slice of
  the bucket from every rank, average in fp32, write ``out`` and add the
  squared norm to ``norm_acc`` ([0] tensor-parallel sharded part, [1]
  replicated part);
* ``adamw_ag(...)`` - AdamW on the slice with fp32 master weights, new 16-bit
  parameters stored straight into every rank's parameter buffer; the launch
  for the last bucket ends with the step barrier.

The reference leaves data parallelism to DeepSpeed ZeRO / Megatron DDP, i.e.
NCCL reduce-scatter + optimizer + NCCL all-gather as separate launches
(examples/utils.py:41-52 of the reference holds only the JSON knobs).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import native


class FusedDP:
    def __init__(self, ctx, total_elems: int, dtype, n_buckets: int, wait_seconds: float = 30.0):
        if dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("fused data parallelism needs 16-bit parameters")
        self.ctx = ctx
        self.world, self.rank = ctx.world, ctx.rank
        self.total, self.dtype, self.n_buckets = total_elems, dtype, n_buckets
        self.wait_seconds = wait_seconds
        nbytes = total_elems * 2
        self.grad_buf = ctx.buffer("dp_flat_grad", nbytes)
        self.param_buf = ctx.buffer("dp_flat_param", nbytes)
        self.flag_buf = ctx.buffer("dp_flags", (n_buckets + 1) * 8 * 4)
        self.flat_grad = self.grad_buf.view(dtype, (total_elems,))
        self.flat_param = self.param_buf.view(dtype, (total_elems,))
        self.flags = self.flag_buf.view(torch.int32, ((n_buckets + 1) * 8,))
        self.flags.zero_()
        self.flat_grad.zero_()
        device = self.flat_grad.device
        # epoch of the last reduce-scatter per bucket / of the last AdamW: the flag protocol
        # counts epochs upwards, a repeated or older epoch would find its flags already set
        # and read peers that are not ready (checked on the host, see _check_epoch)
        self._rs_epoch = [0] * n_buckets
        self._ag_epoch = 0
        self.norm_acc = torch.zeros(2, dtype=torch.float32, device=device)
        self.cta_counter = torch.zeros(1, dtype=torch.int32, device=device)
        from .symm import SymmContext

        if isinstance(ctx, SymmContext):   # every rank's flags are zero before anyone signals
            torch.cuda.synchronize(device)
            dist.barrier(group=ctx.group)

    # ------------------------------------------------------------------ #
    @staticmethod
    def _check_epoch(what, last, epoch):
        if epoch <= last:
            raise RuntimeError(
                f"{what}: epoch {epoch} after epoch {last}; every launch of a flag-synchronised "
                "kernel needs a larger epoch than the one before (a bucket reduced twice in "
                "one step, or a step counter that went backwards)")

    def grad_rs(self, bucket, epoch, lo, out, dup_mask=None, accumulate_norm=True, split=True):
        self._check_epoch(f"gradient reduce-scatter of bucket {bucket}", self._rs_epoch[bucket],
                          epoch)
        self._rs_epoch[bucket] = epoch
        ops = native.ops()
        args = (self.grad_buf.ptrs(), self.flag_buf.ptrs(), self.world, self.rank, bucket, epoch,
                lo, out, dup_mask, self.norm_acc if accumulate_norm else None, self.wait_seconds)
        if split:
            ops.dp_grad_rs(*args, 1)   # handshake, one small CTA
            ops.dp_grad_rs(*args, 2)   # pull + average + norm
        else:
            ops.dp_grad_rs(*args, 0)

    def adamw_ag(self, epoch, last, lo, grad, master, exp_avg, exp_avg_sq, decay_mask, grad_scale,
                 lr, betas, eps, weight_decay, bc1, bc2):
        if epoch < self._ag_epoch:     # one launch per bucket shares the step's epoch
            self._check_epoch("AdamW + parameter all-gather", self._ag_epoch, epoch)
        self._ag_epoch = epoch
        native.ops().dp_adamw_ag(
            self.param_buf.ptrs(), self.flag_buf.ptrs(), self.world, self.rank, self.n_buckets,
            epoch, bool(last), lo, grad, master, exp_avg, exp_avg_sq, decay_mask, grad_scale,
            lr, betas[0], betas[1], eps, weight_decay, bc1, bc2, self.cta_counter,
            self.wait_seconds)

    def take_norm_parts(self):
        """Squared-norm accumulators of this step (cleared for the next one)."""
        parts = self.norm_acc.clone()
        self.norm_acc.zero_()
        return parts
