"""The native training engine: what ``build(sch, target="native")`` returns.

It owns everything the reference leaves to DeepSpeed / Megatron:

* **flat storage** - all parameters live in one contiguous buffer per dtype
  (``p.data`` are views), gradients in a second one (``p.grad`` are views), so
  the optimizer, the gradient-norm and every data-parallel collective are a
  handful of launches over large 180-GB-class HBM buffers, never a Python
  loop over tensors;
* **mixed precision** - bf16 (or fp16/fp32) model parameters, fp32 master
  weights and Adam moments;
* **data parallelism, ZeRO-1 style** - the flat gradient buffer is cut into
  buckets in *reverse* registration order (the order backward produces
  them); as soon as a bucket's last gradient has been accumulated the bucket
  is reduce-scattered on a side stream, overlapping the rest of backward.
  Each data-parallel rank keeps master weights and moments only for its
  1/dp slice of every bucket, updates that slice with the fused AdamW kernel
  and all-gathers the updated parameters in place;
* **tensor / sequence parallel awareness** - gradients of parameters that
  are replicated over the TP group but computed from sequence-sharded
  activations (tagged ``replicated_param`` by the schedules) are all-reduced
  over the TP group; the global gradient norm counts TP-sharded parameters on
  every rank and replicated ones once;
* **device timing** - ``StepTimer`` brackets steps with CUDA events.

It runs on CPU ranks (gloo) too, with PyTorch ops instead of the kernels,
which is how the multi-rank logic is tested without GPUs.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist
from torch import nn

from ..logger import get_logger
from ..ops import native
from ..utils import nvtx

logger = get_logger("engine")


@dataclass
class EngineConfig:
    """Settings of the native engines (``build(..., target="native", config={...})``; a
    DeepSpeed-style dict with ``optimizer.params``, ``gradient_clipping``,
    ``gradient_accumulation_steps`` and an ``fp16`` block is accepted too).

    ``lr``, ``betas``, ``eps``, ``weight_decay`` - AdamW (biases and norm weights are not
    decayed); ``clip_grad`` - global gradient-norm limit over the whole model, 0 = off;
    ``zero`` - shard the optimizer state over the data-parallel group; ``bucket_mb``,
    ``overlap_comm`` - gradient buckets reduced during backward; ``grad_accum_steps`` -
    micro-batches per update; ``lr_schedule`` - ``callable(step) -> multiplier``;
    ``loss_scale``, ``initial_scale_power``, ``loss_scale_window``, ``min_loss_scale`` - fp16
    loss scaling (see the fields); ``profile`` - NVTX ranges and phase timers.  Keys the class
    does not know (``fused_dp``, ``p2p_mode``, ``prefetch_recv``, ...) are kept in ``extra``."""
    lr: float = 1e-4
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.01
    clip_grad: float = 1.0
    bucket_mb: float = 64.0        # DP reduce-scatter bucket (launch-latency sized, not link sized)
    zero: bool = True              # shard optimizer state over the DP group
    overlap_comm: bool = True
    grad_accum_steps: int = 1
    lr_schedule: object = None     # callable(step) -> lr multiplier
    # profile: NVTX ranges around the phases of every step and around the modules that the
    # schedule primitives created, plus device-timed phase durations (``phase_times()``);
    # costs one event pair per phase and no synchronisation
    profile: bool = False
    # fp16 loss scaling: None = dynamic when the parameters are fp16, off otherwise; 0 = dynamic;
    # > 0 = that fixed scale.  Dynamic: start at 2**initial_scale_power, halve (not below
    # min_loss_scale) and skip the update when a gradient overflowed, double after
    # loss_scale_window clean steps.
    loss_scale: float = None
    initial_scale_power: int = 16
    loss_scale_window: int = 1000
    min_loss_scale: float = 1.0
    extra: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, cfg):
        if cfg is None:
            return cls()
        if isinstance(cfg, cls):
            return cfg
        known = {f for f in cls.__dataclass_fields__}
        cfg = dict(cfg)
        # accept the DeepSpeed-style layout used by the reference examples
        opt = cfg.pop("optimizer", None)
        if isinstance(opt, dict):
            params = opt.get("params", {})
            for k in ("lr", "betas", "eps", "weight_decay"):
                if k in params:
                    cfg[k] = tuple(params[k]) if k == "betas" else params[k]
        fp16 = cfg.get("fp16")
        if isinstance(fp16, dict):      # DeepSpeed's block; "enabled" is the model's dtype here
            cfg.pop("fp16")
            for k in ("loss_scale", "initial_scale_power", "loss_scale_window", "min_loss_scale"):
                if k in fp16:
                    cfg.setdefault(k, fp16[k])
        if "gradient_clipping" in cfg:
            cfg["clip_grad"] = cfg.pop("gradient_clipping")
        if "gradient_accumulation_steps" in cfg:
            cfg["grad_accum_steps"] = cfg.pop("gradient_accumulation_steps")
        kwargs = {k: v for k, v in cfg.items() if k in known}
        extra = {k: v for k, v in cfg.items() if k not in known}
        return cls(**kwargs, extra=extra)


def _is_tp_sharded(p) -> bool:
    return hasattr(p, "orig_shape") and tuple(p.orig_shape) != tuple(p.shape)


class _Bucket:
    """A slice of the flat gradient buffer that is reduced as one unit.

    ``fired`` counts gradient-accumulation events of the bucket's parameters during the last
    backward of a step; ``expected`` is that count as calibrated on the first step (a module
    called several times under re-entrant checkpointing accumulates into its parameters once
    per call, so the number of parameters is not the right figure).  The bucket is reduced
    from the hook when ``fired`` reaches ``expected``; ``late`` records an accumulation that
    arrived after that launch."""
    __slots__ = ("start", "end", "n_params", "fired", "expected", "launched", "late", "deferred")

    def __init__(self, start):
        self.start, self.end = start, start
        self.n_params = 0
        self.fired = 0
        self.expected = None
        self.launched = False
        self.late = False
        self.deferred = False


def _release_staging_slots():
    """Staging slots of the pushed all-gather that a backward pass never released (an
    exception, a forward whose loss was dropped) go back to their pools; nothing of the
    previous batch is alive at this point."""
    from ..parallel import fused_tp

    fused_tp.step_boundary()


class TrainEngine:
    """See the module docstring.  ``engine(*inputs)`` runs the forward,
    ``engine.backward(loss)`` the backward, ``engine.step()`` the optimizer;
    ``engine.train_batch(*inputs, **kw)`` does all three and returns the loss."""

    def __init__(self, model: nn.Module, config=None, mesh=None, tp_group=None, dp_group=None,
                 loss_fn=None, dp_symm=None):
        self.model = model
        self.cfg = EngineConfig.from_dict(config)
        self.mesh = mesh
        self.tp_group = tp_group if tp_group is not None else (mesh.tp_group if mesh else None)
        self.dp_group = dp_group if dp_group is not None else (mesh.dp_group if mesh else None)
        self.tp_size = mesh.tp_size if mesh else (
            dist.get_world_size(tp_group) if tp_group is not None else 1)
        if mesh is not None:
            self.dp_size, self.dp_rank = mesh.dp_size, mesh.dp_rank
        elif dp_group is not None:
            self.dp_size, self.dp_rank = dist.get_world_size(dp_group), dist.get_rank(dp_group)
        else:
            self.dp_size, self.dp_rank = 1, 0
        self.loss_fn = loss_fn
        self.dp_symm = dp_symm      # symmetric-memory context of the DP group (made on demand)
        self._params_pushed = False
        self._hyper = None          # device {lr, bc1, bc2} while a captured step is in use
        self.fdp = None
        self.step_count = 0
        self.micro_step = 0
        self.last_grad_norm = None
        self.heartbeat = None       # runtime.health.Heartbeat, told about device-side give-ups
        self._final_backward = True   # the running backward is the last one before step()
        self._status_host = None      # pinned copy of the kernels' status word, one step behind
        self._status_event = None
        self._build_flat_storage()
        self._build_optimizer_state()
        self._install_grad_hooks()
        self._phase_events = []       # (name, start event, end event) of the last step
        if self.cfg.profile:
            nvtx.enable(True)
            n = nvtx.annotate_modules(self.model)
            logger.info("profile: NVTX ranges on %d scheduled modules and on the step phases", n,
                        ranks=0)

    # ------------------------------------------------------------------ #
    def _build_flat_storage(self):
        params, seen = [], set()
        for p in self.model.parameters():
            if p.requires_grad and id(p) not in seen:
                seen.add(id(p))
                params.append(p)
        if not params:
            raise ValueError("the model has no trainable parameter")
        if any(p.is_meta for p in params):
            raise RuntimeError("parameters are still on the meta device; build with init_weights")
        self.device = params[0].device
        self.param_dtype = params[0].dtype
        self._init_loss_scale()     # before the choice of the data-parallel path below
        if any(p.dtype != self.param_dtype for p in params):
            raise ValueError("all trainable parameters must share one dtype")
        # reverse registration order ~ the order in which backward finishes them
        self.params = list(reversed(params))
        # Parameters replicated over the tensor-parallel group whose gradients are partial sums
        # (sequence parallelism) go to the end of the flat buffer as one contiguous region in
        # buckets of their own, so that their gradient sync is ONE in-place all-reduce.
        n_rep = 0
        if self.tp_size > 1:
            rep = [p for p in self.params if getattr(p, "replicated_param", False)]
            n_rep = len(rep)
            if rep:
                self.params = [p for p in self.params
                               if not getattr(p, "replicated_param", False)] + rep
        first_rep = len(self.params) - n_rep
        align = 128 * max(self.dp_size, 1)  # elements; keeps every shard 256-byte aligned
        bucket_elems = max(int(self.cfg.bucket_mb * 2**20 / params[0].element_size()), align)
        self.buckets: list[_Bucket] = []
        self.param_slices = []
        offset = 0
        bucket = _Bucket(0)
        self.sp_region = None
        for i_p, p in enumerate(self.params):
            n = p.numel()
            padded = (n + 7) // 8 * 8
            new_region = n_rep > 0 and i_p == first_rep and bucket.end - bucket.start > 0
            if new_region or (bucket.end - bucket.start > 0
                              and (bucket.end - bucket.start) + padded > bucket_elems):
                offset = (offset + align - 1) // align * align
                bucket.end = offset
                self.buckets.append(bucket)
                bucket = _Bucket(offset)
            if n_rep > 0 and i_p == first_rep:
                self.sp_region = [offset, offset]
            self.param_slices.append((offset, n, len(self.buckets)))
            offset += padded
            bucket.end = offset
            bucket.n_params += 1
        offset = (offset + align - 1) // align * align
        bucket.end = offset
        self.buckets.append(bucket)
        self.total = offset
        if self.sp_region is not None:
            self.sp_region[1] = offset   # padding between parameters stays zero on every rank
            # summed over the tensor-parallel group in step() BEFORE the data-parallel
            # reduction: these buckets are never reduced from the backward hooks
            for b in self.buckets:
                if b.start >= self.sp_region[0]:
                    b.deferred = True
        if self._want_fused_dp():
            from ..parallel.fused_dp import FusedDP
            from ..parallel.symm import SymmContext

            ctx = self.dp_symm if self.dp_symm is not None else SymmContext(
                self.dp_group, device=self.device)
            self.fdp = FusedDP(ctx, self.total, self.param_dtype, len(self.buckets))
            self.flat_param, self.flat_grad = self.fdp.flat_param, self.fdp.flat_grad
            logger.info("data parallelism over peer memory: %d buckets, %.0f MiB of gradients",
                        len(self.buckets), self.total * 2 / 2**20, ranks=0)
        else:
            self.flat_param = torch.zeros(self.total, dtype=self.param_dtype, device=self.device)
            self.flat_grad = torch.zeros(self.total, dtype=self.param_dtype, device=self.device)
        self.sp_sync_params = []
        for p, (off, n, _) in zip(self.params, self.param_slices):
            view = self.flat_param[off:off + n].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.grad = self.flat_grad[off:off + n].view(p.shape)
            if getattr(p, "replicated_param", False) and self.tp_size > 1:
                self.sp_sync_params.append(p)
        self.n_params_local = sum(n for _, n, _ in self.param_slices)

    # ---- fp16 loss scaling --------------------------------------------- #
    def _init_loss_scale(self):
        """``self.loss_scale`` is the factor the loss is multiplied by before backward (a float;
        1.0 = off).  It changes only between steps, on the host, after the one synchronising
        read of the overflow flag that dynamic scaling needs per step."""
        want = self.cfg.loss_scale
        if want is None:
            self.dynamic_scale = self.param_dtype == torch.float16
            self.loss_scale = 2.0 ** self.cfg.initial_scale_power if self.dynamic_scale else 1.0
        elif want == 0:
            self.dynamic_scale = True
            self.loss_scale = 2.0 ** self.cfg.initial_scale_power
        else:
            self.dynamic_scale = False
            self.loss_scale = float(want)
        self.scaling = self.dynamic_scale or self.loss_scale != 1.0
        self._clean_steps = 0
        self.skipped_steps = 0

    def scale_loss(self, loss):
        """The loss as it goes into backward (the pipeline engine scales its last stage's loss
        with this as well)."""
        return loss * self.loss_scale if self.scaling else loss

    def _update_loss_scale(self, overflow: bool):
        if not self.dynamic_scale:
            return
        if overflow:
            self.loss_scale = max(self.loss_scale / 2.0, float(self.cfg.min_loss_scale))
            self._clean_steps = 0
            return
        self._clean_steps += 1
        if self._clean_steps >= self.cfg.loss_scale_window:
            self.loss_scale *= 2.0
            self._clean_steps = 0

    def _want_fused_dp(self):
        """ZeRO-1 over NVLink peer memory instead of NCCL: CUDA, 16-bit parameters, a
        data-parallel group of 2..8 ranks on this node, not switched off by ``fused_dp=False``."""
        if not (self.cfg.zero and 1 < self.dp_size <= 8 and self.device.type == "cuda"):
            return False
        if not self.cfg.extra.get("fused_dp", True) or not native.available():
            return False
        if self.scaling:
            # a step skipped after an overflow must not advance the optimizer, but the peer
            # kernels' hand-shake epochs advance with the step count: NCCL path under scaling
            return False
        if self.param_dtype not in (torch.bfloat16, torch.float16):
            return False
        return hasattr(torch.ops.slapo_b200, "dp_grad_rs")

    def _shard_range(self, bucket):
        if not (self.cfg.zero and self.dp_size > 1):
            return bucket.start, bucket.end
        per = (bucket.end - bucket.start) // self.dp_size
        lo = bucket.start + self.dp_rank * per
        return lo, lo + per

    def _sync_initial_params(self):
        """Data-parallel replicas start from the first replica's parameters.  Replicas that were
        initialised on their own (meta-device build with per-replica seeds) would otherwise
        differ until the first optimizer step mixes their shards - and for good without ZeRO."""
        if self.dp_size > 1 and self.dp_group is not None:
            dist.broadcast(self.flat_param, src=dist.get_global_rank(self.dp_group, 0),
                           group=self.dp_group)

    def _build_optimizer_state(self):
        self._sync_initial_params()
        # this rank's slice of every bucket, packed back to back
        self.shard_ranges = [self._shard_range(b) for b in self.buckets]
        n_own = sum(hi - lo for lo, hi in self.shard_ranges)
        self.master = torch.empty(n_own, dtype=torch.float32, device=self.device)
        self.exp_avg = torch.zeros(n_own, dtype=torch.float32, device=self.device)
        self.exp_avg_sq = torch.zeros(n_own, dtype=torch.float32, device=self.device)
        self.grad_shard = None
        if self.cfg.zero and self.dp_size > 1:
            self.grad_shard = torch.zeros(n_own, dtype=self.param_dtype, device=self.device)
        self.shard_offsets = []
        pos = 0
        for lo, hi in self.shard_ranges:
            self.master[pos:pos + hi - lo].copy_(self.flat_param[lo:hi])
            self.shard_offsets.append(pos)
            pos += hi - lo
        # weight-decay mask: no decay for 1-D tensors (biases, norm weights)
        self.decay_mask = None
        wd_flat = torch.zeros(self.total, dtype=torch.bool, device=self.device)
        for p, (off, n, _) in zip(self.params, self.param_slices):
            if p.dim() > 1 and not getattr(p, "no_weight_decay", False):
                wd_flat[off:off + n] = True
        self.decay_mask = torch.cat([wd_flat[lo:hi] for lo, hi in self.shard_ranges]).to(torch.uint8)
        self._norm_skip = set()
        self._build_norm_classes()
        self.comm_stream = torch.cuda.Stream() if self.device.type == "cuda" else None

    def _build_norm_classes(self):
        """Per-element class of this rank's gradient slices for the global norm: 0 = counted on
        every tensor-parallel rank (sharded parameters), 1 = replicated over the tensor-parallel
        group (counted once), 2 = not counted here (a parameter tied across pipeline stages is
        counted by the first stage that owns it)."""
        self.tp_dup_mask = None
        self.tp_dup_mask_u8 = None
        if self.tp_size <= 1 and not self._norm_skip:
            return
        cls = torch.zeros(self.total, dtype=torch.uint8, device=self.device)
        for p, (off, n, _) in zip(self.params, self.param_slices):
            if id(p) in self._norm_skip:
                cls[off:off + n] = 2
            elif self.tp_size > 1 and not _is_tp_sharded(p):
                cls[off:off + n] = 1
        self.tp_dup_mask_u8 = torch.cat([cls[lo:hi] for lo, hi in self.shard_ranges])
        self.tp_dup_mask = self.tp_dup_mask_u8

    def exclude_from_norm(self, params):
        """Leave ``params`` out of this rank's share of the gradient norm."""
        self._norm_skip |= {id(p) for p in params}
        self._build_norm_classes()

    def _install_grad_hooks(self):
        # on CPU ranks the reduction of a bucket runs synchronously inside the hook; that mode
        # exists to test the hook logic without GPUs (``overlap_on_cpu`` in the config)
        self._overlap = (self.cfg.overlap_comm and self.dp_size > 1 and
                         (self.device.type == "cuda" or bool(self.cfg.extra.get("overlap_on_cpu"))))
        if not self._overlap:
            return
        for p, (_, _, b_idx) in zip(self.params, self.param_slices):
            p.register_post_accumulate_grad_hook(self._make_hook(b_idx))

    def _make_hook(self, b_idx):
        def hook(_param):
            if not self._final_backward:
                return
            bucket = self.buckets[b_idx]
            bucket.fired += 1
            if bucket.launched:
                bucket.late = True      # dealt with in step()
            elif (bucket.expected is not None and not bucket.deferred
                  and bucket.fired == bucket.expected):
                self._launch_bucket_reduce(b_idx)

        return hook

    def set_final_backward(self, flag: bool):
        """Tell the overlap hooks whether the backward about to run is the last one before
        ``step()``.  ``backward()`` does it from the accumulation counter; a caller that drives
        autograd itself (the pipeline engine: one backward per micro-batch) sets it by hand."""
        self._final_backward = bool(flag)

    def defer_params(self, params):
        """Never reduce the buckets of ``params`` from the hooks: their gradients are still
        modified after backward (parameters tied across pipeline stages)."""
        ids = {id(p) for p in params}
        for p, (_, _, b_idx) in zip(self.params, self.param_slices):
            if id(p) in ids:
                self.buckets[b_idx].deferred = True

    # ------------------------------------------------------------------ #
    def _launch_bucket_reduce(self, b_idx):
        bucket = self.buckets[b_idx]
        grad = self.flat_grad[bucket.start:bucket.end]
        if self.comm_stream is not None:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            ctx = torch.cuda.stream(self.comm_stream)
        else:
            import contextlib

            ctx = contextlib.nullcontext()
        with ctx, nvtx.range(f"slapo_b200.dp_reduce.bucket{b_idx}"):
            if self.fdp is not None:
                pos = self.shard_offsets[b_idx]
                lo, hi = self.shard_ranges[b_idx]
                mask = self.tp_dup_mask_u8[pos:pos + hi - lo] if self.tp_dup_mask is not None else None
                self.fdp.grad_rs(b_idx, self.step_count + 1, lo, self.grad_shard[pos:pos + hi - lo],
                                 mask)
            elif self.cfg.zero:
                pos = self.shard_offsets[b_idx]
                lo, hi = self.shard_ranges[b_idx]
                out = self.grad_shard[pos:pos + hi - lo]
                dist.reduce_scatter_tensor(out, grad, op=dist.ReduceOp.AVG
                                           if self.device.type == "cuda" else dist.ReduceOp.SUM,
                                           group=self.dp_group)
                if self.device.type != "cuda":
                    out.div_(self.dp_size)
            else:
                dist.all_reduce(grad, group=self.dp_group)
                grad.div_(self.dp_size)
        bucket.launched = True

    def _reduce_all_buckets(self):
        for i, bucket in enumerate(self.buckets):
            if bucket.launched and bucket.late:
                # A gradient was accumulated after the bucket had been reduced from its hook
                # (the autograd graph differs from the calibrated step).  Reduce-scatter
                # leaves the flat gradient untouched, so it can simply run again; the in-place
                # all-reduce and the peer-memory kernels (one launch per step epoch) cannot.
                if self.fdp is None and self.cfg.zero:
                    bucket.launched = False
                else:
                    raise RuntimeError(
                        "a gradient arrived after its bucket had been reduced during backward "
                        "(the set of gradient accumulations changed between steps); build the "
                        "engine with overlap_comm=False for models whose graph varies")
            if not bucket.launched:
                self._launch_bucket_reduce(i)
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        for bucket in self.buckets:
            if self._overlap and bucket.fired and bucket.expected != bucket.fired:
                bucket.expected = bucket.fired     # first step, or the graph changed
            bucket.fired = 0
            bucket.launched = False
            bucket.late = False

    # ------------------------------------------------------------------ #
    def __call__(self, *args, **kwargs):
        return self.model(*args, **kwargs)

    def backward(self, loss):
        if self.cfg.grad_accum_steps > 1:
            loss = loss / self.cfg.grad_accum_steps
        self._final_backward = (self.micro_step + 1) % self.cfg.grad_accum_steps == 0
        loss = self.scale_loss(loss)
        loss.backward()
        self.micro_step += 1

    def _own_grad(self):
        """This rank's reduced gradient slice as one flat view list."""
        if self.grad_shard is not None:
            return self.grad_shard
        if len(self.shard_ranges) == 1 or not (self.cfg.zero and self.dp_size > 1):
            return self.flat_grad  # ranges cover the whole buffer back to back
        return torch.cat([self.flat_grad[lo:hi] for lo, hi in self.shard_ranges])

    def _grad_norm(self, grad):
        if (self.device.type == "cuda" and native.available() and grad.numel() % 8 == 0
                and hasattr(torch.ops.slapo_b200, "sq_norm")):
            # one streaming pass; [0] = TP-sharded part, [1] = replicated part
            mask = self.tp_dup_mask_u8 if self.tp_dup_mask is not None else None
            parts = native.ops().sq_norm(grad, mask)
            return self._finish_norm(parts)
        g = grad.float()
        if self.tp_dup_mask is not None:
            cls = self.tp_dup_mask
            sq_shard = (g * (cls == 0)).pow(2).sum()
            sq_dup = (g * (cls == 1)).pow(2).sum()
            parts = torch.stack([sq_shard, sq_dup])
        else:
            parts = torch.stack([g.pow(2).sum(), torch.zeros((), device=g.device)])
        return self._finish_norm(parts)

    def _finish_norm(self, parts):
        if self.cfg.zero and self.dp_size > 1:
            dist.all_reduce(parts, group=self.dp_group)
        if self.tp_size > 1:
            shard_part = parts[0:1].clone()
            dist.all_reduce(shard_part, group=self.tp_group)
            total = shard_part[0] + parts[1]
        else:
            total = parts[0] + parts[1]
        if self.mesh is not None and self.mesh.pp_size > 1 and self.mesh.pp_group is not None:
            # one norm for the whole model: the stages add up their parts
            total = total.reshape(1).clone()
            dist.all_reduce(total, group=self.mesh.pp_group)
            total = total[0]
        return total.sqrt()

    def step(self):
        """Synchronise gradients, clip, AdamW-update, re-gather parameters."""
        if self.micro_step % self.cfg.grad_accum_steps != 0:
            return False
        # sequence-parallel: replicated parameters got partial gradients; they are one
        # contiguous region of the flat gradient buffer, summed in place
        if self.sp_sync_params:
            lo, hi = self.sp_region
            dist.all_reduce(self.flat_grad[lo:hi], group=self.tp_group)
        if self.dp_size > 1:
            self._reduce_all_buckets()
        grad = self._own_grad()
        clip_coef = None
        clipping = bool(self.cfg.clip_grad and self.cfg.clip_grad > 0)
        if clipping or self.scaling:
            # the fused reduce-scatter kernels already accumulated the squared norm
            norm = self._finish_norm(self.fdp.take_norm_parts()) if self.fdp is not None \
                else self._grad_norm(grad)
            if self.scaling:
                # the norm is the same on every rank of the job (summed over the tensor-,
                # data- and pipeline-parallel groups), so every rank takes the same branch
                overflow = not bool(torch.isfinite(norm))
                scale_used = self.loss_scale        # the gradients in the buffers carry this one
                self._update_loss_scale(overflow)
                if overflow:
                    self.skipped_steps += 1
                    self.flat_grad.zero_()
                    if self.grad_shard is not None:
                        self.grad_shard.zero_()
                    logger.info("gradient overflow: step skipped, loss scale now %g",
                                self.loss_scale, ranks=0)
                    return False
                norm = norm / scale_used
            self.last_grad_norm = norm
            if clipping:
                clip_coef = torch.clamp(self.cfg.clip_grad / (norm + 1e-6), max=1.0)
            if self.scaling:
                unscale = torch.full((), 1.0 / scale_used, device=norm.device)
                clip_coef = unscale if clip_coef is None else clip_coef * unscale
        self.step_count += 1
        lr = self.cfg.lr
        if self.cfg.lr_schedule is not None:
            lr = lr * self.cfg.lr_schedule(self.step_count)
        self._adamw(grad, lr, clip_coef)
        self._params_pushed = self.fdp is not None
        self._gather_params()
        self.flat_grad.zero_()
        self._poll_device_status()
        return True

    # ---- device status (bounded waits of the peer-memory kernels) -------- #
    def _watches_status(self):
        return (self.device.type == "cuda" and native.available()
                and (self.tp_size > 1 or self.dp_size > 1 or self.mesh is not None))

    def _raise_device_status(self, code):
        native.ops().device_status()     # reads and clears the word
        msg = (f"device status {code} after step {self.step_count}: a bounded wait on a peer ran "
               "out inside a fused kernel (a rank is missing, stuck or more than the wait limit "
               "behind); the outputs of that step are not valid")
        if self.heartbeat is not None:
            self.heartbeat.report_failure(msg)
        raise RuntimeError(msg)

    def _poll_device_status(self):
        """Once per step, without a device synchronisation: the status word of the step that
        just ended is copied to pinned memory behind the step's work, and the copy made at the
        end of the PREVIOUS step - long complete by now - is examined.  A give-up is therefore
        reported one step late; ``check_device_status()`` closes that gap at the end of a run."""
        if not self._watches_status() or torch.cuda.is_current_stream_capturing():
            return
        if self._status_event is None:
            self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._status_event = torch.cuda.Event()
        else:
            self._status_event.synchronize()
            code = int(self._status_host[0])
            if code:
                self._raise_device_status(code)
        self._status_host.copy_(native.ops().device_status_tensor()[:1], non_blocking=True)
        self._status_event.record()

    def check_device_status(self):
        """Synchronise and raise if any kernel of this device gave up a bounded wait."""
        if not self._watches_status():
            return
        code = int(native.ops().device_status())
        if code:
            self._raise_device_status(code)

    def _adamw(self, grad, lr, clip_coef):
        b1, b2 = self.cfg.betas
        t = self.step_count
        bc1, bc2 = 1 - b1**t, 1 - b2**t
        contiguous_owner = not (self.cfg.zero and self.dp_size > 1)
        if self.fdp is not None:
            coef = (clip_coef if clip_coef is not None
                    else torch.ones((), device=self.device)).float().reshape(1)
            last_idx = len(self.shard_ranges) - 1
            for idx, ((lo, hi), pos) in enumerate(zip(self.shard_ranges, self.shard_offsets)):
                n = hi - lo
                self.fdp.adamw_ag(
                    self.step_count, idx == last_idx, lo, grad[pos:pos + n],
                    self.master[pos:pos + n], self.exp_avg[pos:pos + n],
                    self.exp_avg_sq[pos:pos + n], self.decay_mask[pos:pos + n], coef, lr,
                    (b1, b2), self.cfg.eps, self.cfg.weight_decay, bc1, bc2)
            return
        if self.device.type == "cuda" and native.available() and hasattr(
                torch.ops.slapo_b200, "fused_adamw"):
            coef = clip_coef if clip_coef is not None else torch.ones((), device=self.device)
            if contiguous_owner:
                native.ops().fused_adamw(self.flat_param, grad, self.master, self.exp_avg,
                                         self.exp_avg_sq, self.decay_mask, coef.float().reshape(1),
                                         lr, b1, b2, self.cfg.eps, self.cfg.weight_decay, bc1, bc2,
                                         self._hyper)
            else:
                for (lo, hi), pos in zip(self.shard_ranges, self.shard_offsets):
                    n = hi - lo
                    native.ops().fused_adamw(
                        self.flat_param[lo:hi], grad[pos:pos + n], self.master[pos:pos + n],
                        self.exp_avg[pos:pos + n], self.exp_avg_sq[pos:pos + n],
                        self.decay_mask[pos:pos + n], coef.float().reshape(1), lr, b1, b2,
                        self.cfg.eps, self.cfg.weight_decay, bc1, bc2)
            return
        g = grad.float()
        if clip_coef is not None:
            g = g * clip_coef
        self.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
        denom = (self.exp_avg_sq / bc2).sqrt_().add_(self.cfg.eps)
        update = (self.exp_avg / bc1) / denom
        update.add_(self.master * self.decay_mask, alpha=self.cfg.weight_decay)
        self.master.add_(update, alpha=-lr)
        for (lo, hi), pos in zip(self.shard_ranges, self.shard_offsets):
            self.flat_param[lo:hi].copy_(self.master[pos:pos + hi - lo])

    def _gather_params(self):
        if not (self.cfg.zero and self.dp_size > 1):
            return
        if self.fdp is not None and self._params_pushed:
            self._params_pushed = False   # the fused AdamW kernel stored them on every rank
            return
        for bucket, (lo, hi) in zip(self.buckets, self.shard_ranges):
            full = self.flat_param[bucket.start:bucket.end]
            if self.device.type == "cuda":
                dist.all_gather_into_tensor(full, self.flat_param[lo:hi], group=self.dp_group)
            else:
                dist.all_gather_into_tensor(full, self.flat_param[lo:hi].clone(), group=self.dp_group)

    # ------------------------------------------------------------------ #
    def _phase(self, name):
        """Context manager of one step phase: an NVTX range and, with ``profile``, a pair of
        CUDA events whose distance ``phase_times()`` reports (never synchronises here)."""
        import contextlib

        @contextlib.contextmanager
        def ctx():
            timed = self.cfg.profile and self.device.type == "cuda" \
                and not torch.cuda.is_current_stream_capturing()
            if timed:
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
            with nvtx.range(f"slapo_b200.{name}"):
                yield
            if timed:
                end.record()
                self._phase_events.append((name, start, end))

        return ctx()

    def phase_times(self):
        """``{"forward": ms, "backward": ms, "optimizer": ms}`` of the last profiled step
        (device time between the phase's events; synchronises on the last one).  Empty unless
        the engine was built with ``profile=True`` on a CUDA device."""
        out = {}
        for name, start, end in self._phase_events:
            end.synchronize()
            out[name] = out.get(name, 0.0) + start.elapsed_time(end)
        return out

    def train_batch(self, *args, labels=None, **kwargs):
        if self.micro_step % self.cfg.grad_accum_steps == 0:
            self._phase_events = []
        _release_staging_slots()
        with self._phase("forward"):
            out = self.model(*args, **kwargs)
            if self.loss_fn is not None:
                loss = self.loss_fn(out, labels)
            elif torch.is_tensor(out):
                loss = out
            elif isinstance(out, dict):
                loss = out["loss"]
            else:
                loss = out[0]
            if loss.dim() > 0:
                loss = loss.float().mean()
        with self._phase("backward"):
            self.backward(loss)
        with self._phase("optimizer"):
            self.step()
        return loss.detach()

    # ---- checkpoint support ------------------------------------------ #
    def optimizer_state(self):
        return {"step": self.step_count, "master": self.master, "exp_avg": self.exp_avg,
                "exp_avg_sq": self.exp_avg_sq, "shard_ranges": list(self.shard_ranges),
                "dp_size": self.dp_size, "dp_rank": self.dp_rank, "zero": self.cfg.zero,
                "loss_scale": self.loss_scale, "clean_steps": self._clean_steps}

    def load_optimizer_state(self, state):
        self.step_count = int(state["step"])
        if self.scaling and "loss_scale" in state:
            self.loss_scale = float(state["loss_scale"])
            self._clean_steps = int(state.get("clean_steps", 0))
        for key in ("master", "exp_avg", "exp_avg_sq"):
            getattr(self, key).copy_(state[key])
        for (lo, hi), pos in zip(self.shard_ranges, self.shard_offsets):
            self.flat_param[lo:hi].copy_(self.master[pos:pos + hi - lo])
        self._gather_params()

    def _param_names(self):
        names = {}
        for name, p in self.model.named_parameters():
            names.setdefault(id(p), name)
        return [names[id(p)] for p in self.params]

    def _gather_flat_state(self, own: torch.Tensor) -> torch.Tensor:
        """This rank's packed optimizer slices -> the whole flat fp32 vector
        (all-gathered bucket by bucket under ZeRO)."""
        flat = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        sharded = self.cfg.zero and self.dp_size > 1
        for bucket, (lo, hi), pos in zip(self.buckets, self.shard_ranges, self.shard_offsets):
            piece = own[pos:pos + hi - lo]
            if sharded:
                dist.all_gather_into_tensor(flat[bucket.start:bucket.end], piece.contiguous(),
                                            group=self.dp_group)
            else:
                flat[lo:hi].copy_(piece)
        return flat

    def full_optimizer_state(self, to_cpu=True):
        """Optimizer state keyed by parameter name, each tensor in the local
        (tensor-parallel shard) shape of its parameter - the layout-free form
        that checkpoints store, so that a run with another DP size, bucket size
        or ZeRO setting can resume from it.  Collective over the DP group."""
        out = {"step": self.step_count, "state": {}}
        names = self._param_names()
        for key in ("master", "exp_avg", "exp_avg_sq"):
            flat = self._gather_flat_state(getattr(self, key))
            for name, p, (off, n, _) in zip(names, self.params, self.param_slices):
                t = flat[off:off + n].view(p.shape)
                out["state"].setdefault(name, {})[key] = t.cpu() if to_cpu else t.clone()
            del flat
        return out

    def load_full_optimizer_state(self, full):
        """Inverse of :meth:`full_optimizer_state`; parameters missing from
        ``full`` keep a fresh state (master = current weights, moments = 0)."""
        self.step_count = int(full.get("step", 0))
        names = self._param_names()
        for key in ("master", "exp_avg", "exp_avg_sq"):
            flat = torch.zeros(self.total, dtype=torch.float32, device=self.device)
            if key == "master":
                flat.copy_(self.flat_param)
            for name, p, (off, n, _) in zip(names, self.params, self.param_slices):
                entry = full["state"].get(name)
                if entry is None or key not in entry:
                    continue
                src = entry[key]
                if tuple(src.shape) != tuple(p.shape):
                    raise ValueError(f"optimizer state of {name}: shape {tuple(src.shape)} does "
                                     f"not match the parameter's {tuple(p.shape)}")
                flat[off:off + n].copy_(src.reshape(-1))
            own = getattr(self, key)
            for (lo, hi), pos in zip(self.shard_ranges, self.shard_offsets):
                own[pos:pos + hi - lo].copy_(flat[lo:hi])
            del flat
        for (lo, hi), pos in zip(self.shard_ranges, self.shard_offsets):
            self.flat_param[lo:hi].copy_(self.master[pos:pos + hi - lo])
        self._gather_params()

    # ---- CUDA graph of the whole step ------------------------------------ #
    def _hyper_values(self, step):
        lr = self.cfg.lr
        if self.cfg.lr_schedule is not None:
            lr = lr * self.cfg.lr_schedule(step)
        b1, b2 = self.cfg.betas
        return [lr, 1 - b1**step, 1 - b2**step]

    def capture_step(self, *example_inputs, labels=None, warmup=3, **kwargs):
        """Capture forward + backward + optimizer of one step in a CUDA graph and return a
        ``GraphedStep``: ``graphed(*inputs, labels=...)`` copies the batch into the static input
        buffers, refreshes the step-dependent optimizer scalars in device memory and replays
        the graph - one launch instead of ~1500, which removes the host-side launch cost of
        the step.  Single-process engines only (no DP / TP collectives inside the step), fixed
        shapes; dropout is advanced per replay by the generator's graph-safe Philox offset.
        ``warmup`` eager steps run first (they train like ordinary steps)."""
        if self.device.type != "cuda":
            raise RuntimeError("CUDA graphs need a CUDA device")
        if self.dp_size > 1 or self.tp_size > 1:
            raise RuntimeError("capture_step supports single-process engines only")
        if self.cfg.grad_accum_steps != 1:
            raise RuntimeError("capture_step needs grad_accum_steps == 1")
        if self.scaling:
            raise RuntimeError("capture_step does not support fp16 loss scaling (the overflow "
                               "check decides on the host whether the update runs); use bf16")
        static_in = [t.clone() if torch.is_tensor(t) else t for t in example_inputs]
        static_labels = labels.clone() if torch.is_tensor(labels) else labels
        self._hyper = torch.zeros(3, dtype=torch.float32, device=self.device)
        host = torch.zeros(3, dtype=torch.float32).pin_memory()

        def set_hyper(step):
            host.copy_(torch.tensor(self._hyper_values(step)))
            self._hyper.copy_(host, non_blocking=True)

        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                set_hyper(self.step_count + 1)
                self.train_batch(*static_in, labels=static_labels, **kwargs)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        launches0 = native.launch_count()
        set_hyper(self.step_count + 1)
        torch.cuda.synchronize(self.device)
        with torch.cuda.graph(graph):
            static_loss = self.train_batch(*static_in, labels=static_labels, **kwargs)
        launches = native.launch_count() - launches0
        # the capture itself executed nothing: train_batch counted a step that did not happen
        self.step_count -= 1
        return GraphedStep(self, graph, static_in, static_labels, static_loss, set_hyper, launches)

    def refresh_master_from_params(self):
        """After loading model weights into ``p.data``: re-seed the fp32 master."""
        for (lo, hi), pos in zip(self.shard_ranges, self.shard_offsets):
            self.master[pos:pos + hi - lo].copy_(self.flat_param[lo:hi])


class GraphedStep:
    """A captured training step (see :meth:`TrainEngine.capture_step`)."""

    def __init__(self, engine, graph, static_in, static_labels, static_loss, set_hyper, launches):
        self.engine, self.graph = engine, graph
        self.static_in, self.static_labels, self.static_loss = static_in, static_labels, static_loss
        self._set_hyper = set_hyper
        self.kernels_per_step = int(launches)   # launches of this library's kernels in the graph

    def __call__(self, *inputs, labels=None):
        for dst, src in zip(self.static_in, inputs):
            if torch.is_tensor(dst) and src is not dst:
                dst.copy_(src, non_blocking=True)
        if torch.is_tensor(self.static_labels) and labels is not None \
                and labels is not self.static_labels:
            self.static_labels.copy_(labels, non_blocking=True)
        self.engine.step_count += 1
        self._set_hyper(self.engine.step_count)
        self.graph.replay()
        return self.static_loss


class StepTimer:
    """Device-side step timing: CUDA events on the current stream (wall
    clock on CPU); ``max_over_ranks`` reduces with MAX over a group."""

    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        self.t0 = self.t1 = None

    def start(self):
        if self.cuda:
            torch.cuda.synchronize()
            self.t0 = torch.cuda.Event(enable_timing=True)
            self.t1 = torch.cuda.Event(enable_timing=True)
            self.t0.record()
        else:
            import time

            self.t0 = time.perf_counter()

    def stop(self) -> float:
        """Elapsed milliseconds."""
        if self.cuda:
            self.t1.record()
            torch.cuda.synchronize()
            return self.t0.elapsed_time(self.t1)
        import time

        return (time.perf_counter() - self.t0) * 1e3

    @staticmethod
    def max_over_ranks(ms: float, device, group=None) -> float:
        if not (dist.is_available() and dist.is_initialized()):
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return float(t.item())
