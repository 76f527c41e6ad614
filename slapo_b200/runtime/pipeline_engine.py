"""Pipeline-parallel runtime: stage wrappers and the 1F1B engine.

``build(sch, target="native", mesh=..., loss_fn=...)`` on a schedule with
``cut_pipeline_stage`` marks returns a :class:`PipelineEngine`.  Each rank
along the mesh's ``pp`` axis owns one stage module.  ``train_batch`` splits the
global batch into micro-batches and runs the one-forward-one-backward schedule:
``P - 1 - stage`` warm-up forwards, then alternating forward / backward, then
the remaining backwards, so that at most ``P - stage`` micro-batches are alive
per stage.

Stage boundaries are described statically (``live_in`` of
:func:`slapo_b200.parallel.pipeline_partition.analyze_pipeline_module`): the
ordered value names that cross each boundary.  Shapes and dtypes are exchanged
ONCE, with the first micro-batch; afterwards only tensors move.

Transfers overlap compute.  Every pipeline link has one 2-rank process group per
direction (``DeviceMesh.p2p_groups``): on GPUs that is one NCCL communicator
with its own stream for the activations going down and another for the
gradients coming back.  Receives are posted one micro-batch ahead (the input
of micro-batch i + 1 and the output gradient of the oldest micro-batch in
flight are on the wire while micro-batch i computes) and waited for only where
the tensor is consumed; sends are never waited for until the end of the batch
(the Work objects keep the tensors alive).  ``Work.wait()`` on NCCL makes the
compute stream wait, not the host, so the host runs ahead and keeps both
queues full.  On CPU ranks (gloo) the same code runs with host-blocking waits.

Next to the fused tensor-parallel kernels (tensor parallelism on GPUs) the engine runs the
PAIRED schedule instead (``p2p_mode``): every exchange with a neighbour is one batched
send + receive group that the compute stream waits for.  Those kernels are persistent and
need every SM; an NCCL kernel that sits on a few SMs until its peer arrives can keep one of
them from becoming resident, and with receives posted ahead the peer may be waiting for
exactly that kernel (a 2-stage x 4-way run stopped that way).
The reference delegates all of this to DeepSpeed's ``PipelineModule``, which
exchanges blocking send / recv pairs and re-decodes a metadata tensor on the
host for every micro-batch
(slapo/framework_dialect/deepspeed/pipeline.py:205-354).

Parameters shared by two stages (tied embeddings) get their gradients summed
over the owning stages before the optimizer step.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn
from torch.utils._pytree import tree_flatten, tree_unflatten

from ..logger import get_logger
from .engine import EngineConfig, TrainEngine

logger = get_logger("pipeline_engine")


def _dense_like(t):
    """A contiguous receive buffer of ``t``'s shape (``empty_like`` keeps the strides of a
    permuted tensor - a relative-position bias, say - and p2p receives need dense memory)."""
    return torch.empty(t.shape, dtype=t.dtype, device=t.device)


class PipelineStage(nn.Module):
    """One stage: maps value names to the stage module's arguments and back."""

    def __init__(self, module, index, n_stages, input_names, output_names, constants=None):
        super().__init__()
        self.module = module
        self.index, self.n_stages = index, n_stages
        self.input_names = list(input_names)
        self.output_names = list(output_names)
        # buffers / parameters that the split left at the top level (for example a
        # position-id table read by the first stage): owned by the stage that reads them
        self.const_names = {}
        for name, value in (constants or {}).items():
            attr = f"const_{name}"
            if isinstance(value, nn.Parameter):
                self.register_parameter(attr, value)
            else:
                self.register_buffer(attr, value, persistent=False)
            self.const_names[name] = attr

    def _value(self, env, name):
        if name in self.const_names and name not in env:
            return getattr(self, self.const_names[name])
        return env[name]

    def forward(self, env: dict):
        out = self.module(*[self._value(env, n) for n in self.input_names])
        produced = {}
        for name, idx in self.output_names:
            produced[name] = out if idx is None else out[idx]
        return produced


class PipelineModel(nn.Module):
    """All stages plus the boundary contract; runs them in sequence when called
    directly (single process, e.g. for verification)."""

    def __init__(self, stages, live_in, input_names, output_spec, input_hooks=()):
        super().__init__()
        self.stages = nn.ModuleList(stages)
        self.live_in = [list(x) for x in live_in]
        self.input_names = list(input_names)
        self.output_spec = output_spec
        # forward-pre hooks of the unpartitioned model (``sync("fwd_pre", fn)`` on the top
        # schedule): run over the model's inputs, in declaration order, where they enter
        self.input_hooks = list(input_hooks)

    def materialize_output(self, env):
        def pick(x):
            if isinstance(x, str):
                return env[x]
            if isinstance(x, dict):
                return {k: pick(v) for k, v in x.items()}
            if isinstance(x, (tuple, list)):
                return type(x)(pick(v) for v in x)
            return x

        return pick(self.output_spec)

    def bind_inputs(self, args, kwargs, run_hooks=True):
        env = dict(zip(self.input_names, args))
        env.update(kwargs)
        for name in self.input_names:
            env.setdefault(name, None)
        if run_hooks:
            for hook in self.input_hooks:
                result = hook(self, tuple(env[n] for n in self.input_names))
                if result is not None:
                    result = result if isinstance(result, tuple) else (result,)
                    env.update(zip(self.input_names, result))
        return env

    def forward(self, *args, **kwargs):
        env = self.bind_inputs(args, kwargs)
        for stage in self.stages:
            env.update(stage(env))
        return self.materialize_output(env)


def _split_micro(t, m):
    if torch.is_tensor(t) and t.dim() > 0:
        return list(t.chunk(m, dim=0))
    return [t] * m


class PipelineEngine:
    def __init__(self, model: PipelineModel, config=None, mesh=None, loss_fn=None, tp_group=None,
                 num_micro_batches=None, **_unused):
        if mesh is None:
            raise ValueError("the pipeline engine needs mesh=DeviceMesh(pp=..., dp=..., tp=...)")
        self.model = model
        self.mesh = mesh
        self.cfg = EngineConfig.from_dict(config)
        self.loss_fn = loss_fn
        self.stage_id = mesh.pp_rank
        self.n_stages = mesh.pp_size
        if self.n_stages != len(model.stages):
            raise ValueError(f"{len(model.stages)} stages were cut but the mesh has pp={self.n_stages}")
        self.stage = model.stages[self.stage_id]
        self.num_micro_batches = num_micro_batches or self.cfg.extra.get("num_micro_batches") \
            or self.n_stages
        self.prev_rank, self.next_rank = mesh.prev_stage_rank(), mesh.next_stage_rank()
        self.device = next(self.stage.parameters()).device
        self.inner = TrainEngine(self.stage, config=self.cfg, mesh=mesh, tp_group=tp_group,
                                 dp_group=mesh.dp_group)
        self.inner.cfg.grad_accum_steps = 1
        self._meta_fwd = None   # [(name, tree spec, per-leaf description)] of live_in[stage]
        self._meta_sent = False
        self._inflight = []     # Work objects of sends not yet waited for
        # Receives are posted one micro-batch ahead unless the stage runs the fused
        # tensor-parallel kernels.  Those are persistent kernels that need every SM (one CTA
        # each, all of them waiting on each other and on the peers); a receive posted ahead
        # is an NCCL kernel that sits on some SMs until its sender sends, and the sender may
        # be waiting - through its own tensor-parallel peers - for exactly the kernel that
        # cannot become resident.  OPT-2.7B on 2 stages x 4-way tensor parallelism hung that
        # way; with receives posted where the tensor is needed (and sends still not waited
        # for) no such cycle exists.
        fused_tp = mesh.tp_size > 1 and self.device.type == "cuda"
        self._prefetch_recv = not fused_tp
        override = self.cfg.extra.get("prefetch_recv")
        if override is not None:
            self._prefetch_recv = bool(override)
        # "paired": every exchange with a neighbour is ONE batched send + receive group that the
        # compute stream waits for before the next kernel, so that no NCCL kernel is ever
        # resident beside a persistent tensor-parallel kernel (the schedule that ran OPT-2.7B
        # on 2 stages x 4-way tensor parallelism); "overlap": the side-stream schedule above.
        self._p2p_mode = self.cfg.extra.get("p2p_mode") or ("paired" if fused_tp else "overlap")
        if self._p2p_mode not in ("paired", "overlap"):
            raise ValueError(f"p2p_mode must be 'paired' or 'overlap', not {self._p2p_mode!r}")
        self._tied = self._find_tied()
        # gradients of parameters shared with another stage change after backward (the other
        # stage's part is added): their buckets are reduced in step(), never from a hook
        self.inner.defer_params([p for p, stages in self._tied if self.stage_id in stages])
        # ... and they enter the global gradient norm once, on the first stage that owns them
        self.inner.exclude_from_norm([p for p, stages in self._tied
                                      if self.stage_id in stages and self.stage_id != stages[0]])
        self._sync_tied_params()
        self.last_loss = None

    # ---- tied parameters across stages --------------------------------- #
    def _find_tied(self):
        owners = {}
        for s, stage in enumerate(self.model.stages):
            for p in stage.parameters():
                owners.setdefault(id(p), (p, set()))[1].add(s)
        groups = []
        for p, stages in owners.values():
            if len(stages) > 1:
                groups.append((p, sorted(stages)))
        if groups:
            logger.info("tied parameters across stages: %s", [g[1] for g in groups], ranks=0)
        return groups

    def _sync_tied_params(self):
        """Stages initialise their parameters independently; a parameter shared by several
        stages (tied embedding / LM head) takes the value of the first stage that owns it.
        One batched group of sends / receives per rank."""
        c = self.mesh.get_coord()
        ops, copies = [], []
        for p, stages in self._tied:
            if self.stage_id not in stages or p.is_meta:
                continue
            src_stage = stages[0]
            if self.stage_id == src_stage:
                for s in stages[1:]:
                    ops.append(dist.P2POp(dist.isend, p.data.contiguous(),
                                          self.mesh.get_rank(pp=s, dp=c["dp"], tp=c["tp"])))
            else:
                buf = _dense_like(p.data)
                ops.append(dist.P2POp(dist.irecv, buf,
                                      self.mesh.get_rank(pp=src_stage, dp=c["dp"], tp=c["tp"])))
                copies.append((p, buf))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        for p, buf in copies:
            p.data.copy_(buf)
        if copies:
            # the stage engine took its fp32 master copies before the values arrived
            self.inner.refresh_master_from_params()

    def _sync_tied_grads(self):
        c = self.mesh.get_coord()
        ops, adds = [], []
        for p, stages in self._tied:
            if self.stage_id not in stages or p.grad is None:
                continue
            ranks = [self.mesh.get_rank(pp=s, dp=c["dp"], tp=c["tp"]) for s in stages]
            # pairwise exchange keeps it group-free: sum = mine + theirs
            for r in ranks:
                if r == self.mesh.rank:
                    continue
                buf = _dense_like(p.grad)
                ops.append(dist.P2POp(dist.isend, p.grad.contiguous(), r))
                ops.append(dist.P2POp(dist.irecv, buf, r))
                adds.append((p, buf))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        for p, buf in adds:
            p.grad.add_(buf)

    # ---- p2p helpers ---------------------------------------------------- #
    def _link(self, lower_stage, direction):
        group = self.mesh.p2p_groups.get((lower_stage, direction))
        if group is None:
            raise RuntimeError(f"no pipeline link group for stage {lower_stage} ({direction}); "
                               "build the DeviceMesh with create_groups=True")
        return group

    def _isend(self, tensors, peer, group):
        for t in tensors:
            self._inflight.append(dist.isend(t.contiguous(), dst=peer, group=group))

    @staticmethod
    def _irecv(tensors, peer, group):
        return [dist.irecv(t, src=peer, group=group) for t in tensors]

    @staticmethod
    def _wait(works):
        for w in works or ():
            w.wait()

    @staticmethod
    def _flatten_values(values):
        """Per value crossing the stage boundary: ``(tree spec, leaves)``.  A value may be a
        tensor, a Python constant or a nest of them (a Hugging Face layer hands on
        ``(hidden_states, None)``); only the tensor leaves travel with every micro-batch."""
        return [tree_flatten(v) for v in values]

    def _handshake_send(self, flat, names):
        """Once per run: the static description of what will be sent - per value its name,
        tree structure and, per leaf, either (shape, dtype, requires_grad) or the constant."""
        meta = []
        for name, (leaves, spec) in zip(names, flat):
            desc = [(tuple(t.shape), str(t.dtype).replace("torch.", ""), bool(t.requires_grad))
                    if torch.is_tensor(t) else ("const", t) for t in leaves]
            meta.append((name, spec, desc))
        dist.send_object_list([meta], dst=self.next_rank, group=self._link(self.stage_id, "fwd"),
                              device=self.device)

    def _handshake_recv(self):
        box = [None]
        dist.recv_object_list(box, src=self.prev_rank, group=self._link(self.stage_id - 1, "fwd"),
                              device=self.device)
        return box[0]

    def _fwd_recv_buffers(self):
        """Empty tensors for the values entering this stage (None on stage 0)."""
        if self.stage_id == 0:
            return None
        if self._meta_fwd is None:
            self._meta_fwd = self._handshake_recv()
        bufs = []
        for name, spec, desc in self._meta_fwd:
            leaves = []
            for entry in desc:
                if entry[0] == "const":
                    leaves.append((entry[1], False, False))
                else:
                    shape, dtype, rg = entry
                    leaves.append((torch.empty(shape, dtype=getattr(torch, dtype),
                                               device=self.device), True, rg))
            bufs.append((name, spec, leaves))
        return bufs

    @staticmethod
    def _tensor_list(bufs):
        return [v for _, _, leaves in bufs for v, is_tensor, _ in leaves if is_tensor] \
            if bufs else []

    def _post_recv_forward(self):
        """Post the receives of the next micro-batch's inputs: (buffers, works)."""
        if self.stage_id == 0:
            return None, None
        bufs = self._fwd_recv_buffers()
        works = self._irecv(self._tensor_list(bufs), self.prev_rank,
                            self._link(self.stage_id - 1, "fwd"))
        return bufs, works

    def _send_forward(self, rec):
        if self.stage_id < self.n_stages - 1:
            self._isend([t.detach() for t in rec["payload"]], self.next_rank,
                        self._link(self.stage_id, "fwd"))

    def _post_recv_backward(self, rec):
        """Post the receives of the output gradients of a micro-batch in flight."""
        grads = [_dense_like(t) for t in rec["sent"]]
        works = []
        if self.stage_id < self.n_stages - 1 and grads:
            works = self._irecv(grads, self.next_rank, self._link(self.stage_id, "bwd"))
        return grads, works

    def _send_backward(self, in_grads):
        if self.stage_id > 0 and in_grads:
            self._isend(in_grads, self.prev_rank, self._link(self.stage_id - 1, "bwd"))

    # ---- compute ---------------------------------------------------------- #
    def _compute_forward(self, mb_inputs, labels, bufs):
        env, received = {}, []
        if self.stage_id == 0:
            env.update(mb_inputs)
        else:
            for name, spec, leaves in bufs:
                values = []
                for v, is_tensor, rg in leaves:
                    if is_tensor and rg and v.is_floating_point():
                        v.requires_grad_(True)
                        received.append(v)
                    values.append(v)    # constants travelled in the handshake
                env[name] = tree_unflatten(values, spec)
        env.update(self.stage(env))
        rec = {"received": received, "loss": None, "sent": [], "payload": []}
        if self.stage_id == self.n_stages - 1:
            out = self.model.materialize_output(env)
            loss = self.loss_fn(out, labels) if self.loss_fn is not None else (
                out["loss"] if isinstance(out, dict) else out)
            if loss.dim() > 0:
                loss = loss.float().mean()
            rec["loss"] = loss / self.num_micro_batches
            return rec
        names = self.model.live_in[self.stage_id + 1]
        flat = self._flatten_values([env[n] for n in names])
        if not self._meta_sent:
            self._handshake_send(flat, names)
            self._meta_sent = True
        rec["payload"] = [t for leaves, _ in flat for t in leaves if torch.is_tensor(t)]
        rec["sent"] = [t for t in rec["payload"] if t.requires_grad]
        return rec

    def _compute_backward(self, rec, grads):
        if rec["loss"] is not None:
            # fp16 loss scaling: the last stage scales, the earlier ones receive scaled gradients
            self.inner.scale_loss(rec["loss"]).backward()
        elif rec["sent"]:
            torch.autograd.backward(rec["sent"], grads)
        return [t.grad if t.grad is not None else torch.zeros_like(t) for t in rec["received"]]

    # ---- the schedule ---------------------------------------------------- #
    def _exchange(self, sends, recvs):
        """One batched group of sends and receives with neighbours (global ranks, default
        group); the compute stream (NCCL) or the host (gloo) waits for all of it."""
        ops = [dist.P2POp(dist.isend, t.contiguous(), peer) for t, peer in sends]
        ops += [dist.P2POp(dist.irecv, t, peer) for t, peer in recvs]
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    def _finish_batch(self, losses):
        self.inner.set_final_backward(True)
        self._sync_tied_grads()
        self.inner.micro_step = 0
        self.inner.step()
        # the loss lives on the last stage; share it along the pipeline
        loss = torch.zeros((), device=self.device)
        if losses:
            loss = torch.stack(losses).sum().float()
        if self.mesh.pp_group is not None:
            src = self.mesh.get_rank(pp=self.n_stages - 1, dp=self.mesh.dp_rank, tp=self.mesh.tp_rank)
            dist.broadcast(loss, src=src, group=self.mesh.pp_group)
        self.last_loss = loss
        return loss

    def _train_batch_paired(self, micro_inputs, micro_labels):
        """1F1B with paired exchanges: a stage always puts "send to a neighbour" and the
        matching "receive from that neighbour" into one batched group (send forward + receive
        backward, send backward + receive forward), so the two sides of a link never wait for
        each other in opposite order, and waits for the group before it computes on."""
        m = self.num_micro_batches
        first, last = self.stage_id == 0, self.stage_id == self.n_stages - 1
        warmup = min(self.n_stages - self.stage_id - 1, m)
        steady = m - warmup
        prev, nxt = self.prev_rank, self.next_rank
        pending, losses = [], []
        fwd_i = bwd_i = 0

        def recv_forward():
            bufs = self._fwd_recv_buffers()
            if not first:
                self._exchange([], [(t, prev) for t in self._tensor_list(bufs)])
            return bufs

        def backward(done, grads):
            nonlocal bwd_i
            if done["loss"] is not None:
                losses.append(done["loss"].detach())
            # the data-parallel hooks may reduce a bucket only during the step's last backward
            self.inner.set_final_backward(bwd_i == m - 1)
            bwd_i += 1
            return self._compute_backward(done, grads)

        for _ in range(warmup):
            bufs = recv_forward()
            rec = self._compute_forward(micro_inputs[fwd_i], micro_labels[fwd_i], bufs)
            fwd_i += 1
            if not last:
                self._exchange([(t.detach(), nxt) for t in rec["payload"]], [])
            pending.append(rec)
        bufs = recv_forward() if steady > 0 else None
        for it in range(steady):
            rec = self._compute_forward(micro_inputs[fwd_i], micro_labels[fwd_i], bufs)
            fwd_i += 1
            pending.append(rec)
            # send this forward result, receive the gradient of the oldest micro-batch
            done = pending.pop(0)
            grads = [_dense_like(t) for t in done["sent"]]
            if not last:
                self._exchange([(t.detach(), nxt) for t in rec["payload"]],
                               [(g, nxt) for g in grads])
            in_grads = backward(done, grads)
            # send the input gradients, receive the next forward input
            more = it + 1 < steady
            bufs = self._fwd_recv_buffers() if (more and not first) else None
            if not first:
                self._exchange([(g, prev) for g in in_grads],
                               [(t, prev) for t in self._tensor_list(bufs)])
        while pending:
            done = pending.pop(0)
            grads = [_dense_like(t) for t in done["sent"]]
            if not last:
                self._exchange([], [(g, nxt) for g in grads])
            in_grads = backward(done, grads)
            if not first:
                self._exchange([(g, prev) for g in in_grads], [])
        return self._finish_batch(losses)

    def train_batch(self, *args, labels=None, **kwargs):
        m = self.num_micro_batches
        from .engine import _release_staging_slots

        _release_staging_slots()
        # the model's input hooks (collectives inside the first stage's tensor-parallel group)
        # run on the ranks where the inputs enter the pipeline
        env = self.model.bind_inputs(args, kwargs, run_hooks=self.stage_id == 0)
        micro_inputs = [{} for _ in range(m)]
        for name, val in env.items():
            for i, piece in enumerate(_split_micro(val, m)):
                micro_inputs[i][name] = piece
        micro_labels = _split_micro(labels, m) if labels is not None else [None] * m
        self.inner.set_final_backward(False)
        if self._p2p_mode == "paired":
            return self._train_batch_paired(micro_inputs, micro_labels)
        warmup = min(self.n_stages - self.stage_id - 1, m)
        steady = m - warmup
        pending, losses = [], []
        fwd_i = 0
        bwd_i = 0

        def forward_one(cur):
            """Prefetch the next input, then run micro-batch ``fwd_i`` on the input ``cur``
            whose receives were posted one micro-batch ago."""
            nonlocal fwd_i
            if self._prefetch_recv:
                nxt = self._post_recv_forward() if fwd_i + 1 < m else (None, None)
            else:
                cur, nxt = self._post_recv_forward(), (None, None)
            bufs, works = cur
            self._wait(works)
            rec = self._compute_forward(micro_inputs[fwd_i], micro_labels[fwd_i], bufs)
            fwd_i += 1
            self._send_forward(rec)
            pending.append(rec)
            return nxt

        def backward_one(done, posted):
            nonlocal bwd_i
            grads, works = posted
            self._wait(works)
            if done["loss"] is not None:
                losses.append(done["loss"].detach())
            # the data-parallel hooks may reduce a bucket only during the step's last backward
            self.inner.set_final_backward(bwd_i == m - 1)
            bwd_i += 1
            self._send_backward(self._compute_backward(done, grads))

        cur = self._post_recv_forward() if self._prefetch_recv else (None, None)
        for _ in range(warmup):
            cur = forward_one(cur)
        posted = None
        for _ in range(steady):
            # the output gradient of the oldest micro-batch travels during this forward
            if pending and posted is None and self._prefetch_recv:
                posted = self._post_recv_backward(pending[0])
            cur = forward_one(cur)
            done = pending.pop(0)
            if posted is None:     # last stage: nothing in flight before this forward
                posted = self._post_recv_backward(done)
            this, posted = posted, None
            backward_one(done, this)
        while pending:
            done = pending.pop(0)
            this = posted if posted is not None else self._post_recv_backward(done)
            # ... and the next one's during this backward
            posted = self._post_recv_backward(pending[0]) if pending and self._prefetch_recv else None
            backward_one(done, this)
        # sends: make the compute stream (NCCL) or the host (gloo) wait before buffers go away
        self._wait(self._inflight)
        self._inflight = []
        return self._finish_batch(losses)

    def __call__(self, *args, **kwargs):
        return self.model(*args, **kwargs)

    def step(self):
        return self.inner.step()
