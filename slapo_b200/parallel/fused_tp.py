"""Tensor-parallel linear layers on the fused GEMM+collective kernels.

Three differentiable ops replace "collective, then GEMM" / "GEMM, then
collective" pairs that ``shard`` + ``sync`` describe:

=================  ==========================  =====================================
op                 forward                     backward
=================  ==========================  =====================================
``ag_linear``      Y = all_gather(Xs) W^T      dXs = reduce_scatter(dY W)   (fused)
                   (gather inside the GEMM)    dW  = dY^T X, X = the tokens the forward
                                               kernel already gathered into local memory
``rs_linear``      Ys = reduce_scatter(X W^T)  dX  = all_gather(dYs) W      (fused)
                   (+ bias after reduction)    dW  = dY^T X, dY = what the dgrad kernel
                                               gathered (library split-K GEMM, no 2nd gather)
``ar_linear``      Y = all_reduce(X W^T)       dX  = dY W,  dW = dY^T X     (local)
=================  ==========================  =====================================

Activations are 2-D ``[tokens, features]``; the sharded ("sequence-parallel")
dimension is the token dimension, i.e. rank r holds rows ``[r*T/p, (r+1)*T/p)``.
``ctx`` is a :class:`~slapo_b200.parallel.symm.SymmContext` (or the local
stand-in used by the single-GPU tests).  Every op takes the next epoch of the
context, so all ranks must issue the same ops in the same order - which the
SPMD schedules do.

Reference behaviour being replaced: slapo/sharding/sync_ops.py:13-87 (blocking
NCCL collectives around cuBLAS GEMMs) and slapo/op/linear.py:105-111
(matmul -> sync -> bias).
"""
from __future__ import annotations

import torch

from ..ops import functional as NF
from ..ops import native

GATHER_NONE, GATHER_A_ROWS, GATHER_A_K, GATHER_B_K, GATHER_A_ROWS_STAGED = 0, 1, 2, 3, 4
GATHER_A_ROWS_PUSHED = 5
_CHUNK_WORDS = 8192   # kChunkCountOffset of csrc/comm_gemm.cu
# A partial-product (receive) buffer of the scatter modes starts with a header: one flag per
# (source rank, 128-row block of the owner's rows), written by the peers, then as many local
# arrival counters (kRecvHeaderBytes of csrc/comm_gemm.cu).  Symmetric buffers are zero when
# allocated, flags only ever grow (epoch numbers), counters return to zero.
RECV_HEADER_BYTES = 2 * _CHUNK_WORDS * 4
MODE_LOCAL, MODE_RS, MODE_AR = 0, 1, 2


def supported(x: torch.Tensor) -> bool:
    return (torch.is_tensor(x) and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16)
            and native.available() and hasattr(torch.ops.slapo_b200, "comm_gemm"))


def _check_status():
    code = int(native.ops().device_status())
    if code:
        raise RuntimeError(f"fused kernel reported error code {code}: a bounded wait on a peer "
                           "ran out (a rank is missing or stuck)")


_DEBUG = __import__("os").environ.get("SLAPO_B200_DEBUG", "0") == "1"


def _debug_check(ctx, epoch, a_ptrs, b_ptrs, M, N, K, lda, ldb, dtype, gather, seg_len, mode,
                 recv, ar_out, stage, chunk_flags):
    """Host-side checks of one fused launch (``SLAPO_B200_DEBUG=1``): everything a kernel
    would otherwise turn into a wrong peer address - alignment of every operand pointer, the
    sizes of the symmetric buffers against the problem, the flag slots against the pad, the
    epoch against the previous one."""
    esize = 2
    last = ctx.__dict__.get("_debug_last_epoch", 0)
    if epoch <= last:
        raise RuntimeError(f"fused op epoch {epoch} does not follow {last}")
    ctx.__dict__["_debug_last_epoch"] = epoch
    for name, ptrs in (("A", a_ptrs), ("B", b_ptrs)):
        for r, p in enumerate(ptrs):
            if int(p) % 16:
                raise ValueError(f"operand {name} of rank {r}: address {int(p):#x} is not 16-byte aligned")
    if lda % 8 or ldb % 8 or N % 8 or K % 8:
        raise ValueError("leading dimensions / sizes must be multiples of 8: "
                         f"lda={lda} ldb={ldb} N={N} K={K}")
    blocks = (M + 127) // 128
    if (gather == GATHER_A_ROWS_STAGED or mode != MODE_LOCAL) and blocks > _CHUNK_WORDS:
        raise ValueError(f"{blocks} row blocks exceed the {_CHUNK_WORDS} flag slots")
    if gather in (GATHER_A_ROWS, GATHER_A_ROWS_STAGED) and seg_len * ctx.world != M:
        raise ValueError(f"gathered rows: {ctx.world} segments of {seg_len} != M={M}")
    if gather in (GATHER_A_K, GATHER_B_K) and seg_len * ctx.world != K:
        raise ValueError(f"gathered contraction: {ctx.world} segments of {seg_len} != K={K}")
    if mode != MODE_LOCAL:
        need = RECV_HEADER_BYTES + M * N * esize
        if recv is None or recv.nbytes < need:
            raise ValueError(f"partial-product buffer holds {getattr(recv, 'nbytes', 0)} bytes, "
                             f"the op needs {need}")
        if len(recv.peer_ptrs) != ctx.world:
            raise ValueError("partial-product buffer was not rendezvoused over the whole group")
    if mode == MODE_AR and (ar_out is None or ar_out.nbytes < M * N * esize):
        raise ValueError("all-reduce output buffer is too small")
    if gather == GATHER_A_ROWS_STAGED:
        if stage is None or stage.numel() < M * K:
            raise ValueError("staging buffer of the gathered operand is too small")
        if chunk_flags is None or chunk_flags.numel() < 2 * _CHUNK_WORDS:
            raise ValueError("chunk flag pad is too small")


def _wgrad(dy, x):
    """``dW = dY^T X`` on this library's split-K GEMM (both operands read as stored: ``dY``
    M-major, ``X`` N-major); tensors the kernel cannot address go to PyTorch."""
    if (dy.shape[1] % 8 == 0 and x.shape[1] % 8 == 0 and dy.stride(1) == 1 and x.stride(1) == 1
            and dy.stride(0) % 8 == 0 and x.stride(0) % 8 == 0):
        return NF.gemm(dy, x, a_mn=True, b_mn=True, split_k=True)
    return dy.t() @ x


def _dgrad(dy, w):
    """``dX = dY W`` with ``W`` ``[N, K]`` read N-major."""
    if dy.shape[1] % 8 == 0 and w.shape[1] % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0:
        return NF.gemm(dy, w, b_mn=True)
    return dy @ w


def _dbias(dy):
    """Column sums of ``dY`` (one streaming kernel, fp32 accumulation)."""
    if dy.shape[1] % 8 == 0 and dy.stride(1) == 1 and dy.stride(0) % 8 == 0:
        return native.ops().colsum(dy)
    return dy.float().sum(0).to(dy.dtype)


def comm_gemm(ctx, *, a_ptrs, b_ptrs, M, N, K, lda, ldb, a_mn, b_mn, dtype, gather=GATHER_NONE,
              seg_len=0, mode=MODE_LOCAL, out_ptr=0, ldo=0, bias=None, act=-1, recv=None,
              ar_out=None, stage=None, chunk_flags=None, slot=None):
    """Thin wrapper of ``torch.ops.slapo_b200.comm_gemm``; takes the next epoch."""
    epoch = ctx.next_epoch()
    if _DEBUG:
        _debug_check(ctx, epoch, a_ptrs, b_ptrs, M, N, K, lda, ldb, dtype, gather, seg_len, mode,
                     recv, ar_out, stage, chunk_flags)
    native.ops().comm_gemm(
        [int(p) for p in a_ptrs], [int(p) for p in b_ptrs], M, N, K, lda, ldb, a_mn, b_mn,
        dtype == torch.bfloat16, gather, seg_len, mode, ctx.world, ctx.rank, epoch, int(out_ptr),
        ldo, bias.data_ptr() if bias is not None else 0, act, ctx.flags_ptr,
        list(ctx.peer_flag_ptrs), list(recv.ptrs()) if recv is not None else [],
        list(ar_out.ptrs()) if ar_out is not None else [], float(ctx.wait_seconds),
        stage.data_ptr() if stage is not None else 0,
        chunk_flags.data_ptr() if chunk_flags is not None else 0,
        int(getattr(recv, "mc_ptr", 0)) if recv is not None else 0,
        int(getattr(ar_out, "mc_ptr", 0)) if ar_out is not None else 0,
        list(slot.ptrs()) if slot is not None else [],
        int(getattr(slot, "mc_ptr", 0)) if slot is not None else 0)
    return epoch


class StagePool:
    """Staging slots of the pushed all-gather.

    A slot is a symmetric buffer: a header of block flags and slice counters, then the
    gathered operand ``[T, K]``.  In the pushed gather every rank stores its own rows into the
    slot of ALL ranks at the same offset (one multicast store through the NVSwitch), so all
    ranks must use the same slot for the same operation.  They do, because slots are handed
    out by a deterministic rule (a LIFO free list per size) and every rank issues the same
    operations in the same order; releases happen at fixed points of the program (the end of
    the autograd node's backward, or right after the launch when nothing is kept), never from
    a finaliser.  A slot whose operand is kept for the backward pass stays out of the free
    list until then - the gathered tokens are read by the weight-gradient GEMM straight from
    the slot, with no copy.  ``release_all`` (called by the engine at the start of a step)
    returns slots whose backward never ran.

    When the pool's byte limit (``SLAPO_B200_AG_POOL_GB``, default 32) is reached, ``acquire``
    returns ``None`` and the caller uses the size's single transient slot and copies what it
    has to keep."""

    _pools = None

    def __init__(self, ctx):
        import os
        import weakref

        self.ctx = ctx
        self.limit = int(float(os.environ.get("SLAPO_B200_AG_POOL_GB", "32")) * 2**30)
        self.used = 0
        self.free: dict[int, list[int]] = {}
        self.made: dict[int, int] = {}
        self.out: set = set()
        if StagePool._pools is None:
            StagePool._pools = weakref.WeakSet()
        StagePool._pools.add(self)

    def _buf(self, nbytes, idx):
        return self.ctx.buffer(f"ag_slot_{nbytes}_{idx}", RECV_HEADER_BYTES + nbytes)

    def acquire(self, nbytes):
        """(token, buffer) of a free slot for an operand of ``nbytes``, or ``None``."""
        free = self.free.setdefault(nbytes, [])
        if free:
            idx = free.pop()
        elif self.used + nbytes <= self.limit:
            idx = self.made.get(nbytes, 0)
            self.made[nbytes] = idx + 1
            self.used += nbytes
        else:
            return None
        token = (nbytes, idx)
        self.out.add(token)
        return token, self._buf(nbytes, idx)

    def transient(self, nbytes):
        return self._buf(nbytes, "t")

    def release(self, token):
        if token is not None and token in self.out:
            self.out.discard(token)
            self.free[token[0]].append(token[1])

    def release_all(self):
        for token in sorted(self.out, reverse=True):
            self.free[token[0]].append(token[1])
        self.out.clear()


def stage_pool(ctx) -> StagePool:
    pool = ctx.__dict__.get("_stage_pool")
    if pool is None:
        pool = ctx.__dict__["_stage_pool"] = StagePool(ctx)
    return pool


def step_boundary():
    """Start of a training step: every staging slot still held for a backward pass that never
    ran goes back to its pool (all ranks call this at the same point of the program)."""
    for pool in list(StagePool._pools or ()):
        pool.release_all()


def ag_mode(ctx) -> str:
    """How ``all_gather(x) @ w`` runs on this context:

    * ``"pull"``   - fused kernel, consumer loads: copier warps pull the peers' rows (default at
      two or three ranks, where it beats NCCL + a library GEMM by 1.2 - 1.3 x);
    * ``"push"``   - fused kernel, owner stores: every rank pushes its rows into the staging
      slots of all ranks from inside the GEMM kernel;
    * ``"gather"`` - the push as a kernel of its own (``peer_push_gather_kernel``, multicast
      stores through the NVSwitch at the full link rate) followed by this library's CTA-pair
      GEMM on the gathered slot.  Default where the context uses NVLS (four ranks or more): at
      eight GPUs the rows of all owners land in the last third of the transfer whatever the
      order they were sent in, so the fused kernel's GEMM cannot run under the transfer, and
      its single-CTA main loop is slower than the pair GEMM.

    ``SLAPO_B200_AG_MODE`` overrides."""
    mode = __import__("os").environ.get("SLAPO_B200_AG_MODE")
    if mode in ("push", "pull", "gather"):
        return mode
    return "gather" if getattr(ctx, "nvls", False) else "pull"


def push_enabled(ctx) -> bool:
    """The gathered operand goes through a pooled staging slot (``push`` and ``gather``)."""
    return ag_mode(ctx) != "pull"


def _can_push(ctx, shard_rows) -> bool:
    """The pushed gather handles whole 128-row blocks and at most 1024 of them in total (its
    slot header holds 16 flag words per block)."""
    return (ctx.world > 1 and shard_rows % 128 == 0 and shard_rows * ctx.world // 128 <= 1024
            and push_enabled(ctx))


def ag_gemm_pushed(ctx, x_shard, w, bias=None, act=-1, b_mn=False, keep=False, mode=None):
    """``all_gather(x_shard) @ w.T`` with the gather pushed by the owners: inside the GEMM
    kernel (``mode="push"``: ``comm_gemm.cu``, gather mode 5) or as a kernel of its own
    followed by the pair GEMM (``mode="gather"``); default: :func:`ag_mode`.
    Returns ``(y, gathered, token)``: with ``keep`` the gathered operand ``[T, K]`` stays valid
    until ``stage_pool(ctx).release(token)``; without it ``gathered`` is ``None``."""
    ts, k = x_shard.shape
    n = w.shape[1] if b_mn else w.shape[0]
    t = ts * ctx.world
    nbytes = t * k * x_shard.element_size()
    pool = stage_pool(ctx)
    got = pool.acquire(nbytes)
    token, slot = got if got is not None else (None, pool.transient(nbytes))
    if mode is None:
        mode = ag_mode(ctx)
    pair_ok = (x_shard.is_cuda and w.dtype == x_shard.dtype and w.stride(-1) == 1
               and w.stride(0) % 8 == 0 and n % 8 == 0 and k % 8 == 0)
    if mode == "gather" and pair_ok:
        # the gather as a kernel of its own, then the CTA-pair GEMM on the gathered slot
        epoch = ctx.next_epoch()
        native.ops().peer_push_gather(
            x_shard.data_ptr(), list(slot.ptrs(RECV_HEADER_BYTES)),
            int(slot.mc_ptr) + RECV_HEADER_BYTES if getattr(slot, "mc_ptr", 0) else 0,
            ts * k * x_shard.element_size(), ctx.world, ctx.rank, epoch, ctx.flags_ptr,
            list(ctx.peer_flag_ptrs), float(ctx.wait_seconds))
        full = slot.view(x_shard.dtype, (t, k), RECV_HEADER_BYTES)
        y = NF.gemm(full, w, bias=bias, act=act, b_mn=b_mn)
    else:
        y = torch.empty(t, n, dtype=x_shard.dtype, device=x_shard.device)
        a_ptrs = [x_shard.data_ptr() if r == ctx.rank else 0 for r in range(ctx.world)]
        comm_gemm(ctx, a_ptrs=a_ptrs, b_ptrs=[w.data_ptr()], M=t, N=n, K=k, lda=k, ldb=w.stride(0),
                  a_mn=False, b_mn=b_mn, dtype=x_shard.dtype, gather=GATHER_A_ROWS_PUSHED,
                  seg_len=ts, out_ptr=y.data_ptr(), ldo=n, bias=bias, act=act, slot=slot)
    if not keep:
        pool.release(token)
        return y, None, None
    full = slot.view(x_shard.dtype, (t, k), RECV_HEADER_BYTES)
    if token is None:            # pool exhausted: the transient slot is reused by the next gather
        full = full.clone()
    return y, full, token


def _staging(ctx, t, k, dtype, device):
    """Local staging buffer [t, k] and per-block flags for the staged gather."""
    st = ctx.__dict__.setdefault("_stage_local", {})
    key = (dtype, str(device))
    buf = st.get(key)
    if buf is None or buf.numel() < t * k:
        buf = torch.empty(t * k, dtype=dtype, device=device)
        st[key] = buf
    flags = st.get("flags")
    need = (t + 127) // 128
    if need > _CHUNK_WORDS:
        raise ValueError(f"{t} gathered rows exceed the {_CHUNK_WORDS * 128} the staged gather handles")
    if flags is None:
        # [0, 8192): epoch at which a 128-row block was staged; [8192, 16384): slice counters
        flags = torch.zeros(2 * _CHUNK_WORDS, dtype=torch.int32, device=device)
        st["flags"] = flags
    return buf[:t * k].view(t, k), flags


def _stage(ctx, name, t: torch.Tensor):
    """Copy a local tensor into the symmetric buffer ``name`` (peers read it).

    Two physical buffers alternate per name: a peer may still be reading the
    previous contents while this rank is already one operation ahead, but it
    cannot be two behind, because every fused operation waits for all peers to
    have entered it (and hence to have finished the one before)."""
    toggles = ctx.__dict__.setdefault("_stage_toggle", {})
    toggles[name] = toggles.get(name, 0) ^ 1
    name = f"{name}#{toggles[name]}"
    buf = ctx.buffer(name, t.numel() * t.element_size())
    buf.view(t.dtype, tuple(t.shape)).copy_(t)
    return buf


def peer_gather(ctx, shard, name):
    """All-gather ``shard`` (rows) over the group with this framework's own
    pull kernel: stage into symmetric memory, every rank copies the peers'
    segments over NVLink.  Used where the gathered tensor feeds a plain local
    GEMM (weight gradients, whose contraction runs over the gathered tokens)."""
    staged = _stage(ctx, name, shard)
    full = torch.empty((shard.shape[0] * ctx.world,) + tuple(shard.shape[1:]), dtype=shard.dtype,
                       device=shard.device)
    epoch = ctx.next_epoch()
    native.ops().peer_gather([int(p) for p in staged.ptrs()], full.data_ptr(),
                             shard.numel() * shard.element_size(), ctx.world, ctx.rank, epoch,
                             ctx.flags_ptr, list(ctx.peer_flag_ptrs), float(ctx.wait_seconds))
    return full


# ---------------------------------------------------------------------- #
def ag_gemm(ctx, x_shard, w, bias=None, act=-1, name="ag_in", staged=None, b_mn=False,
            keep_gathered=False):
    """``all_gather(x_shard) @ w.T`` with the gather inside the GEMM
    (``b_mn``: ``w`` is ``[K, N]`` and the product is ``all_gather(x) @ w``).

    ``keep_gathered``: also return the gathered operand ``[T, K]``.  The kernel pulls the
    remote rows into a local buffer anyway; with this flag the buffer is private to the call
    (and gets this rank's own rows copied in), so that the weight-gradient GEMM of the same
    layer can contract over it instead of gathering the tokens over NVLink a second time."""
    ts, k = x_shard.shape
    n = w.shape[1] if b_mn else w.shape[0]
    t = ts * ctx.world
    buf = staged if staged is not None else _stage(ctx, name, x_shard)
    y = torch.empty(t, n, dtype=x_shard.dtype, device=x_shard.device)
    if ts % 128 == 0 and ctx.world > 1:
        # remote rows are pulled once into a local staging buffer by copier warps
        stage, flags = _staging(ctx, t, k, x_shard.dtype, x_shard.device)
        if keep_gathered:
            stage = torch.empty(t, k, dtype=x_shard.dtype, device=x_shard.device)
        comm_gemm(ctx, a_ptrs=buf.ptrs(), b_ptrs=[w.data_ptr()], M=t, N=n, K=k, lda=k,
                  ldb=w.stride(0), a_mn=False, b_mn=b_mn, dtype=x_shard.dtype,
                  gather=GATHER_A_ROWS_STAGED, seg_len=ts, out_ptr=y.data_ptr(), ldo=n, bias=bias,
                  act=act, stage=stage, chunk_flags=flags)
        if keep_gathered:
            stage[ctx.rank * ts:(ctx.rank + 1) * ts].copy_(x_shard)   # own rows are read in place
            return y, stage
        return y
    comm_gemm(ctx, a_ptrs=buf.ptrs(), b_ptrs=[w.data_ptr()], M=t, N=n, K=k, lda=k,
              ldb=w.stride(0), a_mn=False, b_mn=b_mn, dtype=x_shard.dtype,
              gather=GATHER_A_ROWS, seg_len=ts, out_ptr=y.data_ptr(), ldo=n, bias=bias, act=act)
    if keep_gathered:
        return y, None
    return y


def gemm_rs(ctx, x, w, bias=None, b_mn=False, name="rs_recv"):
    """``reduce_scatter(x @ w.T)`` (rows) with the scatter in the epilogue;
    ``bias`` is added once, after the reduction.  ``b_mn``: ``w`` is ``[K, N]``."""
    t, k = x.shape
    n = w.shape[1] if b_mn else w.shape[0]
    if t // 128 > _CHUNK_WORDS:
        raise ValueError(f"{t} rows exceed the {_CHUNK_WORDS * 128} a fused reduce-scatter handles")
    recv = ctx.buffer(name, RECV_HEADER_BYTES + t * n * x.element_size())
    y = torch.empty(t // ctx.world, n, dtype=x.dtype, device=x.device)
    comm_gemm(ctx, a_ptrs=[x.data_ptr()], b_ptrs=[w.data_ptr()], M=t, N=n, K=k, lda=x.stride(0),
              ldb=w.stride(0), a_mn=False, b_mn=b_mn, dtype=x.dtype, mode=MODE_RS,
              out_ptr=y.data_ptr(), ldo=n, bias=bias, recv=recv)
    return y


def gemm_ar(ctx, x, w, bias=None, b_mn=False, name="ar"):
    """``all_reduce(x @ w.T)``: reduce-scatter + all-gather halves in one kernel."""
    t, k = x.shape
    n = w.shape[1] if b_mn else w.shape[0]
    if t // 128 > _CHUNK_WORDS:
        raise ValueError(f"{t} rows exceed the {_CHUNK_WORDS * 128} a fused all-reduce handles")
    recv = ctx.buffer(name + "_recv", RECV_HEADER_BYTES + t * n * x.element_size())
    out = ctx.buffer(name + "_out", t * n * x.element_size())
    comm_gemm(ctx, a_ptrs=[x.data_ptr()], b_ptrs=[w.data_ptr()], M=t, N=n, K=k, lda=x.stride(0),
              ldb=w.stride(0), a_mn=False, b_mn=b_mn, dtype=x.dtype, mode=MODE_AR,
              out_ptr=0, ldo=n, bias=bias, recv=recv, ar_out=out)
    # the symmetric output is reused by the next all-reduce: hand out a copy
    return out.view(x.dtype, (t, n)).clone()


# ---------------------------------------------------------------------- #
class _AGLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w, bias, sctx):
        ctx.sctx = sctx
        x_shard = x_shard.contiguous()
        ctx.token = None
        ctx.pooled = False
        if _can_push(sctx, x_shard.shape[0]):
            # no backward will run (evaluation, the first pass of a checkpointed layer): keep nothing
            keep = any(ctx.needs_input_grad[:3])
            y, full_x, ctx.token = ag_gemm_pushed(sctx, x_shard, w, bias, keep=keep)
            ctx.pooled = ctx.token is not None
            if not keep:
                ctx.gathered = False
                ctx.save_for_backward(x_shard, w)
                ctx.has_bias = bias is not None
                return y
        else:
            y, full_x = ag_gemm(sctx, x_shard, w, bias, keep_gathered=True)
        # the gathered tokens are kept for the weight gradient when the kernel staged them
        # (HBM is plentiful; the second NVLink gather in backward is not)
        ctx.gathered = full_x is not None
        ctx.save_for_backward(full_x if ctx.gathered else x_shard, w)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x_saved, w = ctx.saved_tensors
        sctx = ctx.sctx
        if ctx.pooled and ctx.token is None:
            raise RuntimeError(
                "second backward pass through an all-gather whose gathered tokens lived in a "
                "pooled staging slot: the slot went back to the pool after the first pass "
                "(set SLAPO_B200_AG_MODE=pull for graphs that are backpropagated twice)")
        dy = dy.contiguous()
        # dXs = reduce_scatter(dY @ W):  B = W read N-major ([N_local, K] = [contraction, out])
        dx = gemm_rs(sctx, dy, w, None, b_mn=True, name="rs_recv_bwd")
        # dW = dY^T @ all_gather(Xs): few output tiles and a very long
        # contraction - gather the tokens with the pull kernel and let the
        # library's split-K GEMM do the rest
        full_x = x_saved if ctx.gathered else peer_gather(sctx, x_saved.contiguous(), "ag_in_bwd")
        dw = _wgrad(dy, full_x)
        if ctx.token is not None:       # the staging slot that held the gathered tokens
            stage_pool(sctx).release(ctx.token)
            ctx.token = None
        db = _dbias(dy) if ctx.has_bias else None
        return dx, dw, db, None


class _RSLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, sctx):
        ctx.sctx = sctx
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        return gemm_rs(sctx, x.contiguous(), w, bias)

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        sctx = ctx.sctx
        dy_shard = dy_shard.contiguous()
        ts, n = dy_shard.shape
        t, kl = x.shape
        # dX = all_gather(dYs) @ W: A rows gathered inside the GEMM, B = W read N-major
        token = None
        if _can_push(sctx, ts):
            dx, full_dy, token = ag_gemm_pushed(sctx, dy_shard, w, None, b_mn=True, keep=True)
        else:
            dx, full_dy = ag_gemm(sctx, dy_shard, w, None, name="ag_dy_bwd", b_mn=True,
                                  keep_gathered=True)
        # dW = all_gather(dYs)^T @ X: long contraction, few tiles (see _AGLinear); the dgrad
        # kernel above has already gathered dY into local memory
        if full_dy is None:
            full_dy = peer_gather(sctx, dy_shard, "ag_dy_bwd2")
        dw = _wgrad(full_dy, x)
        stage_pool(sctx).release(token)
        # the bias is added on the owner's rows only: its gradient is partial
        # (tagged replicated_param -> summed over the group by the engine)
        db = _dbias(dy_shard) if ctx.has_bias else None
        return dx, dw, db, None


class _ARLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, sctx):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        return gemm_ar(sctx, x.contiguous(), w, bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = _dgrad(dy, w)
        dw = _wgrad(dy, x)
        db = _dbias(dy) if ctx.has_bias else None
        return dx, dw, db, None


class _ColLinearARBwd(torch.autograd.Function):
    """Column-parallel linear with replicated input: the forward is local, the
    input gradient ``dY W`` is a partial sum that the dgrad GEMM all-reduces."""

    @staticmethod
    def forward(ctx, x, w, bias, sctx):
        ctx.sctx = sctx
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        if NF.gemm_supported(x, w):
            return NF.gemm(NF._rows(x), w, bias)
        return torch.nn.functional.linear(x, w, bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        t = dy.shape[0]
        # the fused kernel wants whole 128-row blocks per rank and 16-byte aligned rows
        if t % (128 * ctx.sctx.world) == 0 and dy.shape[1] % 8 == 0 and w.shape[1] % 8 == 0:
            dx = gemm_ar(ctx.sctx, dy, w, None, b_mn=True, name="ar_bwd")
        else:  # row blocks do not split evenly over the group
            import torch.distributed as dist

            dx = _dgrad(dy, w)
            dist.all_reduce(dx, group=ctx.sctx.group)
        dw = _wgrad(dy, x)
        db = _dbias(dy) if ctx.has_bias else None
        return dx, dw, db, None


def col_linear_ar_bwd(x, w, bias, sctx):
    lead = x.shape[:-1]
    y = _ColLinearARBwd.apply(_as_2d(x), w, bias, sctx)
    return y.view(tuple(lead) + (w.shape[0],))


def _as_2d(x):
    return x.reshape(-1, x.shape[-1])


def ag_linear(x_shard, w, bias, sctx):
    """Column-parallel linear under token (sequence) parallelism.  ``x_shard``
    is ``[..., K]`` with this rank's tokens; returns all tokens ``[..., N_local]``
    (the leading dimension grows by the group size)."""
    lead = x_shard.shape[:-1]
    y = _AGLinear.apply(_as_2d(x_shard), w, bias, sctx)
    return y.view((lead[0] * sctx.world,) + tuple(lead[1:]) + (w.shape[0],))


def rs_linear(x, w, bias, sctx):
    """Row-parallel linear whose partial sums are reduce-scattered over tokens."""
    lead = x.shape[:-1]
    if lead[0] % sctx.world:
        raise ValueError(f"leading dimension {lead[0]} is not divisible by {sctx.world}")
    y = _RSLinear.apply(_as_2d(x), w, bias, sctx)
    return y.view((lead[0] // sctx.world,) + tuple(lead[1:]) + (w.shape[0],))


def ar_linear(x, w, bias, sctx):
    """Row-parallel linear whose partial sums are all-reduced."""
    lead = x.shape[:-1]
    y = _ARLinear.apply(_as_2d(x), w, bias, sctx)
    return y.view(tuple(lead) + (w.shape[0],))
