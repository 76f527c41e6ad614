"""Symmetric peer memory for the fused compute+collective kernels.

``SymmContext(group)`` owns, for one tensor-parallel (or data-parallel)
group on one node:

* a flag pad (64 x int32) in symmetric memory - ``ready[8] | done[8] |
  done2[8] | counters[..]`` - that the kernels use for flow control;
* named symmetric buffers (``buffer(name, nbytes)``): the same allocation on
  every rank, reachable from every rank through NVLink with plain loads and
  stores (and TMA tile loads without any cluster options);
* the job-wide *epoch* counter: every fused operation takes the next number,
  identically on all ranks because the program is SPMD.

Allocation goes through ``torch.distributed._symmetric_memory`` (CUDA
virtual-memory handles exchanged over the process group).  ``LocalSymmContext``
is a stand-in with ``world`` fake ranks whose buffers all live on one GPU: the
kernels are exercised rank by rank with the peers' flags pre-set, which is how
their numerics are tested without several GPUs and without ever running two
mutually waiting kernels on one device.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..logger import get_logger

logger = get_logger("symm")

FLAG_WORDS = 64


def _align(n, a=256):
    return (n + a - 1) // a * a


class SymmBuffer:
    """A symmetric allocation: local tensor (uint8) + every rank's base address."""

    def __init__(self, local: torch.Tensor, peer_ptrs, handle=None, mc_ptr=0):
        self.local = local
        self.peer_ptrs = list(peer_ptrs)
        self.handle = handle
        # NVLS address: loads through it return a reduction over every rank's copy, stores
        # land in every copy (0 = the buffer is not bound to an NVSwitch group)
        self.mc_ptr = int(mc_ptr)
        self.nbytes = local.numel() * local.element_size()

    def view(self, dtype, shape, offset_bytes=0):
        n = 1
        for s in shape:
            n *= s
        esize = torch.empty((), dtype=dtype).element_size()
        if offset_bytes + n * esize > self.nbytes:
            raise ValueError("view exceeds the symmetric buffer")
        flat = self.local.view(torch.uint8)[offset_bytes:offset_bytes + n * esize]
        return flat.view(dtype).view(shape)

    def ptrs(self, offset_bytes=0):
        return [p + offset_bytes for p in self.peer_ptrs]


class SymmContext:
    def __init__(self, group=None, device=None, wait_seconds: float = 30.0, nvls=None):
        """``wait_seconds``: limit of a kernel's wait for a peer (ranks of a training job drift
        apart by whole seconds around checkpoints and data stalls; tests that make a wait run
        out pass a short limit).  ``nvls``: let the kernels reduce through the NVSwitch
        (``multimem``) where the buffers have such an address; default: groups of four ranks
        or more - at two ranks peer loads are faster - unless ``SLAPO_B200_NVLS`` is 0 / 1.
        Jobs in which a rank may leave while others run keep it off."""
        import os

        import torch.distributed._symmetric_memory as symm_mem

        self._symm = symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("fused kernels support groups of at most 8 ranks (one NVSwitch node)")
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda", torch.cuda.current_device())
        self.wait_seconds = wait_seconds
        env = os.environ.get("SLAPO_B200_NVLS")
        if nvls is None:
            nvls = self.world >= 4 if env is None else env == "1"
        self.nvls = bool(nvls)
        self.epoch = 0
        self._buffers: dict[str, SymmBuffer] = {}
        flags = self._alloc("__flags__", FLAG_WORDS * 4)
        self.flags = flags
        flags.local.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def _alloc(self, name, nbytes) -> SymmBuffer:
        nbytes = _align(nbytes)
        t = self._symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        # Buffers start out zero (flag words inside them count epochs upwards), and the zeros
        # are in memory on every rank before any peer learns the address.
        t.zero_()
        torch.cuda.synchronize(self.device)
        hdl = self._symm.rendezvous(t, group=self.group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        mc = 0
        if self.nvls:
            try:
                mc = int(hdl.multicast_ptr)
            except Exception:   # no NVSwitch group on this system
                mc = 0
        buf = SymmBuffer(t, ptrs, hdl, mc)
        self._buffers[name] = buf
        return buf

    def buffer(self, name: str, nbytes: int) -> SymmBuffer:
        """Get (or grow) the symmetric buffer ``name``.  Collective: every rank
        of the group must call it with the same arguments in the same order."""
        buf = self._buffers.get(name)
        if buf is None or buf.nbytes < nbytes:
            buf = self._alloc(name, nbytes)
        return buf

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    @property
    def flags_ptr(self):
        return self.flags.peer_ptrs[self.rank]

    @property
    def peer_flag_ptrs(self):
        return self.flags.peer_ptrs


class LocalSymmContext:
    """``world`` fake ranks on one GPU (see the module docstring).  ``as_rank(r)``
    selects which rank the next kernels impersonate."""

    def __init__(self, world: int, device=None, wait_seconds: float = 0.05):
        self.world, self.rank = world, 0
        self.group = None
        self.nvls = False
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda", torch.cuda.current_device())
        self.wait_seconds = wait_seconds
        self.epoch = 0
        self._buffers: dict[str, list[torch.Tensor]] = {}
        self._flag_pads = [torch.zeros(FLAG_WORDS, dtype=torch.int32, device=self.device)
                           for _ in range(world)]

    def as_rank(self, rank: int):
        self.rank = rank
        return self

    def buffer(self, name, nbytes) -> SymmBuffer:
        nbytes = _align(nbytes)
        bufs = self._buffers.get(name)
        if bufs is None or bufs[0].numel() < nbytes:
            bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
                    for _ in range(self.world)]
            self._buffers[name] = bufs
        return SymmBuffer(bufs[self.rank], [b.data_ptr() for b in bufs])

    def rank_view(self, name, rank, dtype, shape):
        return SymmBuffer(self._buffers[name][rank], []).view(dtype, shape)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def preset_flags(self, epoch, ready=True, done=False, done2=False):
        """Pretend that every other rank has reached the given stages."""
        pad = self._flag_pads[self.rank]
        for r in range(self.world):
            if r == self.rank:
                continue
            if ready:
                pad[r] = epoch
            if done:
                pad[8 + r] = epoch
            if done2:
                pad[16 + r] = epoch

    def preset_block_flags(self, name, epoch, blocks_per_owner):
        """Pretend that every other rank has stored all row blocks of the current rank's rows in
        its partial-product buffer: the flags of those blocks in the header of every other
        rank's buffer ``name`` (one word per 128-row block of the ``[M, N]`` buffer)."""
        lo = self.rank * blocks_per_owner
        for r in range(self.world):
            if r != self.rank:
                hdr = self._buffers[name][r][:self.world * blocks_per_owner * 4].view(torch.int32)
                hdr[lo:lo + blocks_per_owner] = epoch

    @property
    def flags_ptr(self):
        return self._flag_pads[self.rank].data_ptr()

    @property
    def peer_flag_ptrs(self):
        return [p.data_ptr() for p in self._flag_pads]
