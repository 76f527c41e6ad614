"""Host-side failure detection for multi-rank jobs.

Device kernels that wait on a peer (the fused GEMM + collective kernels) give
up after a bounded spin and raise a status word, which keeps the CUDA context
usable but says nothing about *why* the peer is late.  This module answers
that on the host, before the next launch:

* :class:`Heartbeat` - every rank bumps a counter in the job's key-value
  store (the ``TCPStore`` / ``FileStore`` behind ``torch.distributed``) from a
  daemon thread; ``check()`` raises :class:`PeerFailure` naming the ranks
  whose counter stopped for longer than ``timeout`` seconds or that posted an
  error.  A rank that fails calls ``report_failure`` (the engines do so from
  their exception handlers), so peers learn the reason, not just the silence.
* :func:`guarded_step` - wraps one training step: checks the peers first,
  runs the step, turns a non-zero device status (a bounded wait that ran
  out) or an exception into a posted failure and re-raises.

Everything here runs on the CPU; the tests inject failures on the host (a
rank that raises, a rank that leaves between steps) with gloo ranks.  The
reference has no failure detection: its auto-tuner only classifies the log of
a process that already died (slapo/framework_dialect/deepspeed/utils.py:24-31).
"""
from __future__ import annotations

import threading
import time

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, message, ranks):
        super().__init__(message)
        self.ranks = list(ranks)


class Heartbeat:
    def __init__(self, store, rank, world_size, interval=0.2, timeout=5.0, prefix="hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self._halt = threading.Event()
        self._thread = None
        self._last_seen = {}      # rank -> (counter, local time it last changed)
        self._beat = 0

    # ---- keys ---------------------------------------------------------- #
    def _key(self, kind, rank):
        return f"{self.prefix}/{kind}/{rank}"

    def start(self):
        self.store.set(self._key("beat", self.rank), "0")
        self._thread = threading.Thread(target=self._run, daemon=True, name="slapo-heartbeat")
        self._thread.start()
        return self

    def _run(self):
        while not self._halt.wait(self.interval):
            self._beat += 1
            try:
                self.store.set(self._key("beat", self.rank), str(self._beat))
            except Exception:   # the store is gone: the job is being torn down
                return

    def stop(self, leaving=True):
        """Stop beating; ``leaving`` marks an orderly exit (not a failure)."""
        self._halt.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if leaving:
            try:
                self.store.set(self._key("left", self.rank), "1")
            except Exception:
                pass

    def report_failure(self, reason: str):
        try:
            self.store.set(self._key("error", self.rank), reason[:500])
        except Exception:
            pass

    # ---- observation ---------------------------------------------------- #
    def _get(self, key):
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def status(self):
        """``{rank: "ok" | "left" | "stale" | "error: ..."}`` for every other rank."""
        now = time.monotonic()
        out = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            err = self._get(self._key("error", r))
            if err is not None:
                out[r] = f"error: {err}"
                continue
            if self._get(self._key("left", r)) is not None:
                out[r] = "left"
                continue
            beat = self._get(self._key("beat", r))
            seen = self._last_seen.get(r)
            if beat is None:
                # never started: give it the timeout from our own first look
                if seen is None:
                    self._last_seen[r] = (None, now)
                    seen = self._last_seen[r]
            elif seen is None or seen[0] != beat:
                self._last_seen[r] = (beat, now)
                seen = self._last_seen[r]
            out[r] = "stale" if now - seen[1] > self.timeout else "ok"
        return out

    def check(self, allow_left=False):
        """Raise :class:`PeerFailure` if a peer failed, went silent or left."""
        bad = {r: s for r, s in self.status().items()
               if s != "ok" and not (allow_left and s == "left")}
        if bad:
            detail = ", ".join(f"rank {r}: {s}" for r, s in sorted(bad.items()))
            raise PeerFailure(f"peer failure detected by rank {self.rank}: {detail}", bad)


def default_store():
    """The key-value store of the default process group."""
    store = dist.distributed_c10d._get_default_store()
    if store is None:
        raise RuntimeError("torch.distributed is not initialised")
    return store


def guarded_step(heartbeat, step_fn, device_status_fn=None):
    """Run ``step_fn()`` between peer checks; post and re-raise any failure.

    ``device_status_fn`` returns the device status word of the native kernels
    (0 = fine); a non-zero value means a bounded wait gave up - most likely
    because a peer never arrived - so the peers are checked again to name it."""
    heartbeat.check()
    try:
        result = step_fn()
        if device_status_fn is not None:
            status = int(device_status_fn())
            if status != 0:
                try:
                    heartbeat.check()
                except PeerFailure as err:
                    raise PeerFailure(f"device status {status} (a bounded wait ran out); {err}",
                                      err.ranks) from None
                raise RuntimeError(f"device status {status}: a bounded wait in a kernel ran out "
                                   "although every peer is alive")
        return result
    except PeerFailure:
        raise
    except Exception as err:
        heartbeat.report_failure(f"{type(err).__name__}: {err}")
        raise
