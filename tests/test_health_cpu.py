"""Failure detection, with every failure made on the host: a rank that raises,
a rank that leaves between steps, a rank that goes silent, and a (faked)
device status word that reports a bounded wait running out."""
import time

import pytest
import torch
import torch.distributed as dist

from slapo_b200.runtime.health import Heartbeat, PeerFailure, default_store, guarded_step

from dist_utils import run_distributed


def _hb(rank, world, timeout=1.0):
    return Heartbeat(default_store(), rank, world, interval=0.05, timeout=timeout).start()


def _raise_worker(rank, world):
    hb = _hb(rank, world)
    dist.barrier()
    if rank == 1:
        with pytest.raises(ValueError):
            guarded_step(hb, lambda: (_ for _ in ()).throw(ValueError("loss is NaN")))
        # rank 1 does not enter the next collective; it stays alive until rank 0 noticed
        time.sleep(1.0)
    else:
        deadline = time.monotonic() + 5
        seen = None
        while time.monotonic() < deadline and seen is None:
            try:
                guarded_step(hb, lambda: None)    # would launch the next step
                time.sleep(0.05)
            except PeerFailure as err:
                seen = err
        assert seen is not None and seen.ranks == [1]
        assert "loss is NaN" in str(seen)
    hb.stop()


def test_rank_that_raises_is_reported_to_its_peers():
    run_distributed(_raise_worker, 2)


def _leave_worker(rank, world):
    hb = _hb(rank, world)
    dist.barrier()
    x = torch.ones(4)
    dist.all_reduce(x)                 # step 0: everybody is here
    if rank == 1:
        hb.stop(leaving=True)          # leaves between steps, nothing in flight
        time.sleep(1.0)
        return
    time.sleep(0.3)
    with pytest.raises(PeerFailure) as info:
        hb.check()                     # learnt on the host, before the next collective
    assert "left" in str(info.value)
    hb.check(allow_left=True)          # an elastic caller may carry on without that rank
    hb.stop()


def test_rank_that_leaves_between_steps_is_seen_before_the_next_launch():
    run_distributed(_leave_worker, 2)


def _silent_worker(rank, world):
    hb = _hb(rank, world, timeout=0.5)
    dist.barrier()
    if rank == 1:
        hb.stop(leaving=False)         # stops beating without a word (a hung process)
        time.sleep(2.0)
        return
    time.sleep(0.2)
    hb.check()                         # still within the timeout
    time.sleep(1.0)
    with pytest.raises(PeerFailure) as info:
        hb.check()
    assert "stale" in str(info.value)
    hb.stop()


def test_silent_rank_becomes_stale_after_the_timeout():
    run_distributed(_silent_worker, 2)


def _status_worker(rank, world):
    hb = _hb(rank, world)
    dist.barrier()
    assert guarded_step(hb, lambda: 7, device_status_fn=lambda: 0) == 7
    dist.barrier()
    if rank == 0:
        # all peers alive, but the (fake) device status says a bounded wait ran out
        with pytest.raises(RuntimeError) as info:
            guarded_step(hb, lambda: 1, device_status_fn=lambda: 4)
        assert "bounded wait" in str(info.value) and not isinstance(info.value, PeerFailure)
        time.sleep(1.0)
    else:
        deadline = time.monotonic() + 5
        seen = None
        while time.monotonic() < deadline and seen is None:
            try:
                guarded_step(hb, lambda: None, device_status_fn=lambda: 0)
                time.sleep(0.05)
            except PeerFailure as err:
                seen = err
        assert seen is not None and "bounded wait" in str(seen)
    hb.stop()


def test_device_status_word_turns_into_an_error():
    run_distributed(_status_worker, 2)
