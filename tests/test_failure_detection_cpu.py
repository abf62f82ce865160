"""Failure detection without any device fault: failures are made on the host (a rank that raises, a rank that goes
silent) and the peers learn of them through the store-based heartbeat before their next collective."""
import time

import pytest
import torch
import torch.distributed as dist

from fairscale_b200.fair_dev.testing.testing import spawn_ranks
from fairscale_b200.utils.failure import CommTimeoutError, Heartbeat, PeerFailureError, make_heartbeat


def test_heartbeat_single_process_hashstore():
    store = dist.HashStore()
    a, b = Heartbeat(store, 0, 2, timeout_s=0.3), Heartbeat(store, 1, 2, timeout_s=0.3)
    a.beat(0)
    b.beat(0)
    a.sync_step(0)  # both at step 0: returns at once
    a.beat(0)       # repeating a step does not move the counter backwards or forwards
    assert store.add("fsb_hb/beat/0", 0) == 1
    t0 = time.monotonic()
    with pytest.raises(PeerFailureError) as err:
        a.sync_step(1)  # rank 1 never reaches step 1
    assert err.value.ranks == [1] and "no heartbeat" in err.value.reasons[1] and time.monotonic() - t0 < 5
    with pytest.raises(ValueError):
        with b.guard():
            raise ValueError("boom")
    with pytest.raises(PeerFailureError) as err:
        a.check()
    assert "ValueError: boom" in err.value.reasons[1]
    assert b.failed_peers() == {}  # a rank does not report itself
    with pytest.raises(PeerFailureError):
        with a.guard():  # reacting to a peer's failure does not mark this rank as failed
            a.check()
    assert b.failed_peers() == {}


def test_comm_timeout_error_message():
    e = CommTimeoutError(1, "cuda:0")
    assert e.code == 1 and "bounded device-side wait" in str(e)


def _job(rank, world, victim, mode):
    hb = make_heartbeat(timeout_s=3.0)
    done = 0
    caught = None
    try:
        for step in range(6):
            with hb.guard():
                if rank == victim and step == 3:
                    if mode == "raise":
                        raise RuntimeError("injected failure before the collective")
                    return  # "silent": leaves between steps without a word, nothing of it in flight
                hb.sync_step(step)
                t = torch.ones(1)
                dist.all_reduce(t)
                assert t.item() == world
                done += 1
    except PeerFailureError as e:
        caught = e
    except RuntimeError as e:
        assert rank == victim and "injected" in str(e)
        return
    # survivors: three full steps, then the failure is seen on the host and no fourth collective is entered
    assert rank != victim and done == 3 and caught is not None and caught.ranks == [victim]
    if mode == "raise":
        assert "injected failure" in caught.reasons[victim]
    else:
        assert "no heartbeat for step 3" in caught.reasons[victim]


@pytest.mark.parametrize("mode", ["raise", "silent"])
def test_peers_stop_before_the_next_collective(mode):
    spawn_ranks(_job, 3, (1, mode), backend="gloo", timeout=120)
