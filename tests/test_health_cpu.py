"""Failure detection without a GPU fault: CPU ranks over gloo, failures made on the host
(a rank that raises, a rank that silently stops, a rank that never joins)."""
import time

import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_ranks


def _store():
    from torch.distributed.distributed_c10d import _get_default_store
    return _get_default_store()


def _steps_with_failure(rank, world, mode):
    """Every rank runs guarded steps with one all-reduce each; rank `world - 1` fails before step 3."""
    from cosmos_b200.parallel.health import Heartbeat, PeerFailure, guarded_step

    hb = Heartbeat(_store(), rank, world)
    done = 0
    t0 = time.time()
    try:
        for k in range(1, 6):
            if rank == world - 1 and k == 3:
                if mode == "between":   # host code between two steps raises (data loading, checkpointing)
                    with hb.guard():
                        raise ValueError("injected host-side failure between steps")
                elif mode == "inside":  # the step itself raises on this rank before its collective
                    def boom():
                        raise ValueError("injected host-side failure inside the step")
                    guarded_step(hb, boom, timeout_s=3.0)
                else:  # "silent": stops taking part without a word (killed, hung on the host)
                    return {"rank": rank, "done": done, "failure": "self", "elapsed": time.time() - t0}

            def step():
                x = torch.ones(4) * (rank + 1)
                dist.all_reduce(x)
                return float(x[0])

            total = guarded_step(hb, step, timeout_s=1.5)
            assert total == world * (world + 1) / 2
            done += 1
    except PeerFailure as e:
        return {"rank": rank, "done": done, "failure": e.ranks, "reason": e.reason, "elapsed": time.time() - t0}
    except ValueError:
        return {"rank": rank, "done": done, "failure": "self", "elapsed": time.time() - t0}
    return {"rank": rank, "done": done, "failure": None, "elapsed": time.time() - t0}


@pytest.mark.parametrize("mode", ["between", "inside", "silent"])
def test_peers_stop_on_the_host_when_a_rank_fails_between_steps(mode):
    world = 3
    out = run_ranks(_steps_with_failure, world, mode, timeout=60)
    for r in out[:-1]:
        assert r["done"] == 2, r                       # the two steps before the failure completed everywhere
        assert r["failure"] == [world - 1], r          # and the survivors name the failed rank
        assert r["elapsed"] < 20, r                    # without waiting for a collective timeout
    assert out[-1]["failure"] == "self" and out[-1]["done"] == 2
    if mode == "between":
        assert all(r["reason"] == "announced departure" for r in out[:-1])
    elif mode == "inside":    # the survivors' all-reduce broke; they report the peer, not the transport error
        assert all("announced departure during step 3" in r["reason"] for r in out[:-1])
    else:
        assert all("did not show up for step 3" in r["reason"] for r in out[:-1])


def _rendezvous_missing(rank, world):
    from cosmos_b200.parallel.health import PeerFailure, bounded_rendezvous

    if rank == 1:
        time.sleep(2.5)  # never joins within the limit
        return {"missing": "late"}
    try:
        bounded_rendezvous(_store(), "startup", rank, world, timeout_s=1.0)
    except PeerFailure as e:
        return {"missing": e.ranks}
    return {"missing": []}


def test_bounded_rendezvous_names_the_rank_that_never_joined():
    out = run_ranks(_rendezvous_missing, 3, timeout=60)
    assert out[0]["missing"] == [1] and out[2]["missing"] == [1]


def test_heartbeat_age_with_a_fake_clock():
    """Single process, HashStore, injected clock: a beat older than the limit marks the peer stale."""
    from cosmos_b200.parallel.health import Heartbeat, PeerFailure

    store = dist.HashStore()
    now = [100.0]
    a = Heartbeat(store, 0, 2, clock=lambda: now[0])
    b = Heartbeat(store, 1, 2, clock=lambda: now[0])
    a.beat()
    b.beat()
    a.check_peers(max_age_s=5.0)
    assert a.peer_state(1) == (1, 100.0)
    now[0] = 103.0
    b.beat()
    now[0] = 107.0
    a.check_peers(max_age_s=5.0)            # 4 s old: fine
    now[0] = 109.5
    with pytest.raises(PeerFailure) as ei:  # 6.5 s old and the (fake) clock does not advance: stale at once
        a.check_peers(max_age_s=5.0)
    assert ei.value.ranks == [1]
    b.leave("shutting down")
    with pytest.raises(PeerFailure) as ei:
        a.check_peers(max_age_s=1e9)
    assert "shutting down" in str(ei.value)


def _symm_alloc_with_a_missing_rank(rank, world):
    """The handle exchange of a symmetric buffer is guarded on the host: a rank that never reaches the
    allocation is named on the others instead of leaving them inside the exchange."""
    import os

    from cosmos_b200.parallel.health import PeerFailure
    from cosmos_b200.parallel.symm import SymmGroup

    os.environ["COSMOS_SYMM_TIMEOUT_S"] = "1.0"
    sg = SymmGroup(dist.group.WORLD, list(range(world)), torch.device("cpu"))      # everybody allocates the pads
    sg.alloc("shared_a", 1024)
    if rank == 2:
        time.sleep(2.5)                                                           # drops out before the next buffer
        return {"missing": "gone"}
    t0 = time.time()
    try:
        sg.alloc("shared_b", 1024)
    except PeerFailure as e:
        return {"missing": e.ranks, "waited": time.time() - t0}
    return {"missing": []}


def test_symmetric_allocation_names_the_rank_that_dropped_out():
    out = run_ranks(_symm_alloc_with_a_missing_rank, 3, timeout=60)
    for r in (0, 1):
        assert out[r]["missing"] == [2] and 0.9 < out[r]["waited"] < 8.0
