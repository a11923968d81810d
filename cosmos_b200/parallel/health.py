"""Host-side failure detection for multi-rank jobs: heartbeats and bounded rendezvous over the
`torch.distributed` key-value store.

A rank that dies between steps (exception, lost node, operator kill) would otherwise be noticed
by its peers only when their next collective blocks until the process-group timeout. Here every
rank publishes `hb/<rank> = <step>:<wall time>` between steps, and before it launches the next
step it checks that every peer has published a recent beat; a peer that announced its departure
(`leave/<rank>`) or whose beat is older than the limit raises `PeerFailure` on the survivors, on
the host, with no kernel or collective in flight. `bounded_rendezvous` is the same idea for start-up:
it names the ranks that never arrived instead of waiting forever.

The reference has no failure handling beyond client-side timeouts (`--init-timeout 1800`,
reference README.md:304; job status polling in cookbooks/cosmos3/generator/action/
run_fd_with_vllm.ipynb). Device-side waits are bounded separately (csrc/common.cuh, csrc/comm.cu).
"""
from __future__ import annotations

import time
from typing import Iterable, List, Optional, Sequence


class PeerFailure(RuntimeError):
    """Raised on the surviving ranks; `ranks` lists the peers considered gone and `reason` why."""

    def __init__(self, ranks: Sequence[int], reason: str):
        self.ranks, self.reason = list(ranks), reason
        super().__init__(f"peer rank(s) {self.ranks} {reason}")


def _get(store, key: str) -> Optional[str]:
    """Non-blocking read: `check([key])` first, because `get` on a missing key blocks until the store's timeout."""
    if not store.check([key]):
        return None
    return store.get(key).decode()


class Heartbeat:
    """Per-rank liveness published through a c10d store (TCPStore / FileStore / HashStore)."""

    def __init__(self, store, rank: int, world: int, prefix: str = "health", clock=time.time):
        self.store, self.rank, self.world, self.prefix, self.clock = store, rank, world, prefix, clock
        self.step = 0

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def beat(self, step: Optional[int] = None) -> None:
        """Call between steps (no kernel or collective of this rank in flight)."""
        self.step = self.step + 1 if step is None else step
        self.store.set(self._key("hb", self.rank), f"{self.step}:{self.clock():.6f}")

    def leave(self, reason: str = "left") -> None:
        """Announces an orderly or failed departure so that peers stop before their next launch."""
        self.store.set(self._key("leave", self.rank), reason)

    def guard(self):
        """Context manager for host code between steps (data loading, checkpointing): an exception is
        announced to the peers before it propagates."""
        hb = self

        class _Guard:
            def __enter__(self):
                return hb

            def __exit__(self, exc_type, exc, tb):
                if exc_type is not None:
                    hb.leave(f"rank {hb.rank} failed between steps: {exc_type.__name__}")
                return False

        return _Guard()

    def peer_state(self, rank: int):
        """(step, wall time of the beat) of a peer, or None if it never published one."""
        v = _get(self.store, self._key("hb", rank))
        if v is None:
            return None
        s, t = v.split(":")
        return int(s), float(t)

    def check_peers(self, max_age_s: float, min_step: Optional[int] = None, peers: Optional[Iterable[int]] = None
                    ) -> None:
        """Raises PeerFailure if a peer announced that it left or has no beat younger than `max_age_s`
        (checked once, without waiting); with `min_step` it waits up to `max_age_s` for every peer to
        reach that step first."""
        peers = [r for r in (range(self.world) if peers is None else peers) if r != self.rank]
        gone = [r for r in peers if _get(self.store, self._key("leave", r)) is not None]
        if gone:
            raise PeerFailure(gone, "announced departure: " + ", ".join(
                _get(self.store, self._key("leave", r)) or "" for r in gone))
        deadline = self.clock() + max_age_s
        while True:
            now = self.clock()
            stale: List[int] = []
            for r in peers:
                st = self.peer_state(r)
                if st is None or now - st[1] > max_age_s or (min_step is not None and st[0] < min_step):
                    stale.append(r)
            if not stale:
                return
            left = [r for r in stale if _get(self.store, self._key("leave", r)) is not None]
            if left:
                raise PeerFailure(left, "announced departure")
            if min_step is None or now >= deadline:  # a plain age check does not wait
                raise PeerFailure(stale, f"sent no heartbeat within {max_age_s:.1f} s")
            time.sleep(min(0.05, max(0.0, deadline - now)))


def bounded_rendezvous(store, name: str, rank: int, world: int, timeout_s: float, clock=time.time) -> None:
    """All ranks call this with the same `name`; returns when everyone has arrived, raises PeerFailure
    naming the missing ranks after `timeout_s` (a rank that never joins must not hang the others)."""
    store.set(f"rdv/{name}/{rank}", "1")
    deadline = clock() + timeout_s
    while True:
        missing = [r for r in range(world) if not store.check([f"rdv/{name}/{r}"])]
        if not missing:
            return
        if clock() >= deadline:
            raise PeerFailure(missing, f"never reached rendezvous '{name}' within {timeout_s:.1f} s")
        time.sleep(0.02)


def guarded_step(hb: Optional[Heartbeat], fn, timeout_s: float = 30.0):
    """Runs one training / sampling step behind a bounded host-side rendezvous.

    A peer that died after its last heartbeat cannot be told from a slow one by the age of the beat
    alone, so before a step is launched every rank publishes `ready/<step>` and waits, with a limit,
    for the others: a rank that is gone never publishes it, and the survivors raise PeerFailure on the
    host instead of entering a collective that would block. If the step itself raises, the departure
    is announced before the exception propagates, so the peers stop at their next rendezvous at once."""
    if hb is None:
        return fn()
    k = hb.step + 1
    gone = [r for r in range(hb.world) if r != hb.rank and _get(hb.store, hb._key("leave", r)) is not None]
    if gone:
        raise PeerFailure(gone, "announced departure")
    hb.store.set(hb._key(f"ready{k}", hb.rank), "1")
    deadline = hb.clock() + timeout_s
    while True:
        missing = [r for r in range(hb.world) if not hb.store.check([hb._key(f"ready{k}", r)])]
        if not missing:
            break
        left = [r for r in missing if _get(hb.store, hb._key("leave", r)) is not None]
        if left:
            raise PeerFailure(left, "announced departure")
        if hb.clock() >= deadline:
            raise PeerFailure(missing, f"did not show up for step {k} within {timeout_s:.1f} s")
        time.sleep(0.005)
    if k > 2:  # keys of finished steps are not needed any more
        try:
            hb.store.delete_key(hb._key(f"ready{k - 2}", hb.rank))
        except (RuntimeError, NotImplementedError):
            pass
    try:
        out = fn()
    except BaseException as e:  # noqa: BLE001 - classify, announce, then re-raise
        # A rank whose own code failed announces it before the exception leaves this frame, i.e. before
        # its process can exit and break the peers' collectives. So a survivor whose collective broke
        # finds the announcement already there and reports the peer instead of the transport error.
        left = [r for r in range(hb.world) if r != hb.rank and _get(hb.store, hb._key("leave", r)) is not None]
        if left:
            raise PeerFailure(left, f"announced departure during step {k}") from e
        hb.leave(f"rank {hb.rank} failed in step {k}: {type(e).__name__}")
        raise
    hb.beat(k)
    return out
