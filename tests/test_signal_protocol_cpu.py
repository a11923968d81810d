"""Threaded host model of the signal-pad protocol of csrc/comm.cu (`barrier_device`, the one-shot
all-reduce's leading / trailing barrier and its device-kept epoch counters): pads are int arrays
[slot][64] per rank, a rank writes its epoch into every peer's pad row and waits, with a bound, until its
own row shows that epoch (or a later one) from everybody. The model checks the properties the kernels
rely on: data published before a barrier is visible after it, epochs that only grow need no reset (a
fast rank may run one barrier ahead), a missing peer ends in a timeout status instead of a hang, and
the epoch counters stay in step across ranks without any launch argument changing."""
import random
import threading
import time

import numpy as np

ST_OK, ST_TIMEOUT_PEER = 0, 5


class Pads:
    def __init__(self, world, slots=64):
        self.world = world
        self.pad = [np.zeros((slots, 64), dtype=np.int64) for _ in range(world)]
        self.status = [ST_OK] * world


def barrier(p: Pads, rank: int, slot: int, epoch: int, limit_s: float = 2.0, skip_signal: bool = False) -> bool:
    if not skip_signal:
        for peer in range(p.world):          # st.release.sys into every peer's pad[slot][rank]
            p.pad[peer][slot, rank] = epoch
    t0 = time.time()
    for peer in range(p.world):              # ld.acquire.sys on the own pad, bounded
        while p.pad[rank][slot, peer] < epoch:
            if time.time() - t0 > limit_s:
                if p.status[rank] == ST_OK:  # first writer wins
                    p.status[rank] = ST_TIMEOUT_PEER
                return False
            time.sleep(0)
    return True


def _run(world, fn):
    errs = []

    def wrap(r):
        try:
            fn(r)
        except Exception as e:  # noqa: BLE001 - collected for the assertion below
            errs.append((r, repr(e)))

    ts = [threading.Thread(target=wrap, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(60)
    assert not errs, errs
    assert not any(t.is_alive() for t in ts)


def test_published_data_is_visible_after_the_barrier_and_epochs_need_no_reset():
    world, rounds = 4, 200
    p = Pads(world)
    data = np.zeros(world, dtype=np.int64)
    rnd = [random.Random(r) for r in range(world)]

    def body(r):
        for e in range(1, rounds + 1):
            if rnd[r].random() < 0.2:
                time.sleep(rnd[r].random() * 1e-3)   # ranks drift apart, a fast one runs a barrier ahead
            data[r] = e                              # publish, then signal
            assert barrier(p, r, slot=3, epoch=e)
            seen = data.copy()
            assert (seen >= e).all(), (r, e, seen)   # everybody's round-e data is there
            assert (seen <= e + 1).all(), (r, e, seen)  # and nobody can be two rounds ahead

    _run(world, body)
    assert all(s == ST_OK for s in p.status)


def test_missing_peer_gives_a_timeout_status_not_a_hang():
    world = 3
    p = Pads(world)
    out = {}

    def body(r):
        if r == 2:
            return                                    # never signals (host never launched it)
        t0 = time.time()
        out[r] = (barrier(p, r, slot=0, epoch=1, limit_s=0.3), time.time() - t0)

    _run(world, body)
    for r in (0, 1):
        ok, dt = out[r]
        assert ok is False and 0.25 < dt < 5.0
        assert p.status[r] == ST_TIMEOUT_PEER


def test_device_kept_epochs_stay_in_step_across_ranks():
    """One-shot all-reduce with `counters`: epoch = counters[slot] + 1 for the leading barrier, + 2 for
    the trailing one, and the counter is stored back, so the same launch can be replayed from a graph."""
    world, calls, n = 4, 50, 16
    p = Pads(world)
    counters = [np.zeros(64, dtype=np.int64) for _ in range(world)]
    bufs = [np.zeros(n) for _ in range(world)]
    results = [[] for _ in range(world)]

    def allreduce(r, slot):
        e = counters[r][slot] + 1
        assert barrier(p, r, slot, e)                 # inputs of every rank are in place
        acc = sum(bufs[q] for q in range(world)).copy()
        assert barrier(p, r, slot, e + 1)             # nobody overwrites its input early
        counters[r][slot] = e + 1
        return acc

    def body(r):
        for c in range(calls):
            bufs[r][:] = (r + 1) * (c + 1)
            results[r].append(allreduce(r, slot=16))

    _run(world, body)
    for c in range(calls):
        want = sum((q + 1) * (c + 1) for q in range(world))
        for r in range(world):
            assert (results[r][c] == want).all(), (r, c)
    assert all(cnt[16] == 2 * calls for cnt in counters)


def test_alternating_buffers_need_only_a_leading_barrier_and_a_new_user_continues_the_epochs():
    """Protocol of the fused all-reduce + residual + RMS-norm kernel (`allreduce_norm_kernel`): every call writes this
    rank's values into one of TWO buffers (alternating), meets the peers on a barrier whose epoch comes from a counter
    that belongs to the group, then reads all ranks' buffers; there is no trailing barrier. A rank that has passed the
    barrier of call c knows that every peer has finished reading the buffer of call c - 1, which is the one call c + 1
    overwrites. One counted barrier opens every step (graph replay) and resets the alternation. A second "decoder" that
    starts later on the same group keeps using the group's counters, so its first barrier is not satisfied by stale pads."""
    world, steps, calls = 4, 12, 7          # an odd number of calls per step: the step-opening barrier covers the wrap
    p = Pads(world)
    counters = [np.zeros(64, dtype=np.int64) for _ in range(world)]      # owned by the group, not by a decoder
    bufs = [[np.zeros(8), np.zeros(8)] for _ in range(world)]
    rnd = [random.Random(10 + r) for r in range(world)]
    results = [[] for _ in range(world)]

    def counted_barrier(r, slot):
        e = counters[r][slot] + 1
        ok = barrier(p, r, slot, e)
        counters[r][slot] = e                 # advanced even after a timeout, so ranks stay in step
        return ok

    def decoder_step(r, tag):
        assert counted_barrier(r, 15)         # begin_step: peers are done with the previous step's buffers
        parity = 0
        for c in range(calls):
            parity ^= 1
            if rnd[r].random() < 0.3:
                time.sleep(rnd[r].random() * 5e-4)
            bufs[r][parity][:] = (r + 1) * (tag * 100 + c + 1)           # split-K partials reduced into the own buffer
            assert counted_barrier(r, 16)
            results[r].append(sum(bufs[q][parity] for q in range(world)).copy())   # no barrier after the reads

    def body(r):
        for s in range(steps):
            decoder_step(r, s)
        # a second decoder on the same ranks (engine rebuilt): same counters, epochs continue
        for s in range(steps, steps + 3):
            decoder_step(r, s)

    _run(world, body)
    k = 0
    for s in range(steps + 3):
        for c in range(calls):
            want = sum((q + 1) * (s * 100 + c + 1) for q in range(world))
            for r in range(world):
                assert (results[r][k] == want).all(), (r, s, c, results[r][k][0], want)
            k += 1
    assert all(cnt[16] == (steps + 3) * calls and cnt[15] == steps + 3 for cnt in counters)
    assert all(s == ST_OK for s in p.status)
