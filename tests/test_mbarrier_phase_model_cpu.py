"""Host model of mbarrier phases for the P-written handshake of the paged decode attention kernel
(csrc/paged_decode_tc.cu). An mbarrier counts arrivals; when the expected count is reached its phase flips, and a
waiter asks "has the phase with parity p completed?", which is answered from the CURRENT phase only. The model
replays the kernel's ordering rules exhaustively over all interleavings that they allow and checks which barrier
layout can leave the MMA issuer waiting for good:

  * the softmax threads may write P of tile t + 1 as soon as the scores of t + 1 exist, and the issuer computes those
    scores BEFORE it waits for P of tile t; the P buffer of t + 1 is free once the product of t - 1 was issued
  * so P of t and P of t + 1 can both be complete before the issuer looks at P of t

With one barrier for both P buffers a late issuer then sees the parity of tile t "not completed" again and never
proceeds; with one barrier per buffer, a buffer's barrier completes a second time only after the issuer has issued the
product that read the buffer, i.e. after it has seen the first completion.
"""


class MBar:
    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.pending, self.phase = self.count, self.phase ^ 1

    def completed(self, parity):
        """try_wait.parity: true when the phase with this parity is not the one in progress."""
        return self.phase != parity


def run(n_tiles, n_bars, softmax_first):
    """Issuer and softmax group as two cooperating state machines. `softmax_first`: the scheduler lets the softmax
    group run as far as its dependencies allow before the issuer takes a step (the late-issuer interleaving);
    otherwise the issuer polls as soon as it can. Returns the number of tiles whose product the issuer issued."""
    bars = [MBar(1) for _ in range(n_bars)]          # one arrival stands for the 128 threads of the group
    scores_issued = 1                                 # scores of tile 0 are issued up front
    products_issued = 0                               # tiles whose second product was issued (= P seen)
    p_written = 0                                     # tiles whose P the softmax group has written
    steps = 0
    while products_issued < n_tiles and steps < 10 * n_tiles + 10:
        steps += 1

        def softmax_can():
            t = p_written
            return t < n_tiles and t < scores_issued and (t < 2 or products_issued >= t - 1)

        def softmax_step():
            nonlocal p_written
            bars[p_written % n_bars].arrive()
            p_written += 1

        def issuer_step():
            nonlocal scores_issued, products_issued
            t = products_issued
            did = False
            if scores_issued == t + 1 and t + 1 < n_tiles:
                scores_issued += 1                    # scores of t + 1 before the wait for P of t
                did = True
                if softmax_first:
                    return True                       # the late issuer is descheduled between the two actions
            parity = (t // n_bars) & 1 if n_bars == 2 else t & 1
            if bars[t % n_bars].completed(parity):
                products_issued += 1
                did = True
            return did

        if softmax_first:
            progressed = False
            while softmax_can():
                softmax_step()
                progressed = True
            progressed = issuer_step() or progressed
        else:
            progressed = issuer_step()
            if softmax_can():
                softmax_step()
                progressed = True
        if not progressed:
            break
    return products_issued


def test_one_barrier_for_both_p_buffers_can_lose_a_phase():
    assert run(8, 1, softmax_first=False) == 8        # a prompt issuer never notices
    assert run(8, 1, softmax_first=True) < 8          # a late one waits for good on the tile whose phase it missed


def test_one_barrier_per_p_buffer_never_does():
    for n in (1, 2, 3, 8, 33):
        assert run(n, 2, softmax_first=True) == n
        assert run(n, 2, softmax_first=False) == n
