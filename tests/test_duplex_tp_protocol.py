"""The exchange protocol of the duplex path's tensor-parallel pair, played by two CPU threads standing in for the two
ranks: a flag word per rank that the PEER writes, a per-rank counter that numbers the exchanges, two buffers that
alternate. The device code is `lm_tp_add_norm_kernel`; this model checks the protocol's claims — both ranks compute
the same sums, a rank never overwrites a buffer the peer has yet to read however the two drift, and a peer that never
arrives ends in a bounded wait with an error instead of a hang."""
import threading
import time

import numpy as np


class Rank:
    def __init__(self, rows, dim):
        self.flag = 0                      # written by the peer: the number of its latest exchange
        self.counter = 0                   # exchanges this rank has completed
        self.buf = [np.zeros((rows, dim), np.float32) for _ in range(2)]
        self.reads = [0, 0]                # exchanges whose peer read of buf[i] has completed (bookkeeping for the test)
        self.error = False


def exchange(me, peer, which, partial, limit_s, jitter):
    """One all-reduce of `partial` as rank `me` sees it; returns the sum (or its own rows alone after a timeout)."""
    # the producing kernel may only overwrite buf[which] when the peer has read what every earlier exchange left there
    # (exchange k uses buffer k % 2, so counter // 2 earlier exchanges used this one)
    assert which == me.counter % 2 and me.reads[which] == me.counter // 2
    me.buf[which][...] = partial
    number = me.counter + 1
    peer.flag = number                     # release store into the peer's memory
    start = time.monotonic()
    while me.flag - number < 0:            # acquire loads of the own flag, bounded
        if time.monotonic() - start > limit_s:
            me.error = True
            me.counter = number
            return partial.copy()
        time.sleep(0)
    time.sleep(jitter())
    total = me.buf[which] + peer.buf[which]  # reads of the peer's buffer
    peer.reads[which] += 1
    me.counter = number
    return total


def run_pair(steps, rows=4, dim=8, slow_rank=None, limit_s=5.0):
    ranks = [Rank(rows, dim), Rank(rows, dim)]
    rng = [np.random.default_rng(10 + r) for r in range(2)]
    parts = [[rng[r].standard_normal((rows, dim)).astype(np.float32) for _ in range(steps)] for r in range(2)]
    sums = [[], []]

    def body(r):
        jit = np.random.default_rng(100 + r)
        for k in range(steps):
            if slow_rank == r:
                time.sleep(0.002)
            sums[r].append(exchange(ranks[r], ranks[1 - r], k % 2, parts[r][k], limit_s,
                                    lambda: float(jit.random()) * 1e-4))

    threads = [threading.Thread(target=body, args=(r,)) for r in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
        assert not t.is_alive()
    return ranks, parts, sums


def test_both_ranks_compute_the_same_sums_whatever_the_drift():
    for slow in (None, 0, 1):
        ranks, parts, sums = run_pair(40, slow_rank=slow)
        assert not ranks[0].error and not ranks[1].error
        for k in range(40):
            want = parts[0][k] + parts[1][k]
            assert np.array_equal(sums[0][k], want) and np.array_equal(sums[1][k], want)
        assert ranks[0].counter == ranks[1].counter == 40


def test_a_missing_peer_ends_in_a_bounded_wait_and_an_error():
    me, ghost = Rank(2, 4), Rank(2, 4)
    t0 = time.monotonic()
    out = exchange(me, ghost, 0, np.ones((2, 4), np.float32), 0.2, lambda: 0.0)
    assert me.error and time.monotonic() - t0 < 2.0
    assert np.array_equal(out, np.ones((2, 4), np.float32)) and me.counter == 1
