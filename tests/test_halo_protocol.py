"""The hand-shake of the peer-memory halo exchange (csrc/wmm_halo.cu: halo_pull_kernel), restated with one Python thread
per rank and plain lists for the flag words, to check the protocol itself on the CPU:
  * with every rank present, repeated exchanges complete, every rank reads exactly the rows its neighbours published for
    THAT epoch (an owner may overwrite its rows right after its own call returns), and nobody waits forever;
  * with one rank absent, its neighbours' bounded waits run out, they report it and return; ranks further away finish
    normally.
The kernel's steps per launch with epoch e: publish ready = e; wait for the neighbours' ready >= e; copy; write ack = e
into both neighbours' flag blocks; wait for their acks; epoch = e."""
import threading
import time

WAIT_LIMIT = 0.5   # seconds (the kernel's limit is one second per wait)


class Rank:
    def __init__(self, r, world):
        self.r, self.world = r, world
        self.flags = [0, 0, 0]     # ready, ack from the lower neighbour, ack from the upper neighbour
        self.epoch = 0
        self.rows = ("rank%d" % r, 0)          # what this rank currently holds: (owner, version)
        self.seen = []             # per exchange: what it copied from (lower, upper)
        self.timed_out = False


def wait_at_least(get, want):
    t0 = time.monotonic()
    while get() < want:
        if time.monotonic() - t0 > WAIT_LIMIT:
            return False
        time.sleep(0.0005)
    return True


def pull(me, ranks):
    lo = ranks[me.r - 1] if me.r > 0 else None
    hi = ranks[me.r + 1] if me.r < me.world - 1 else None
    e = me.epoch + 1
    me.flags[0] = e
    ok = all(wait_at_least(lambda n=n: n.flags[0], e) for n in (lo, hi) if n is not None)
    if ok:
        me.seen.append((lo.rows if lo else None, hi.rows if hi else None))
    if lo is not None:
        lo.flags[2] = e      # I am the lower neighbour's UPPER neighbour
    if hi is not None:
        hi.flags[1] = e
    fine = ok
    if lo is not None:
        fine = wait_at_least(lambda: me.flags[1], e) and fine
    if hi is not None:
        fine = wait_at_least(lambda: me.flags[2], e) and fine
    me.epoch = e
    me.timed_out = me.timed_out or not fine


def run(world, steps, absent=()):
    ranks = [Rank(r, world) for r in range(world)]

    def body(me):
        for s in range(steps):
            pull(me, ranks)
            me.rows = (me.rows[0], s + 1)      # the owner rewrites its rows as soon as its exchange has returned

    threads = [threading.Thread(target=body, args=(rk,)) for rk in ranks if rk.r not in absent]
    t0 = time.monotonic()
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=30)
        assert not t.is_alive(), "a rank is stuck: the protocol deadlocked"
    return ranks, time.monotonic() - t0


def test_repeated_exchanges_complete_and_read_the_rows_of_their_epoch():
    for world in (2, 3, 5):
        ranks, _ = run(world, steps=25)
        for rk in ranks:
            assert not rk.timed_out and rk.epoch == 25 and len(rk.seen) == 25
            for s, (lo, hi) in enumerate(rk.seen):
                if rk.r > 0:
                    assert lo == ("rank%d" % (rk.r - 1), s), (world, rk.r, s, lo)
                if rk.r < world - 1:
                    assert hi == ("rank%d" % (rk.r + 1), s), (world, rk.r, s, hi)


def test_an_absent_rank_makes_only_its_neighbours_time_out():
    ranks, elapsed = run(5, steps=1, absent=(2,))
    assert ranks[1].timed_out and ranks[3].timed_out          # they waited for rank 2, gave up and returned
    assert ranks[1].seen == [] and ranks[3].seen == []        # nothing was copied from a neighbour that was not ready
    assert not ranks[0].timed_out and not ranks[4].timed_out  # their neighbours did acknowledge
    assert ranks[0].epoch == ranks[1].epoch == ranks[3].epoch == ranks[4].epoch == 1
    assert elapsed < 10 * WAIT_LIMIT
