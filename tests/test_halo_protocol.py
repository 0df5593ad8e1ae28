"""The hand-shake of the peer-memory halo exchange (csrc/wmm_halo.cu: halo_pull_kernel), restated on the CPU with one
Python thread per CTA (several CTAs per rank, started at staggered times) and plain lists for the flag words, to check
the protocol itself:
  * with every rank present, repeated exchanges complete, every CTA reads exactly the rows its neighbours published for
    THAT epoch (an owner may overwrite its rows right after its own call returns), and nobody waits forever;
  * with one rank absent, ONLY its two neighbours report a time-out, and each of them still copies from its live
    neighbour; ranks further away finish cleanly (the ack wait is longer than a neighbour's ready wait plus its copy);
  * whenever a CTA skips its share of a copy, the rank's status is set.
The kernel's steps per launch with epoch e: CTA 0 publishes ready = e and polls the neighbours' ready words (one thread
per side, READY limit), then publishes each side's verdict in a local go word; the other CTAs poll the go words (GO
limit); every CTA copies from the sides whose verdict is good and reports the others; the last CTA to finish writes
ack = e into both neighbours' flag blocks, waits for their acks (ACK limit) and closes the epoch."""
import threading
import time

READY_LIMIT = 0.04            # seconds; the kernel's limits are 1 s, 1.5 s and 3 s: the same ratios
GO_LIMIT = 1.5 * READY_LIMIT
ACK_LIMIT = 3.0 * READY_LIMIT
CTAS = 3


class Rank:
    def __init__(self, r, world):
        self.r, self.world = r, world
        self.flags = [0, 0, 0]     # ready, ack from the lower neighbour, ack from the upper neighbour
        self.epoch = 0
        self.done = 0              # CTAs finished in the running launch
        self.go = [0, 0]           # local verdict words: 2 * epoch + ok
        self.lock = threading.Lock()
        self.rows = ("rank%d" % r, 0)          # what this rank currently holds: (owner, version)
        self.seen = [[] for _ in range(CTAS)]  # per CTA and exchange: what it copied from (lower, upper)
        self.skipped = 0           # shares of a copy that some CTA did not do
        self.status = 0


def wait_until(pred, limit):
    t0 = time.monotonic()
    while not pred():
        if time.monotonic() - t0 > limit:
            return False
        time.sleep(0.0003)
    return True


def cta(me, ranks, c, e, stagger):
    """One CTA of one launch of rank `me` for epoch e."""
    time.sleep(stagger * c)
    nb = [ranks[me.r - 1] if me.r > 0 else None, ranks[me.r + 1] if me.r < me.world - 1 else None]
    ok = [False, False]
    if c == 0:
        me.flags[0] = e
        sides = []
        for side in (0, 1):      # the kernel polls both sides at the same time, one thread each
            def poll(side=side):
                if nb[side] is not None:
                    ok[side] = wait_until(lambda: nb[side].flags[0] >= e, READY_LIMIT)
                me.go[side] = 2 * e + (1 if ok[side] else 0)
            t = threading.Thread(target=poll)
            t.start()
            sides.append(t)
        for t in sides:
            t.join()
    else:
        for side in (0, 1):
            if nb[side] is not None:
                ok[side] = wait_until(lambda: me.go[side] >> 1 >= e, GO_LIMIT) and bool(me.go[side] & 1)
    for side in (0, 1):
        if nb[side] is not None and not ok[side]:
            me.status |= 32        # every CTA reports the share it skips
            me.skipped += 1
    me.seen[c].append(tuple(nb[s].rows if ok[s] else None for s in (0, 1)))
    with me.lock:
        me.done += 1
        last = me.done == CTAS
    if not last:
        return
    me.done = 0
    for side in (0, 1):            # acks go out whether the copy was done or given up
        if nb[side] is not None:
            nb[side].flags[2 if side == 0 else 1] = e     # I am the lower neighbour's UPPER neighbour
    for side in (0, 1):
        if nb[side] is not None and not wait_until(lambda: me.flags[1 + side] >= e, ACK_LIMIT):
            me.status |= 32
    me.epoch = e


def run(world, steps, absent=(), stagger=0.0):
    ranks = [Rank(r, world) for r in range(world)]

    def body(me):
        for s in range(steps):
            e = me.epoch + 1
            ts = [threading.Thread(target=cta, args=(me, ranks, c, e, stagger)) for c in range(CTAS)]
            for t in ts:
                t.start()
            for t in ts:
                t.join(timeout=30)
                assert not t.is_alive(), "a CTA is stuck: the protocol deadlocked"
            me.rows = (me.rows[0], s + 1)      # the owner rewrites its rows as soon as its exchange has returned

    threads = [threading.Thread(target=body, args=(rk,)) for rk in ranks if rk.r not in absent]
    t0 = time.monotonic()
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
        assert not t.is_alive(), "a rank is stuck: the protocol deadlocked"
    return ranks, time.monotonic() - t0


def test_repeated_exchanges_complete_and_read_the_rows_of_their_epoch():
    for world in (2, 3, 5):
        ranks, _ = run(world, steps=25, stagger=0.001)
        for rk in ranks:
            assert rk.status == 0 and rk.skipped == 0 and rk.epoch == 25
            for c in range(CTAS):
                assert len(rk.seen[c]) == 25
                for s, (lo, hi) in enumerate(rk.seen[c]):
                    if rk.r > 0:
                        assert lo == ("rank%d" % (rk.r - 1), s), (world, rk.r, c, s, lo)
                    if rk.r < world - 1:
                        assert hi == ("rank%d" % (rk.r + 1), s), (world, rk.r, c, s, hi)


def test_an_absent_rank_makes_only_its_neighbours_time_out():
    """200 runs: the outcome must not depend on how the waits of different ranks interleave."""
    for trial in range(200):
        ranks, elapsed = run(5, steps=1, absent=(2,), stagger=0.002 if trial % 2 else 0.0)
        assert ranks[1].status == 32 and ranks[3].status == 32, trial   # they waited for rank 2, gave up and returned
        assert ranks[0].status == 0 and ranks[4].status == 0, trial     # their neighbours did acknowledge in time
        for c in range(CTAS):
            # each neighbour of the absent rank still copied from its live neighbour, and nothing from the absent one
            assert ranks[1].seen[c] == [(("rank0", 0), None)], (trial, c, ranks[1].seen[c])
            assert ranks[3].seen[c] == [(None, ("rank4", 0))], (trial, c, ranks[3].seen[c])
            assert ranks[0].seen[c] == [(None, ("rank1", 0))] and ranks[4].seen[c] == [(("rank3", 0), None)]
        assert ranks[0].epoch == ranks[1].epoch == ranks[3].epoch == ranks[4].epoch == 1
        assert elapsed < 3 * (READY_LIMIT + ACK_LIMIT)


def test_skipped_work_always_sets_the_status():
    """A neighbour that shows up about one ready-limit late: whichever way the race goes, a rank whose CTAs skipped a
    share of the copy has its status set, and all CTAs of a rank agree on what they copied."""
    for trial in range(30):
        ranks = [Rank(r, 2) for r in range(2)]
        delay = READY_LIMIT * (0.8 + 0.4 * (trial % 5) / 4.0)

        def launch(me, wait):
            time.sleep(wait)
            ts = [threading.Thread(target=cta, args=(me, ranks, c, 1, 0.002)) for c in range(CTAS)]
            for t in ts:
                t.start()
            for t in ts:
                t.join(timeout=30)
                assert not t.is_alive()

        ts = [threading.Thread(target=launch, args=(ranks[0], 0.0)), threading.Thread(target=launch, args=(ranks[1], delay))]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        for rk in ranks:
            assert (rk.skipped > 0) <= (rk.status != 0), (trial, rk.r, rk.skipped, rk.status)
            assert len({tuple(rk.seen[c]) for c in range(CTAS)}) == 1, (trial, rk.r, rk.seen)
