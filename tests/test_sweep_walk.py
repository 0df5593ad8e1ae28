"""The walk of the one-sweep window-backward kernel (csrc/wmm_tc_sweep.cuh: sweep_walk), restated in Python and checked
for the properties the kernel relies on, for many (sequences, row tiles, window, grid) combinations:
  * every box (row tile r, position tile pt), |r - pt| <= D, feeds the row product exactly once and the column product
    exactly once (by the CTA that owns the column), replayed rows included;
  * every row accumulator and every column accumulator is flushed exactly once, after its last contribution;
  * a column's tensor-memory slot (pt mod (2D + 2)) is never claimed while another column still lives in it.
No GPU needed: this is the index arithmetic all four roles of the kernel execute in lock step."""
import collections
import itertools


def walk(B, T, D, grid, cta):
    total = B * T
    per, rem = divmod(total, grid)
    g = cta * per + min(cta, rem)
    g_end = g + per + (1 if cta < rem else 0)
    events = []
    while g < g_end:
        b, ra = divmod(g, T)
        rb = min(T, ra + (g_end - g))
        own_lo, own_hi = ra - D, (T if rb == T else rb - D)
        for r in range(max(ra - 2 * D, 0), rb):
            warm = r < ra
            pt_lo, pt_hi = max(r - D, 0), min(r + D, T - 1)
            if warm:
                pt_lo, pt_hi = max(pt_lo, own_lo), min(pt_hi, own_hi - 1)
                if pt_lo > pt_hi:
                    continue
            for pt in range(pt_lo, pt_hi + 1):
                events.append(("box", b, r, pt, warm, own_lo <= pt < own_hi))
            if not warm:
                if r - D >= 0:
                    events.append(("flush_col", b, r - D))
                events.append(("flush_row", b, r))
                if r == T - 1:
                    for pt in range(max(T - D, 0), T):
                        events.append(("flush_col", b, pt))
        g += rb - ra
    return events


def check(B, T, D, grid):
    grid = min(grid, B * T)
    nslots = 2 * D + 2
    row_pass, col_pass = collections.Counter(), collections.Counter()
    rows_flushed, cols_flushed = collections.Counter(), collections.Counter()
    for cta in range(grid):
        live, contributions = {}, collections.Counter()
        for ev in walk(B, T, D, grid, cta):
            if ev[0] == "box":
                _, b, r, pt, warm, t_pass = ev
                if not warm:
                    row_pass[(b, r, pt)] += 1
                if t_pass:
                    col_pass[(b, r, pt)] += 1
                    slot = pt % nslots
                    if r == max(pt - D, 0):          # the column's first contribution claims the slot
                        assert slot not in live, (B, T, D, grid, cta, ev, live)
                        live[slot] = (b, pt)
                    assert live.get(slot) == (b, pt), (B, T, D, grid, cta, ev, live)
                    contributions[(b, pt)] += 1
            elif ev[0] == "flush_col":
                _, b, pt = ev
                cols_flushed[(b, pt)] += 1
                assert contributions[(b, pt)] == min(pt + D, T - 1) - max(pt - D, 0) + 1, (B, T, D, grid, cta, ev)
                assert live.pop(pt % nslots) == (b, pt)
            else:
                rows_flushed[(ev[1], ev[2])] += 1
        assert not live
    for b in range(B):
        for r in range(T):
            assert rows_flushed[(b, r)] == 1 and cols_flushed[(b, r)] == 1, (B, T, D, grid, b, r)
            for pt in range(max(r - D, 0), min(r + D, T - 1) + 1):
                assert row_pass[(b, r, pt)] == 1 and col_pass[(b, r, pt)] == 1, (B, T, D, grid, b, r, pt)


def test_every_box_feeds_both_products_once_and_slots_never_collide():
    for B, T, D, grid in itertools.product([1, 2, 3, 5], [1, 2, 3, 4, 5, 7, 32], [1, 2], [1, 2, 3, 4, 7, 148]):
        check(B, T, D, grid)


def test_replay_overhead_at_the_benchmark_configuration():
    """Config 2 (96 sequences of 32 row tiles, D = 2) on 148 CTAs: the replayed boxes add about 9 % to the band traffic."""
    B, T, D, grid = 96, 32, 2, 148
    boxes = [sum(1 for ev in walk(B, T, D, grid, c) if ev[0] == "box") for c in range(grid)]
    ideal = B * sum(min(r + D, T - 1) - max(r - D, 0) + 1 for r in range(T))
    assert ideal == 14784 and 1.08 < sum(boxes) / ideal < 1.10 and max(boxes) <= 115
