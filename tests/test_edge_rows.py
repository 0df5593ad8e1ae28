"""The row arithmetic of the edge-row path of a sequence shard (csrc/wmm_tc_mm.cuh: the fp32 copy band_t writes;
csrc/wmm_halo.cu: the reduction in its third mode), restated in numpy on a small sequence split over several ranks:

  * band_t on a shard writes partial grad rows for positions [first - w, last + w) into an extended buffer of rows + 2w
    rows (16-bit), and output rows e in [edge_skip, edge_rows) and [ext - edge_rows, ext - edge_skip) once more unrounded
    into row e resp. e - (ext - 2 * edge_rows) of an fp32 buffer of 2 * edge_rows rows (edge_rows = 2w, edge_skip = w:
    the shard's own first and last w rows land in rows [w, 2w) and [2w, 3w));
  * the reduction sets own rows [w, 2w) of the extended buffer to round(fp32 rows [w, 2w) + the lower neighbour's rows
    [w + rows, ext)) and own rows [rows, rows + w) to round(fp32 rows [2w, 3w) + the upper neighbour's rows [0, w)).

The result must be the unsharded sum with at most one rounding of the neighbour's partial row more; adding the two 16-bit
partial rows has the rounding of the own partial row on top.
"""
import numpy as np
import pytest


def band_t_exact(band, x, w):
    """out[p] = sum_i band[i, p - i + w] x[i] in float64; band (M, 2w+1), x (M, N)."""
    M, N = x.shape
    out = np.zeros((M, N))
    for i in range(M):
        for j in range(2 * w + 1):
            p = i + j - w
            if 0 <= p < M:
                out[p] += band[i, j] * x[i]
    return out


def r16(a):
    return a.astype(np.float16)


@pytest.mark.parametrize("world,rows,w", [(2, 8, 2), (3, 6, 3), (4, 4, 2)])
def test_edge_row_reduction_matches_the_unsharded_sum(world, rows, w):
    rng = np.random.default_rng(world * 100 + w)
    M, N = world * rows, 3
    band = r16(rng.standard_normal((M, 2 * w + 1))).astype(np.float64)
    x = r16(rng.standard_normal((M, N))).astype(np.float64)
    exact = band_t_exact(band, x, w)
    ext = rows + 2 * w
    edge_rows, edge_skip = 2 * w, w
    ext16, edges = [], []
    for r in range(world):
        # partial rows of rank r: its own query rows only, positions first - w .. last + w
        part = np.zeros((ext, N))
        for i in range(r * rows, (r + 1) * rows):
            for j in range(2 * w + 1):
                p = i + j - w
                if 0 <= p < M:
                    part[p - (r * rows - w)] += band[i, j] * x[i]
        ext16.append(r16(part))
        e32 = np.full((2 * edge_rows, N), np.nan, dtype=np.float32)
        for e in range(ext):                      # the kernel's row rule
            er = e if e < edge_rows else (e - (ext - 2 * edge_rows) if e >= ext - edge_rows else -1)
            if er >= edge_skip and er < 2 * edge_rows - edge_skip:
                e32[er] = part[e].astype(np.float32)
        edges.append(e32)
        assert np.isnan(e32[:w]).all() and np.isnan(e32[3 * w:]).all() and not np.isnan(e32[w:3 * w]).any()
    for r in range(world):
        mine = ext16[r].copy()
        plain = ext16[r].astype(np.float32)       # what summing 16-bit rows gives, for comparison
        if r > 0:                                 # side 0: + the lower neighbour's upper margin
            mine[w:2 * w] = r16(edges[r][w:2 * w] + ext16[r - 1][w + rows:].astype(np.float32))
            plain[w:2 * w] = r16(plain[w:2 * w] + ext16[r - 1][w + rows:].astype(np.float32))
        if r < world - 1:                         # side 1: + the upper neighbour's lower margin
            mine[rows:rows + w] = r16(edges[r][2 * w:3 * w] + ext16[r + 1][:w].astype(np.float32))
            plain[rows:rows + w] = r16(plain[rows:rows + w] + ext16[r + 1][:w].astype(np.float32))
        got = mine[w:w + rows].astype(np.float64)
        want = exact[r * rows:(r + 1) * rows]
        # error budget per element: half an ulp of the result, plus half an ulp of the neighbour's partial row where one
        # was added (it crossed the link rounded to 16 bits; under cancellation it can be much larger than the sum)
        half = 2.0 ** -11
        theirs = np.zeros((rows, N))
        if r > 0:
            theirs[:w] = np.abs(ext16[r - 1][w + rows:].astype(np.float64))
        if r < world - 1:
            theirs[rows - w:] = np.abs(ext16[r + 1][:w].astype(np.float64))
        budget = half * (np.abs(want) + theirs) * 1.01 + 1e-7
        assert (np.abs(got - want) <= budget).all(), (r, (np.abs(got - want) / budget).max())
        inner = slice(w if r > 0 else 0, rows - w if r < world - 1 else rows)
        assert (got[inner] == r16(want[inner]).astype(np.float64)).all()
        # the 16-bit sum has the rounding of this rank's own partial row on top of that budget
        own = np.zeros((rows, N))
        own[:w] = np.abs(ext16[r][w:2 * w].astype(np.float64)) if r > 0 else 0
        own[rows - w:] = np.abs(ext16[r][rows:rows + w].astype(np.float64)) if r < world - 1 else 0
        assert (np.abs(plain[w:w + rows].astype(np.float64) - want) <= budget + half * own * 1.01).all()
