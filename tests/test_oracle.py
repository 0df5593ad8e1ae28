"""Pins the CPU oracle (oracle/wmm_oracle.c) against golden vectors made by the compiled reference
(tests/golden/make_golden.py), bit for bit, and against an independent dense formulation."""
import numpy as np
import pytest

from oracle import oracle


def _w(name):
    return int(name.split("_w")[1].split("_")[0])


def test_golden_has_all_reference_test_shapes(golden):
    # tests/conftest.py:5-13 of the reference: DIMS x WINDOW_SIZES (w = 0 never reaches the kernels)
    for (b, m, n) in [(2, 1, 3), (2, 4, 3), (2, 16, 3), (2, 32, 3), (2, 16, 32)]:
        for w in (1, 4, 16):
            assert any(("_b%d_m%d_n%d_w%d_float32" % (b, m, n, w)) in k for k in golden)


def test_oracle_matches_reference_bit_for_bit(golden):
    assert len(golden) >= 35
    for name, c in golden.items():
        w = _w(name)
        a = oracle.window_matmul_forward(c["q"], c["k"], w)
        assert a.dtype == c["a"].dtype and np.array_equal(a, c["a"]), name
        gq, gk = oracle.window_matmul_backward(c["q"], c["k"], w, c["g_band"])
        assert np.array_equal(gq, c["gq"]) and np.array_equal(gk, c["gk"]), name
        o = oracle.unwindow_matmul_forward(c["att"], c["v"], w)
        assert np.array_equal(o, c["o"]), name
        gatt, gv = oracle.unwindow_matmul_backward(c["att"], c["v"], w, c["g_out"])
        assert np.array_equal(gatt, c["gatt"]) and np.array_equal(gv, c["gv"]), name


def _dense_band(q, kt, w):
    """Independent formulation: full Q.K^T in float64, then gather the diagonals."""
    B, M, _ = q.shape
    full = np.einsum("bih,bkh->bik", q.astype(np.float64), kt.astype(np.float64))
    band = np.zeros((B, M, 2 * w + 1))
    for i in range(M):
        for j in range(2 * w + 1):
            p = i + j - w
            if 0 <= p < M:
                band[:, i, j] = full[:, i, p]
    return band


def _dense_from_band(band, w):
    B, M, _ = band.shape
    full = np.zeros((B, M, M))
    for i in range(M):
        for j in range(2 * w + 1):
            p = i + j - w
            if 0 <= p < M:
                full[:, i, p] = band[:, i, j]
    return full


@pytest.mark.parametrize("shape", [(2, 16, 3, 4), (1, 33, 8, 40), (2, 70, 20, 7)])
def test_oracle_matches_dense_formulation(shape):
    B, M, Nn, w = shape
    rng = np.random.default_rng(7)
    q, kt, v = (rng.standard_normal((B, M, Nn)) for _ in range(3))
    k = np.ascontiguousarray(kt.transpose(0, 2, 1))
    att = rng.standard_normal((B, M, 2 * w + 1))
    g_band = rng.standard_normal((B, M, 2 * w + 1))
    g_out = rng.standard_normal((B, M, Nn))

    a = oracle.window_matmul_forward(q, k, w)
    np.testing.assert_allclose(a, _dense_band(q, kt, w), rtol=1e-12, atol=1e-12)
    # out-of-sequence entries are exact zeros
    for i in range(M):
        for j in range(2 * w + 1):
            if not 0 <= i + j - w < M:
                assert (a[:, i, j] == 0).all()

    full = _dense_from_band(att, w)
    np.testing.assert_allclose(oracle.unwindow_matmul_forward(att, v, w), full @ v, rtol=1e-12, atol=1e-12)

    gq, gk = oracle.window_matmul_backward(q, k, w, g_band)
    gfull = _dense_from_band(g_band, w)
    np.testing.assert_allclose(gq, gfull @ kt, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(gk, (gfull.transpose(0, 2, 1) @ q).transpose(0, 2, 1), rtol=1e-12, atol=1e-12)

    gatt, gv = oracle.unwindow_matmul_backward(att, v, w, g_out)
    np.testing.assert_allclose(gatt, _dense_band(g_out, v, w), rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(gv, full.transpose(0, 2, 1) @ g_out, rtol=1e-12, atol=1e-12)


def test_oracle_ignores_out_of_sequence_band_input():
    rng = np.random.default_rng(3)
    B, M, Nn, w = 1, 6, 4, 4
    att = rng.standard_normal((B, M, 2 * w + 1)).astype(np.float32)
    v = rng.standard_normal((B, M, Nn)).astype(np.float32)
    poisoned = att.copy()
    for i in range(M):
        for j in range(2 * w + 1):
            if not 0 <= i + j - w < M:
                poisoned[:, i, j] = np.nan
    assert np.array_equal(oracle.unwindow_matmul_forward(att, v, w), oracle.unwindow_matmul_forward(poisoned, v, w))


@pytest.mark.parametrize("mask", [False, True])
@pytest.mark.parametrize("M,w", [(7, 3), (16, 16), (33, 5), (5, 9)])
def test_oracle_band_softmax_matches_the_torch_composition(M, w, mask):
    """The reference composes the step between its two operators from torch ops (tests/test_attention.py:60-61:
    scores / sqrt(N), softmax over the last dimension); the oracle's softmax is pinned to that composition on CPU,
    forward and (through autograd) backward."""
    import torch

    g = torch.Generator().manual_seed(M * 100 + w)
    B, W = 2, 2 * w + 1
    scores = torch.randn(B, M, W, generator=g, dtype=torch.float64, requires_grad=True)
    gp = torch.randn(B, M, W, generator=g, dtype=torch.float64)
    scale = 1.0 / 8.0
    s = scores * scale
    if mask:
        i = torch.arange(M)[:, None]
        j = torch.arange(W)[None, :]
        outside = ((i + j - w) < 0) | ((i + j - w) >= M)
        s = s.masked_fill(outside, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p.backward(gp)
    po = oracle.band_softmax(scores.detach().numpy(), scale, mask)
    np.testing.assert_allclose(po, p.detach().numpy(), rtol=1e-13, atol=1e-15)
    go = oracle.band_softmax_backward(po, gp.numpy(), scale, mask)
    np.testing.assert_allclose(go, scores.grad.numpy(), rtol=1e-12, atol=1e-15)
    if mask:
        assert (po[:, outside.numpy()] == 0).all() and (go[:, outside.numpy()] == 0).all()


def test_row_slices_of_a_truncated_sequence_equal_the_full_sequence():
    """The slicing rule the full-size GPU tests rely on (helpers.slice_window / check_chain_slice): the oracle run on
    positions [r0 - 2w, r1 + 2w) reproduces rows [r0, r1) of all six results of the chain on the whole sequence."""
    import torch

    import helpers as H

    B, M, N, w = 2, 96, 8, 5
    d = H.rand_inputs(B, M, N, w, seed=3)
    q, kt, v, go = (torch.from_numpy(d[k]) for k in ("q", "kt", "v", "g_out"))
    k = np.ascontiguousarray(d["kt"].transpose(0, 2, 1))
    a, o, gq, gk, ga, gv = oracle.chain_fwd_bwd(d["q"], k, d["v"], w, d["g_out"])
    got = {name: torch.from_numpy(np.ascontiguousarray(x)) for name, x in
           dict(a=a, o=o, gq=gq, gk=gk.transpose(0, 2, 1), ga=ga, gv=gv).items()}
    for b, r0, r1 in ((0, 0, 7), (1, 30, 41), (1, 80, 96), (0, 0, 96), (0, 9, 10)):
        H.check_chain_slice(got, q, kt, v, go, w, b, r0, r1, rel=1e-6)
    # and the check does notice a wrong row just inside a slice
    bad = dict(got, gv=got["gv"].clone())
    bad["gv"][1, 40] += 0.5
    import pytest

    with pytest.raises(AssertionError):
        H.check_chain_slice(bad, q, kt, v, go, w, 1, 30, 41, rel=1e-6)
    H.check_chain_slice(bad, q, kt, v, go, w, 1, 41, 52, rel=1e-6)   # ... and only there
