"""The band softmax (wmm_band_softmax / wmm_band_softmax_bwd) against the float64 oracle on the same inputs.

Tolerances: float32 |err| <= 1e-6 + 1e-5|x| (probabilities are <= 1, so this is ~10 ulp at the top); float64 1e-12;
16-bit results carry one rounding of the output (2^-8 relative for bfloat16, 2^-11 for float16) plus the fast exponential
of the 16-bit kernels: |err| <= 1e-2|x| + 1e-6 for bfloat16, 2e-3|x| + 1e-6 for float16.
"""
import math

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

# (B, M, w): row lengths that need 1, 2, 3, 4, 6, 8, 12 and 16 vectors per lane and the looping kernel, sequences shorter
# than the window, the windows of the benchmark configurations
SHAPES = [(3, 5, 1), (2, 40, 4), (2, 33, 17), (2, 130, 64), (1, 300, 256), (1, 200, 384), (1, 70, 512), (1, 40, 700),
          (1, 24, 1100), (1, 16, 1500), (1, 12, 2100), (2, 9, 12), (4, 2048, 8)]

TOL = {torch.float32: (1e-5, 1e-6), torch.float64: (1e-12, 1e-14), torch.bfloat16: (1e-2, 1e-6),
       torch.float16: (2e-3, 1e-6)}


@pytest.fixture(scope="module")
def sm():
    from window_matmul import softmax

    return softmax


def _close(got, want, dtype, what):
    rtol, atol = TOL[dtype]
    g = got.detach().double().cpu().numpy()
    err = np.abs(g - want)
    bound = atol + rtol * np.abs(want)
    assert (err <= bound).all(), "%s: worst err/bound %.2f (max abs err %.3e)" % (what, (err / bound).max(), err.max())


def _scores(B, M, w, dtype, seed=11, spread=3.0):
    g = torch.Generator().manual_seed(seed)
    s = torch.randn(B, M, 2 * w + 1, generator=g) * spread
    gp = torch.randn(B, M, 2 * w + 1, generator=g)
    return s.to(dtype), gp.to(dtype)


@pytest.mark.parametrize("mask", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("shape", SHAPES)
def test_band_softmax_forward_backward(sm, shape, dtype, mask):
    B, M, w = shape
    s, gp = _scores(B, M, w, dtype)
    scale = 1.0 / math.sqrt(64)
    want_p = H.oracle.band_softmax(s.double().numpy(), scale, mask)
    sd, gd = s.cuda(), gp.cuda()
    out = torch.full_like(sd, float("nan"))           # every element must be written
    p = sm.band_softmax(sd, scale, mask, out=out)
    torch.cuda.synchronize()
    _close(p, want_p, dtype, "probabilities")
    if mask:
        outside = H.out_of_sequence_mask(M, w)
        assert (p.double().cpu().numpy()[:, outside] == 0).all()
    # the backward is checked on the probabilities the kernel itself produced (what autograd hands it)
    want_g = H.oracle.band_softmax_backward(p.double().cpu().numpy(), gp.double().numpy(), scale, mask)
    gs = sm.band_softmax_backward(p, gd, scale, mask, out=torch.full_like(sd, float("nan")))
    torch.cuda.synchronize()
    rtol, atol = TOL[dtype]
    g = gs.double().cpu().numpy()
    # a gradient is a difference of products: bound it by the magnitude of its terms, scale * p * (|g| + |dot|)
    pd, gpd = p.double().cpu().numpy(), gp.double().numpy()
    dot = (pd * gpd).sum(-1, keepdims=True)
    bound = atol + rtol * abs(scale) * pd * (np.abs(gpd) + np.abs(dot)) * 4
    assert (np.abs(g - want_g) <= bound).all(), "gradient: worst %.2f" % (np.abs(g - want_g) / bound).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_band_softmax_in_place_and_poisoned_padding(sm, dtype):
    """In place, and with NaN stored in the out-of-sequence slots of the scores and of the incoming gradient: the masked
    softmax never lets them through (window_matmul writes zeros there, but a caller's own band tensor may hold anything)."""
    B, M, w = 2, 96, 40
    s, gp = _scores(B, M, w, dtype, seed=5)
    outside = torch.from_numpy(H.out_of_sequence_mask(M, w))
    want_p = H.oracle.band_softmax(s.double().numpy(), 0.5, True)
    s[:, outside] = float("nan")
    gp_poisoned = gp.clone()
    gp_poisoned[:, outside] = float("inf")
    sd = s.cuda()
    p = sm.band_softmax(sd, 0.5, True, out=sd)
    assert p.data_ptr() == sd.data_ptr()
    _close(p, want_p, dtype, "in place")
    want_g = H.oracle.band_softmax_backward(p.double().cpu().numpy(), gp.double().numpy(), 0.5, True)
    gd = gp_poisoned.cuda()
    gs = sm.band_softmax_backward(p, gd, 0.5, True, out=gd)
    assert torch.isfinite(gs.float()).all()
    rtol, atol = TOL[dtype]
    assert np.abs(gs.double().cpu().numpy() - want_g).max() <= 4 * rtol + atol


def test_band_softmax_shard_geometry(sm):
    """Rows of a sequence shard: the in-sequence rule uses the shard's offset and range, as in the three primitives."""
    B, M, w = 2, 160, 24
    s, _ = _scores(B, M, w, torch.float32, seed=9)
    want = H.oracle.band_softmax(s.double().numpy(), 1.0, True)
    lo_rows = slice(0, 64)
    hi_rows = slice(64, 160)
    sd = s.cuda()
    # first shard: rows 0..63, halo buffer of 64 + 2w rows whose first w are before the sequence
    p0 = sm.band_softmax(sd[:, lo_rows].contiguous(), 1.0, True, other_off=w, other_rows=64 + 2 * w, seq=(w, 64 + 2 * w))
    # second shard: rows 64..159, the sequence ends w rows before the end of its halo buffer
    p1 = sm.band_softmax(sd[:, hi_rows].contiguous(), 1.0, True, other_off=w, other_rows=96 + 2 * w, seq=(0, 96 + w))
    _close(torch.cat([p0, p1], 1), want, torch.float32, "sharded rows")


@pytest.mark.parametrize("dtype,mask", [(torch.float32, False), (torch.float32, True), (torch.bfloat16, True)])
def test_attention_block_with_fused_softmax(sm, dtype, mask):
    """window_matmul -> window_softmax -> unwindow_matmul, forward and backward through autograd, against the same
    block written with torch ops in float64 (the composition of the reference's tests/test_attention.py:48-70)."""
    from window_matmul import unwindow_matmul, window_matmul, window_softmax

    B, H_, M, Nn, w = 2, 2, 192, 64, 32
    g = torch.Generator().manual_seed(21)
    q, k, v, go = (torch.randn(B, H_, M, Nn, generator=g).to(dtype) for _ in range(4))
    scale = 1.0 / math.sqrt(Nn)

    def dense(qq, kk, vv):
        s = qq @ kk.transpose(-1, -2)                       # (B,H,M,M)
        i = torch.arange(M)[:, None]
        j = torch.arange(M)[None, :]
        inside = (j - i).abs() <= w
        if mask:
            pr = torch.softmax((s * scale).masked_fill(~inside, float("-inf")), -1)
        else:
            # padding slots take part with score 0: add their count to the denominator
            npad = (2 * w + 1 - inside.sum(-1)).double()
            e = torch.exp(s * scale - 0.0) * inside
            pr = e / (e.sum(-1, keepdim=True) + npad[:, None])
        return pr @ vv

    qd, kd, vd = (t.double().requires_grad_() for t in (q, k, v))
    od = dense(qd, kd, vd)
    od.backward(go.double())

    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    a = window_matmul(qc, kc.transpose(-1, -2), w)
    p = window_softmax(a, scale, mask)
    o = unwindow_matmul(p, vc, w)
    o.backward(go.cuda())
    torch.cuda.synchronize()
    rel = 1e-4 if dtype == torch.float32 else 3e-2
    for name, got, want in (("o", o, od), ("gq", qc.grad, qd.grad), ("gk", kc.grad, kd.grad), ("gv", vc.grad, vd.grad)):
        H.assert_lowp_close(got, want.detach().numpy(), name, rel=rel)


def test_band_softmax_rejects_bad_arguments(sm):
    with pytest.raises(RuntimeError):
        sm.band_softmax(torch.zeros(1, 4, 8, device="cuda"))          # even row length is not a band
    with pytest.raises(RuntimeError):
        sm.band_softmax(torch.zeros(1, 4, 9))                          # CPU tensor
    with pytest.raises(RuntimeError):
        sm.band_softmax_backward(torch.zeros(1, 4, 9, device="cuda"), torch.zeros(1, 4, 7, device="cuda"))
    assert sm.window_softmax(torch.zeros(0, 4, 9, device="cuda")).shape == (0, 4, 9)
