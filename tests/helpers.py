"""Shared helpers of the parity tests: seeded inputs, the oracle as checker, comparison rules."""
import numpy as np
import torch

from oracle import oracle

# Tolerances: exact-order fp32 within rtol 1e-5 / atol 1e-6 of the reference;
# 16-bit (fp32-accumulating tensor-core) results within 1e-2 relative of the fp32 reference on the
# same (rounded) inputs.
FP32_RTOL, FP32_ATOL = 1e-5, 1e-6
LOWP_REL = 1e-2


def rand_inputs(B, M, N, w, seed, dist="normal", scale=1.0):
    g = np.random.default_rng(seed)
    mk = (lambda *s: g.standard_normal(s)) if dist == "normal" else (lambda *s: g.random(s))
    d = dict(
        q=mk(B, M, N) * scale,
        kt=mk(B, M, N) * scale,
        v=mk(B, M, N) * scale,
        att=mk(B, M, 2 * w + 1),
        g_band=mk(B, M, 2 * w + 1),
        g_out=mk(B, M, N),
    )
    return {k: v.astype(np.float32) for k, v in d.items()}


def round_to(x: np.ndarray, dtype: torch.dtype) -> np.ndarray:
    """Rounds float32 values to `dtype` and back, so oracle and kernel see identical inputs."""
    return torch.from_numpy(x).to(dtype).to(torch.float32).numpy()


def to_dev(x: np.ndarray, dtype: torch.dtype, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x)).to(dtype).to(device)


def oracle_all(d, w, dtype=np.float32):
    """All six contractions from the oracle, in `dtype`.  k is passed as contiguous (B,N,M)."""
    c = {k: np.ascontiguousarray(v.astype(dtype)) for k, v in d.items()}
    k = np.ascontiguousarray(c["kt"].transpose(0, 2, 1))
    a = oracle.window_matmul_forward(c["q"], k, w)
    gq, gk = oracle.window_matmul_backward(c["q"], k, w, c["g_band"])
    o = oracle.unwindow_matmul_forward(c["att"], c["v"], w)
    gatt, gv = oracle.unwindow_matmul_backward(c["att"], c["v"], w, c["g_out"])
    return dict(a=a, gq=gq, gk=gk, o=o, gatt=gatt, gv=gv)


def assert_lowp_close(got: torch.Tensor, want: np.ndarray, what="", rel=LOWP_REL):
    """16-bit result vs fp32 reference: |got - want| <= rel * (|want| + rms(want))."""
    g = got.detach().float().cpu().numpy().astype(np.float64)
    wv = want.astype(np.float64)
    assert g.shape == wv.shape, (what, g.shape, wv.shape)
    rms = float(np.sqrt(np.mean(wv * wv))) if wv.size else 0.0
    err = np.abs(g - wv)
    bound = rel * (np.abs(wv) + rms) + 1e-30
    worst = float((err / bound).max()) if wv.size else 0.0
    assert worst <= 1.0, "%s: max err/bound %.3f (max abs err %.3e, rms %.3e)" % (what, worst, err.max(), rms)


def assert_fp32_close(got: torch.Tensor, want: np.ndarray, what=""):
    g = got.detach().cpu().numpy()
    assert g.shape == want.shape, (what, g.shape, want.shape)
    ok = np.abs(g.astype(np.float64) - want.astype(np.float64)) <= FP32_ATOL + FP32_RTOL * np.abs(want)
    assert ok.all(), "%s: %d of %d outside rtol 1e-5 / atol 1e-6, max abs %.3e" % (
        what, (~ok).sum(), ok.size, np.abs(g - want).max())


def assert_bit_equal(got: torch.Tensor, want: np.ndarray, what=""):
    g = got.detach().cpu().numpy()
    assert g.shape == want.shape and g.dtype == want.dtype, (what, g.shape, want.shape, g.dtype, want.dtype)
    # -0.0 == 0.0 is accepted; NaNs never appear in these inputs
    assert np.array_equal(g, want), "%s: %d of %d elements differ, max abs %.3e" % (
        what, (g != want).sum(), g.size, np.abs(g.astype(np.float64) - want.astype(np.float64)).max())


def out_of_sequence_mask(M, w):
    i = np.arange(M)[:, None]
    j = np.arange(2 * w + 1)[None, :]
    p = i + j - w
    return (p < 0) | (p >= M)


# ---- oracle parity on row slices of sequences too long for the CPU ------------------------------------------------


def slice_window(M, w, r0, r1):
    """Rows [r0, r1) of all six results of the chain depend on positions [r0 - 2w, r1 + 2w) only (the band rows that
    feed grad_K / grad_V of a position p are rows p-w .. p+w, and those rows see positions up to 2w away).  Returns
    the truncated range [t0, t1) clipped to the sequence: the oracle run on it gives the exact values of those rows,
    because for every band row within w of the slice the truncation cuts nothing the full sequence has."""
    return max(0, r0 - 2 * w), min(M, r1 + 2 * w)


def check_chain_slice(got, q, kt, v, go, w, b, r0, r1, rel=LOWP_REL, tag=""):
    """Compares rows [r0, r1) of batch entry b of the GPU's a, o, ga, gv, gq, gk with the oracle.

    `got`: GPU tensors a, ga (B,M,2w+1); o, gq, gv and gk (the gradient of K^T) (B,M,N).  q, kt, v, go: CPU tensors (B,M,N) holding the
    (already rounded) values the GPU consumed.  Every contraction is checked on ITS OWN inputs as the GPU saw them: the
    oracle of the second operator and of the backward passes is fed the GPU's rounded band tensors, so each result is
    within `rel` of the reference arithmetic on identical inputs."""
    M = q.shape[1]
    t0, t1 = slice_window(M, w, r0, r1)
    f = lambda t: np.ascontiguousarray(t[b:b + 1, t0:t1].float().cpu().numpy())  # noqa: E731
    qs, kts, vs, gos = f(q), f(kt), f(v), f(go)
    ks = np.ascontiguousarray(kts.transpose(0, 2, 1))
    a_gpu, ga_gpu = f(got["a"]), f(got["ga"])
    lo, hi = r0 - t0, r1 - t0
    what = "%sb=%d rows [%d,%d)" % (tag, b, r0, r1)
    a = oracle.window_matmul_forward(qs, ks, w)
    assert_lowp_close(got["a"][b:b + 1, r0:r1], a[:, lo:hi], what + " a", rel)
    o = oracle.unwindow_matmul_forward(a_gpu, vs, w)
    assert_lowp_close(got["o"][b:b + 1, r0:r1], o[:, lo:hi], what + " o", rel)
    ga, gv = oracle.unwindow_matmul_backward(a_gpu, vs, w, gos)
    assert_lowp_close(got["ga"][b:b + 1, r0:r1], ga[:, lo:hi], what + " ga", rel)
    assert_lowp_close(got["gv"][b:b + 1, r0:r1], gv[:, lo:hi], what + " gv", rel)
    gq, gk = oracle.window_matmul_backward(qs, ks, w, ga_gpu)
    assert_lowp_close(got["gq"][b:b + 1, r0:r1], gq[:, lo:hi], what + " gq", rel)
    assert_lowp_close(got["gk"][b:b + 1, r0:r1], gk.transpose(0, 2, 1)[:, lo:hi], what + " gk", rel)


def check_chain_slices(got, q, kt, v, go, w, cases, rel=LOWP_REL, tag=""):
    """check_chain_slice over (b, r0, r1) cases, on host threads (the oracle releases the GIL inside its C loops)."""
    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(max_workers=8) as ex:
        futs = [ex.submit(check_chain_slice, got, q, kt, v, go, w, b, r0, r1, rel, tag) for b, r0, r1 in cases]
        for fu in futs:
            fu.result()
