"""Shared helpers of the parity tests: seeded inputs, the oracle as checker, comparison rules."""
import numpy as np
import torch

from oracle import oracle

# Tolerances (north star of this build): exact-order fp32 within rtol 1e-5 / atol 1e-6 of the reference;
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
