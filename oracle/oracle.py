"""ctypes/numpy front end of the CPU oracle (oracle/wmm_oracle.c).  TEST INFRASTRUCTURE ONLY.

Mirrors the four entry points of the reference's pybind module (csrc/window_matmul/window_matmul.cpp:100-106)
on numpy arrays: float32, float64 and float16 exactly as the reference's CPU path computes them
(csrc/window_matmul/cpu/window_matmul_cpu.cpp); bfloat16 has no reference implementation, so 16-bit GPU
results are checked against the float32/float64 oracle on the rounded inputs.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_SUF = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64", np.dtype(np.float16): "f16"}


def build() -> str:
    subprocess.run(["make", "-s", "-C", _HERE, "libwmm_oracle.so"], check=True)
    return os.path.join(_HERE, "libwmm_oracle.so")


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libwmm_oracle.so")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(os.path.join(_HERE, "wmm_oracle.c")):
            build()
        _LIB = ctypes.CDLL(path)
    return _LIB


def _fn(name, dt):
    f = getattr(_lib(), "wmm_oracle_%s_%s" % (name, _SUF[np.dtype(dt)]))
    f.restype = None
    return f


def _p(a):
    return ctypes.c_void_p(a.ctypes.data)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def window_matmul_forward(src, other, w):
    """src (B,M,N), other (B,N,M) -> (B,M,2w+1).  window_matmul_cpu.cpp:6-50."""
    dt = src.dtype
    src, other = _c(src, dt), _c(other, dt)
    B, M, N = src.shape
    assert other.shape == (B, N, M)
    out = np.empty((B, M, 2 * w + 1), dtype=dt)
    _fn("window_fw", dt)(_p(src), _p(other), _p(out), B, M, N, w)
    return out


def window_matmul_backward(src, other, w, gout):
    """-> (grad_src (B,M,N), grad_other (B,N,M)).  window_matmul_cpu.cpp:52-99."""
    dt = src.dtype
    src, other, gout = _c(src, dt), _c(other, dt), _c(gout, dt)
    B, M, N = src.shape
    assert other.shape == (B, N, M) and gout.shape == (B, M, 2 * w + 1)
    gs, go = np.empty((B, M, N), dtype=dt), np.empty((B, N, M), dtype=dt)
    _fn("window_bw", dt)(_p(src), _p(other), _p(gout), _p(gs), _p(go), B, M, N, w)
    return gs, go


def unwindow_matmul_forward(band, other, w):
    """band (B,M,2w+1), other (B,M,N) -> (B,M,N).  window_matmul_cpu.cpp:101-144."""
    dt = band.dtype
    band, other = _c(band, dt), _c(other, dt)
    B, M, N = other.shape
    assert band.shape == (B, M, 2 * w + 1)
    out = np.empty((B, M, N), dtype=dt)
    _fn("unwindow_fw", dt)(_p(band), _p(other), _p(out), B, M, N, w)
    return out


def unwindow_matmul_backward(band, other, w, gout):
    """-> (grad_band (B,M,2w+1), grad_other (B,M,N)).  window_matmul_cpu.cpp:146-193."""
    dt = band.dtype
    band, other, gout = _c(band, dt), _c(other, dt), _c(gout, dt)
    B, M, N = other.shape
    assert band.shape == (B, M, 2 * w + 1) and gout.shape == (B, M, N)
    gb, go = np.empty((B, M, 2 * w + 1), dtype=dt), np.empty((B, M, N), dtype=dt)
    _fn("unwindow_bw", dt)(_p(band), _p(other), _p(gout), _p(gb), _p(go), B, M, N, w)
    return gb, go


def chain_fwd_bwd(q, k, v, w, gout):
    """window -> unwindow -> backward, the chain bench.py times.  k is (B,N,M).
    Returns a, o, gq, gk, ga, gv."""
    a = window_matmul_forward(q, k, w)
    o = unwindow_matmul_forward(a, v, w)
    ga, gv = unwindow_matmul_backward(a, v, w, gout)
    gq, gk = window_matmul_backward(q, k, w, ga)
    return a, o, gq, gk, ga, gv


def band_softmax(scores, scale=1.0, mask=True):
    """float64 softmax over the band (any leading dims folded into B): scores (B,M,2w+1) -> probabilities."""
    x = _c(scores, np.float64)
    B, M, W = x.shape
    out = np.empty_like(x)
    f = _lib().wmm_oracle_band_softmax_f64
    f.restype = None
    f(_p(x), _p(out), ctypes.c_long(B), ctypes.c_long(M), ctypes.c_long((W - 1) // 2), ctypes.c_double(scale),
      ctypes.c_int(1 if mask else 0))
    return out


def band_softmax_backward(probs, grad_probs, scale=1.0, mask=True):
    p, g = _c(probs, np.float64), _c(grad_probs, np.float64)
    B, M, W = p.shape
    out = np.empty_like(p)
    f = _lib().wmm_oracle_band_softmax_bw_f64
    f.restype = None
    f(_p(p), _p(g), _p(out), ctypes.c_long(B), ctypes.c_long(M), ctypes.c_long((W - 1) // 2), ctypes.c_double(scale),
      ctypes.c_int(1 if mask else 0))
    return out
