"""Generates tests/golden/reference_cpu.npz from the reference itself.

Run in a container that has the reference tree and its compiled module (oracle/build_ref.py builds
oracle/_ref/window_matmul_kernel.so from the unmodified sources):

    python tests/golden/make_golden.py

For every case the four entry points of the reference's pybind module
(csrc/window_matmul/window_matmul.cpp:100-106) are run on its CPU path
(csrc/window_matmul/cpu/window_matmul_cpu.cpp) and inputs and outputs are stored.  The shapes are the
reference's own test parameters (tests/conftest.py:5-13: DIMS x WINDOW_SIZES without w = 0, which never
reaches the kernels) in float32, a subset in float64 and float16, and a few ragged extras.  The band
input of the unwindow cases holds non-zero values in its out-of-sequence slots, which pins that the
reference never reads them.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
import window_matmul_kernel as ref  # noqa: E402  (the reference's own module)

REF_DIMS = [(2, 1, 3), (2, 4, 3), (2, 16, 3), (2, 32, 3), (2, 16, 32)]  # (batch*heads, seq, hidden)
REF_WINDOWS = [1, 4, 16]
EXTRA = [(1, 130, 8, 5), (2, 70, 20, 33), (1, 150, 32, 40), (3, 5, 7, 9), (1, 257, 16, 8)]


def cases():
    out = []
    for (b, m, n) in REF_DIMS:
        for w in REF_WINDOWS:
            out.append((b, m, n, w, "float32"))
    for (b, m, n) in [(2, 16, 3), (2, 16, 32), (2, 4, 3)]:
        for w in [1, 4, 16]:
            out.append((b, m, n, w, "float64"))
            out.append((b, m, n, w, "float16"))
    for (b, m, n, w) in EXTRA:
        out.append((b, m, n, w, "float32"))
    out.append((1, 130, 8, 5, "float16"))
    return out


def main():
    store = {}
    names = []
    for idx, (b, m, n, w, dt) in enumerate(cases()):
        rng = np.random.default_rng(1000 + idx)
        W = 2 * w + 1
        mk = lambda *s: rng.standard_normal(s).astype(dt)  # noqa: E731
        q, k, v = mk(b, m, n), mk(b, n, m), mk(b, m, n)
        att, g_band, g_out = mk(b, m, W), mk(b, m, W), mk(b, m, n)
        tq, tk, tv, ta, tgb, tgo = (torch.from_numpy(x) for x in (q, k, v, att, g_band, g_out))
        a = ref.window_matmul_forward(tq, tk, w)
        gq, gk = ref.window_matmul_backward(tq, tk, w, tgb)
        o = ref.unwindow_matmul_forward(ta, tv, w)
        gatt, gv = ref.unwindow_matmul_backward(ta, tv, w, tgo)
        name = "c%02d_b%d_m%d_n%d_w%d_%s" % (idx, b, m, n, w, dt)
        names.append(name)
        for key, val in dict(q=q, k=k, v=v, att=att, g_band=g_band, g_out=g_out, a=a, gq=gq, gk=gk, o=o,
                             gatt=gatt, gv=gv).items():
            arr = val.numpy() if isinstance(val, torch.Tensor) else val
            store[name + "/" + key] = np.ascontiguousarray(arr)
    store["names"] = np.array(names)
    path = os.path.join(HERE, "reference_cpu.npz")
    np.savez_compressed(path, **store)
    print(path, os.path.getsize(path), "bytes,", len(names), "cases")


if __name__ == "__main__":
    main()
