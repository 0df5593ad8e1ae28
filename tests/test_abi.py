"""CPU-side checks of the native boundary: the library loads, exports every symbol the public header
declares, and validates arguments without touching a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "wmm_b200.h")


def _declared():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"WMM_API\s+[\w\s\*]+?\b(wmm_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared()
    for n in ("wmm_band_nt", "wmm_band_n", "wmm_band_t", "wmm_window_bwd", "wmm_unwindow_bwd", "wmm_version",
              "wmm_last_error_string", "wmm_band_softmax", "wmm_band_softmax_bwd", "wmm_query_path", "wmm_device_status"):
        assert n in names


def test_library_exports_every_declared_symbol():
    from window_matmul import _native as N

    lib = ctypes.CDLL(N.LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), name
    assert lib.wmm_version() == 3


def test_cta_limits_are_validated_and_reset():
    from window_matmul import _native as N

    assert N.lib.wmm_set_cta_limits(-1, 0) == -2 and b">= 0" in N.lib.wmm_last_error_string()
    assert N.lib.wmm_set_cta_limits(0, -3) == -2
    with N.cta_limits(140, 16):
        pass
    assert N.lib.wmm_set_cta_limits(0, 0) == 0


def test_edge_row_entry_points_validate_without_a_gpu():
    import ctypes as C

    from window_matmul import _native as N

    g = N.geometry(2, 256, 64, 64, 384, 64, (0, 384), 0)
    x = N.Operand(4096, 256 * 64, 64, 1)
    o = N.Operand(8192, 384 * 64, 64, 1)
    # (status, message): NULL edges, misaligned, too many rows, wrong dtype
    assert N.lib.wmm_band_t_edges(1024, C.byref(x), C.byref(o), None, 128, 64, g, N.BF16, 0, None) == -1
    assert N.lib.wmm_band_t_edges(1024, C.byref(x), C.byref(o), 4100, 128, 64, g, N.BF16, 0, None) == -4
    assert N.lib.wmm_band_t_edges(1024, C.byref(x), C.byref(o), 4096, 200, 0, g, N.BF16, 0, None) == -2
    assert N.lib.wmm_band_t_edges(1024, C.byref(x), C.byref(o), 4096, 128, 128, g, N.BF16, 0, None) == -2   # nothing left to write
    assert N.lib.wmm_band_t_edges(1024, C.byref(x), C.byref(o), 4096, 128, 64, g, N.F32, 0, None) == -7
    assert b"edge rows" in N.lib.wmm_last_error_string()
    e = (N.HaloEdges * 1)(N.HaloEdges(256, 512, 768, 1024))
    fl = N.HaloFlags(2048, 4096, 8192, 16384)
    assert N.lib.wmm_halo_reduce_edges(e, 1, C.byref(fl), 2, 256, 64, 64, N.F32, None) == -7
    assert N.lib.wmm_halo_reduce_edges(e, 1, C.byref(fl), 2, 100, 64, 64, N.BF16, None) == -2      # shard shorter than 2w
    assert N.lib.wmm_halo_reduce_edges(e, 1, C.byref(fl), 2, 256, 60, 64, N.BF16, None) == -4      # row not a multiple of 16 B
    assert N.lib.wmm_halo_reduce_edges(e, 1, C.byref(fl), 0, 256, 64, 64, N.BF16, None) == 0       # nothing to do


def test_argument_validation_needs_no_gpu():
    from window_matmul import _native as N

    g = N.geometry(2, 8, 4, 2)
    op = N.Operand(0, 0, 0, 0)
    # NULL data pointers
    assert N.lib.wmm_band_nt(op, op, None, g, N.F32, 0, None) == -1
    assert b"NULL" in N.lib.wmm_last_error_string()
    # unknown dtype
    ok = N.Operand(256, 32, 4, 1)
    assert N.lib.wmm_band_nt(ok, ok, 256, g, 17, 0, None) == -3
    # sequence range outside the other operand's rows
    bad = N.geometry(2, 8, 4, 2, other_rows=8, seq=(0, 9))
    assert N.lib.wmm_band_n(256, ok, ok, bad, N.F32, 0, None) == -2
    assert b"Input mismatch" in N.lib.wmm_last_error_string()
    # negative window
    assert N.lib.wmm_band_t(256, ok, ok, N.geometry(2, 8, 4, -1), N.F32, 0, None) == -2
    # overlapping output
    assert N.lib.wmm_band_n(256, ok, N.Operand(256, 32, 0, 1), g, N.F32, 0, None) == -4
    # contradictory flags
    assert N.lib.wmm_band_nt(ok, ok, 256, g, N.F32, N.FLAG_FORCE_GENERIC | N.FLAG_REQUIRE_TENSOR, None) == -7
    # the fused backward entry points take the plain geometry only
    sharded = N.geometry(2, 8, 4, 2, other_rows=12, other_off=2)
    assert N.lib.wmm_window_bwd(ok, ok, 256, ok, ok, sharded, N.F32, 0, None) == -2
    # empty problems succeed without a launch
    before = N.launch_count()
    assert N.lib.wmm_band_nt(op, op, None, N.geometry(0, 8, 4, 2), N.F32, 0, None) == 0
    assert N.launch_count() == before
    assert N.lib.wmm_status_string(-6) == b"WMM_ERR_CUDA"


def test_band_batch_stride_validation_needs_no_gpu():
    from window_matmul import _native as N

    op = N.Operand(256, 64, 8, 1)
    g = N.geometry(2, 8, 8, 2, band_stride_b=8 * 5 - 1)           # smaller than one batch entry of the band
    assert N.lib.wmm_band_nt(op, op, 512, g, N.F32, 0, None) == -4
    assert b"batch stride" in N.lib.wmm_last_error_string()
    g = N.geometry(2, 8, 0, 2, band_stride_b=8 * 5 + 8)           # the softmax takes contiguous bands only
    assert N.lib.wmm_band_softmax(256, 256, g, N.BF16, 1.0, 0, None) == -4


def test_band_softmax_argument_validation_needs_no_gpu():
    from window_matmul import _native as N

    g = N.geometry(2, 8, 0, 2)
    assert N.lib.wmm_band_softmax(None, None, g, N.BF16, 1.0, 0, None) == -1          # NULL band pointers
    assert N.lib.wmm_band_softmax(256, 256, None, N.BF16, 1.0, 0, None) == -1         # NULL geometry
    assert N.lib.wmm_band_softmax(256, 264, g, N.BF16, 1.0, 0, None) == -4            # not 16-byte aligned
    assert b"16-byte" in N.lib.wmm_last_error_string()
    assert N.lib.wmm_band_softmax(256, 256, g, 9, 1.0, 0, None) == -3                 # unknown dtype
    assert N.lib.wmm_band_softmax(256, 256, g, N.BF16, float("nan"), 0, None) == -2   # NaN scale
    assert N.lib.wmm_band_softmax(256, 256, g, N.BF16, 1.0, N.FLAG_SPLIT_ROUNDING, None) == -7   # a flag of the contractions
    assert N.lib.wmm_band_softmax_bwd(256, None, 256, g, N.BF16, 1.0, 0, None) == -1  # backward needs both inputs
    before = N.launch_count()
    assert N.lib.wmm_band_softmax(None, None, N.geometry(0, 8, 0, 2), N.BF16, 1.0, 0, None) == 0   # empty: no launch
    assert N.launch_count() == before


def test_python_surface_matches_the_reference():
    import inspect

    import window_matmul as wm

    # the reference's two names (window_matmul/__init__.py:2-4) first, unchanged; the band softmax is an addition
    assert wm.__all__[:2] == ["window_matmul", "unwindow_matmul"]
    assert wm.__all__[2:] == ["window_softmax"]
    for fn in (wm.window_matmul, wm.unwindow_matmul):
        assert list(inspect.signature(fn).parameters) == ["inp", "other", "window_size"]
    assert list(inspect.signature(wm.window_softmax).parameters) == ["scores", "scale", "mask"]
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        wm.window_softmax(__import__("torch").zeros(1, 4, 9))


def test_cpu_tensors_are_refused_loudly():
    import torch

    import window_matmul as wm

    with pytest.raises(RuntimeError, match="CUDA tensor"):
        wm.window_matmul(torch.randn(2, 4, 3), torch.randn(2, 3, 4), 1)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        wm.unwindow_matmul(torch.randn(2, 4, 3), torch.randn(2, 4, 3), 1)
    # window_size == 0 never reaches the kernels (window_matmul/window_matmul.py:33-34, 69-70 of the reference)
    q, k = torch.randn(2, 4, 3), torch.randn(2, 3, 4)
    assert wm.window_matmul(q, k, 0).shape == (2, 4, 1)
    a, v = torch.randn(2, 4, 1), torch.randn(2, 4, 3)
    assert torch.equal(wm.unwindow_matmul(a, v, 0), a * v)


def test_public_header_is_plain_c_and_cxx(tmp_path):
    """include/wmm_b200.h is the whole contract of the native boundary: it must compile on its own as C and as C++
    (no torch, CUDA or project headers behind it)."""
    import shutil
    import subprocess

    if not shutil.which("gcc") or not shutil.which("g++"):
        pytest.skip("no host compiler")
    src = tmp_path / "use.c"
    src.write_text('#include "wmm_b200.h"\nint main(void) { wmm_geometry g = {1, 8, 4, 2, 8, 0, 0, 8, 0}; wmm_operand o = {0, 32, 4, 1};\n'
                   '  return (int)(g.window + o.stride_c) * 0 + (WMM_OK != 0) + (sizeof(wmm_geometry) != 40); }\n')
    inc = os.path.join(ROOT, "include")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-fsyntax-only", "-I", inc, str(src)], check=True)
    cxx = tmp_path / "use.cc"
    cxx.write_text(src.read_text())
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-I", inc, str(cxx)], check=True)


def test_halo_pull_argument_validation_needs_no_gpu():
    import ctypes as C

    from window_matmul import _native as N

    def call(bufs, flags, batch=2, rows=64, cols=8, window=16, dtype=N.BF16, acc=0):
        arr = (N.HaloBuffer * len(bufs))(*bufs)
        return N.lib.wmm_halo_pull(arr, len(bufs), C.byref(flags) if flags is not None else None, batch, rows, cols, window, dtype, acc, None)

    both = N.HaloFlags(1024, 2048, 4096, 8192)
    buf = N.HaloBuffer(256, 512, 768)
    assert call([buf], None) == -1                                         # no flags
    assert call([buf] * 5, both) == -2                                     # more than 4 buffers
    assert call([buf], both, dtype=11) == -3                               # unknown dtype
    assert call([buf], both, rows=8, window=16) == -2                      # shard shorter than the window
    assert call([buf], both, rows=24, window=16, acc=1) == -2              # reduction needs rows >= 2 w
    assert call([buf], both, cols=3) == -4                                 # rows that are not a multiple of 16 bytes
    assert call([N.HaloBuffer(260, 512, 768)], both) == -4                 # unaligned buffer
    assert call([N.HaloBuffer(256, None, 768)], both) == -1                # buffer and flags disagree on the neighbours
    assert call([N.HaloBuffer(None, 512, 768)], both) == -1                # no local buffer
    before = N.launch_count()
    assert call([buf], both, batch=0) == 0                                 # empty: no launch
    assert N.launch_count() == before


def test_caller_supplied_outputs_are_validated_before_any_launch():
    """The wrappers hand `out=` to the library as a bare pointer (plus strides for the operand outputs): shape, dtype,
    device and layout are checked in Python first, with the reference's error wording (cuda/utils.cuh:3-4)."""
    import importlib

    import torch

    from window_matmul import _native as N
    from window_matmul import softmax as sm

    impl = importlib.import_module("window_matmul.window_matmul")
    like = torch.zeros(2, 8, 4)
    before = N.launch_count()
    assert impl._check_out(torch.empty(2, 8, 5), (2, 8, 5), like, True) is not None
    bad_band = [torch.empty(2, 8, 7), torch.empty(2, 8, 5, dtype=torch.float64), torch.empty(2, 8, 10)[:, :, ::2],
                torch.empty(2, 8, 5, device="meta"), None]
    for out in bad_band:
        with pytest.raises(RuntimeError, match="Input mismatch"):
            impl._check_out(out, (2, 8, 5), like, True)
    # operand outputs may be strided views, but not of another shape, nor with overlapping elements
    assert impl._check_out(torch.empty(2, 8, 8)[:, :, :4], (2, 8, 4), like, False) is not None
    for out in (torch.empty(2, 9, 4), torch.empty(8, 4).expand(2, 8, 4), torch.empty(2, 8, 4, dtype=torch.float16)):
        with pytest.raises(RuntimeError, match="Input mismatch"):
            impl._check_out(out, (2, 8, 4), like, False)
    band = torch.zeros(2, 8, 5)
    for out in (torch.empty(2, 8, 7), torch.empty(2, 8, 5, dtype=torch.float16), torch.empty(2, 8, 10)[:, :, ::2],
                torch.empty(2 * 8 * 5 + 1)[1:].view(2, 8, 5)):
        with pytest.raises(RuntimeError, match="Input mismatch"):
            sm._check_out(out, band)
    assert N.launch_count() == before
