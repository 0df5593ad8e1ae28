"""ctypes binding of the C ABI declared in include/wmm_b200.h (libwmm_b200.so, built by build.py).

There is no fallback: if the library is missing, importing this module raises, and every operator of
the package with it.  Tensors cross the boundary as (device pointer, element strides); torch is used
for device memory and streams only.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# WMM_B200_LIBRARY may name a variant build of the same ABI (e.g. one compiled with -DWMM_TRACE for kernel timelines).
LIB_PATH = os.environ.get("WMM_B200_LIBRARY") or os.path.join(_HERE, "libwmm_b200.so")

F16, BF16, F32, F64 = 0, 1, 2, 3
FLAG_SPLIT_ROUNDING = 1 << 0
FLAG_FORCE_GENERIC = 1 << 1
FLAG_REQUIRE_TENSOR = 1 << 2
FLAG_SOFTMAX_KEEP_PADDING = 1 << 3
FLAG_PREFER_SWEEP = 1 << 4
FLAG_TF32 = 1 << 5
BAND_NT, BAND_N, BAND_T = 1, 2, 3

_DTYPES = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32, torch.float64: F64}


class Operand(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("stride_b", ctypes.c_int64),
        ("stride_r", ctypes.c_int64),
        ("stride_c", ctypes.c_int64),
    ]


class Geometry(ctypes.Structure):
    _fields_ = [
        ("batch", ctypes.c_int32),
        ("rows", ctypes.c_int32),
        ("cols", ctypes.c_int32),
        ("window", ctypes.c_int32),
        ("other_rows", ctypes.c_int32),
        ("other_off", ctypes.c_int32),
        ("seq_lo", ctypes.c_int32),
        ("seq_hi", ctypes.c_int32),
        ("band_stride_b", ctypes.c_int64),
    ]


class HaloBuffer(ctypes.Structure):
    """wmm_halo_buffer of include/wmm_b200.h."""
    _fields_ = [("local", ctypes.c_void_p), ("lower", ctypes.c_void_p), ("upper", ctypes.c_void_p)]


class HaloEdges(ctypes.Structure):
    """wmm_halo_edges of include/wmm_b200.h."""
    _fields_ = [("local", ctypes.c_void_p), ("mine", ctypes.c_void_p), ("lower", ctypes.c_void_p), ("upper", ctypes.c_void_p)]


class HaloFlags(ctypes.Structure):
    """wmm_halo_flags of include/wmm_b200.h."""
    _fields_ = [("mine", ctypes.c_void_p), ("lower", ctypes.c_void_p), ("upper", ctypes.c_void_p), ("counters", ctypes.c_void_p)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "window_matmul: native library %s is missing; build it with "
            "`python pytorch-window-matmul_b200/build.py` (there is no non-CUDA fallback)" % LIB_PATH
        )
    lib = ctypes.CDLL(LIB_PATH)
    P = ctypes.POINTER
    vp, i32, u32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint
    lib.wmm_version.restype = i32
    lib.wmm_version.argtypes = []
    lib.wmm_last_error_string.restype = ctypes.c_char_p
    lib.wmm_last_error_string.argtypes = []
    lib.wmm_status_string.restype = ctypes.c_char_p
    lib.wmm_status_string.argtypes = [i32]
    lib.wmm_launch_count.restype = ctypes.c_uint64
    lib.wmm_launch_count.argtypes = []
    lib.wmm_set_cta_limits.restype = i32
    lib.wmm_set_cta_limits.argtypes = [i32, i32]
    lib.wmm_device_status.restype = ctypes.c_int64
    lib.wmm_device_status.argtypes = [i32]
    lib.wmm_query_path.restype = i32
    lib.wmm_query_path.argtypes = [i32, P(Operand), P(Operand), vp, P(Geometry), i32, u32]
    lib.wmm_band_nt.restype = i32
    lib.wmm_band_nt.argtypes = [P(Operand), P(Operand), vp, P(Geometry), i32, u32, vp]
    lib.wmm_band_n.restype = i32
    lib.wmm_band_n.argtypes = [vp, P(Operand), P(Operand), P(Geometry), i32, u32, vp]
    lib.wmm_band_t.restype = i32
    lib.wmm_band_t.argtypes = [vp, P(Operand), P(Operand), P(Geometry), i32, u32, vp]
    lib.wmm_window_bwd.restype = i32
    lib.wmm_window_bwd.argtypes = [P(Operand), P(Operand), vp, P(Operand), P(Operand), P(Geometry), i32, u32, vp]
    lib.wmm_unwindow_bwd.restype = i32
    lib.wmm_unwindow_bwd.argtypes = [vp, P(Operand), P(Operand), vp, P(Operand), P(Geometry), i32, u32, vp]
    lib.wmm_halo_pull.restype = i32
    lib.wmm_halo_pull.argtypes = [P(HaloBuffer), i32, P(HaloFlags), i32, i32, i32, i32, i32, i32, vp]
    lib.wmm_halo_pull_static.restype = i32
    lib.wmm_halo_pull_static.argtypes = [P(HaloBuffer), i32, P(HaloFlags), i32, i32, i32, i32, i32, i32, i32, vp]
    lib.wmm_band_t_edges.restype = i32
    lib.wmm_band_t_edges.argtypes = [vp, P(Operand), P(Operand), vp, i32, i32, P(Geometry), i32, u32, vp]
    lib.wmm_halo_reduce_edges.restype = i32
    lib.wmm_halo_reduce_edges.argtypes = [P(HaloEdges), i32, P(HaloFlags), i32, i32, i32, i32, i32, vp]
    lib.wmm_band_softmax.restype = i32
    lib.wmm_band_softmax.argtypes = [vp, vp, P(Geometry), i32, ctypes.c_float, u32, vp]
    lib.wmm_band_softmax_bwd.restype = i32
    lib.wmm_band_softmax_bwd.argtypes = [vp, vp, vp, P(Geometry), i32, ctypes.c_float, u32, vp]
    if lib.wmm_version() != 3:
        raise RuntimeError("window_matmul: %s has ABI version %d, expected 3" % (LIB_PATH, lib.wmm_version()))
    return lib


lib = _load()


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise RuntimeError('"window_matmul" not implemented for \'%s\'' % str(t.dtype).replace("torch.", ""))


def operand(t: torch.Tensor, swap_inner: bool = False) -> Operand:
    """(batch, rows, cols) view of a 3-D tensor; swap_inner presents a (B, cols, rows) tensor that way."""
    sb, sr, sc = t.stride()
    if swap_inner:
        sr, sc = sc, sr
    return Operand(t.data_ptr(), sb, sr, sc)


def geometry(batch, rows, cols, window, other_rows=None, other_off=0, seq=None, band_stride_b=0) -> Geometry:
    other_rows = rows if other_rows is None else other_rows
    lo, hi = (0, other_rows) if seq is None else seq
    return Geometry(batch, rows, cols, window, other_rows, other_off, lo, hi, band_stride_b)


def stream_of(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def check(status: int) -> None:
    if status != 0:
        raise RuntimeError(
            "%s (%s)" % (lib.wmm_last_error_string().decode(), lib.wmm_status_string(status).decode())
        )


def launch_count() -> int:
    return int(lib.wmm_launch_count())


class cta_limits:
    """`with cta_limits(140, 16): ...` caps the grids of the contractions / exchanges launched (or captured) inside the
    block (wmm_set_cta_limits) and lifts the caps afterwards.  Process-wide: not for threads that launch concurrently."""

    def __init__(self, contraction_ctas: int = 0, exchange_ctas: int = 0):
        self.c, self.x = int(contraction_ctas), int(exchange_ctas)

    def __enter__(self):
        check(lib.wmm_set_cta_limits(self.c, self.x))
        return self

    def __exit__(self, *exc):
        lib.wmm_set_cta_limits(0, 0)
        return False


def device_status(clear: bool = True) -> int:
    r = int(lib.wmm_device_status(1 if clear else 0))
    if r < 0:
        check(r)
    return r
