"""The reference's Python surface (window_matmul/window_matmul.py:1-76), rewired to the C ABI.

Same names, argument meaning, shapes, dtype rule and error type as the reference:
  window_matmul(inp (*,M,N), other (*,N,M), w)   -> (*,M,2w+1)     window_matmul.py:30-40
  unwindow_matmul(inp (*,M,2w+1), other (*,M,N), w) -> (*,M,N)     window_matmul.py:66-76
both differentiable in their two tensors (window_matmul.py:7-27, 43-63), with the window_size == 0
shortcuts of :33-34 and :69-70 and the fp16 cast under autocast of :9 and :45.
Differences, all on purpose: bfloat16 is supported; CUDA tensors only (there is no CPU path, a CPU tensor
raises RuntimeError); kernels run on torch's current stream instead of the legacy default stream
(csrc/window_matmul/cuda/window_matmul_cuda.cu:263); K is consumed in either memory order without the
transposing copy of window_matmul_cuda.cu:236; a gradient that autograd does not need is not computed.
"""
from typing import Optional, Tuple

import torch

from . import _native as N

# Process-wide flags OR-ed into every call made through the operators below (see include/wmm_b200.h).
# Set with set_flags(); meant for tests and for choosing the exact-order fp32 kernels.
_FLAGS = 0


def set_flags(flags: int) -> int:
    """Sets the flags passed with every operator call; returns the previous value."""
    global _FLAGS
    old, _FLAGS = _FLAGS, int(flags)
    return old


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("window_matmul: tensor must be CUDA tensor (this package has no CPU path)")
    dev, dt = tensors[0].device, tensors[0].dtype
    for t in tensors[1:]:
        if t.device != dev:
            raise RuntimeError("window_matmul: tensors are on different devices")
        if t.dtype != dt:
            raise RuntimeError("expected scalar type %s but found %s" % (dt, t.dtype))


def _mismatch(cond: bool) -> None:
    if not cond:
        raise RuntimeError("Input mismatch")


def _check_out(out: torch.Tensor, shape, like: torch.Tensor, band: bool) -> torch.Tensor:
    """A caller-supplied output must be exactly what the kernel is about to write: the library sees only a pointer
    (and, for the operand outputs, strides), so a wrong shape, dtype or device would be an out-of-bounds device write."""
    _mismatch(isinstance(out, torch.Tensor) and tuple(out.shape) == tuple(shape))
    _mismatch(out.dtype == like.dtype and out.device == like.device)
    if band:        # band outputs: contiguous (B, M, 2w+1), or a range of rows of such a tensor (see _band_stride)
        _mismatch(_band_stride(out) is not None)
    else:           # operand outputs go through their strides; elements must not overlap
        _mismatch(all(st > 0 for st, n in zip(out.stride(), out.shape) if n > 1))
    return out


def _band_stride(t: torch.Tensor):
    """Batch stride to pass for a band tensor (B, M, 2w+1): 0 for a contiguous one, the stride of dim 0 for a range of rows
    cut out of a longer band tensor (rows and slots dense, batch entries further apart), None for anything else."""
    if t.is_contiguous():
        return 0
    B, M, W = t.shape
    if t.stride(2) == 1 and t.stride(1) == W and t.stride(0) >= M * W:
        return t.stride(0)
    return None


def _band_in(t: torch.Tensor):
    """A band operand as the kernels can read it: itself if dense or a row range of a dense tensor, else a copy."""
    sb = _band_stride(t)
    return (t, sb) if sb is not None else (t.contiguous(), 0)


def _addressable(t: torch.Tensor) -> torch.Tensor:
    """A 3-D operand the kernels can address well: one of the two inner strides is 1."""
    if t.stride(-1) == 1 or t.stride(-2) == 1:
        return t
    return t.contiguous()


# ---- the three primitives on 3-D tensors ---------------------------------------------------------


def band_nt(x, y, window, *, other_off=0, seq=None, out=None, flags=None):
    """Band[b,i,j] = X[b,i,:] . Y[b,i+j-w+other_off,:], zero outside seq.  x (B,M,N), y (B,Mo,N) -> (B,M,2w+1)."""
    _require_cuda(x, y)
    x, y = _addressable(x), _addressable(y)
    B, M, Nn = x.shape
    _mismatch(y.dim() == 3 and y.shape[0] == B and y.shape[2] == Nn)
    shape = (B, M, 2 * window + 1)
    band = torch.empty(shape, dtype=x.dtype, device=x.device) if out is None else _check_out(out, shape, x, True)
    g = N.geometry(B, M, Nn, window, y.shape[1], other_off, seq, _band_stride(band))
    with torch.cuda.device(x.device):
        N.check(N.lib.wmm_band_nt(N.operand(x), N.operand(y), band.data_ptr(), g, N.dtype_code(x),
                                  _FLAGS if flags is None else flags, N.stream_of(x)))
    return band


def band_n(band, y, window, *, rows_out=None, other_off=0, seq=None, out=None, flags=None):
    """Out[b,i,:] = sum_j Band[b,i,j] Y[b,i+j-w+other_off,:].  band (B,M,2w+1), y (B,Mo,N) -> (B,M,N)."""
    _require_cuda(band, y)
    (band, band_sb), y = _band_in(band), _addressable(y)
    B, M, W = band.shape
    _mismatch(W == 2 * window + 1 and y.dim() == 3 and y.shape[0] == B)
    Nn = y.shape[2]
    o = torch.empty((B, M, Nn), dtype=y.dtype, device=y.device) if out is None else _check_out(out, (B, M, Nn), y, False)
    g = N.geometry(B, M, Nn, window, y.shape[1], other_off, seq, band_sb)
    with torch.cuda.device(y.device):
        N.check(N.lib.wmm_band_n(band.data_ptr(), N.operand(y), N.operand(o), g, N.dtype_code(y),
                                 _FLAGS if flags is None else flags, N.stream_of(y)))
    return o


def band_t(band, x, window, *, other_rows=None, other_off=0, seq=None, out=None, flags=None, edges=None, edge_skip=0):
    """Out[b,p,:] = sum_i Band[b,i,p-other_off-i+w] X[b,i,:].  band (B,M,2w+1), x (B,M,N) -> (B,Mo,N).
    `edges`: a contiguous fp32 (B, 2r, N) tensor that receives the first and the last r output rows unrounded, minus
    the outermost `edge_skip` rows at each end (wmm_band_t_edges; 16-bit types on the tensor-core kernels only)."""
    _require_cuda(band, x)
    (band, band_sb), x = _band_in(band), _addressable(x)
    B, M, W = band.shape
    _mismatch(W == 2 * window + 1 and x.dim() == 3 and x.shape[0] == B and x.shape[1] == M)
    Nn = x.shape[2]
    Mo = M if other_rows is None else other_rows
    o = torch.empty((B, Mo, Nn), dtype=x.dtype, device=x.device) if out is None else _check_out(out, (B, Mo, Nn), x, False)
    g = N.geometry(B, M, Nn, window, Mo, other_off, seq, band_sb)
    if edges is not None:
        _mismatch(edges.dim() == 3 and edges.shape[0] == B and edges.shape[2] == Nn and edges.shape[1] % 2 == 0
                  and 0 < edges.shape[1] <= Mo and edges.dtype == torch.float32 and edges.device == x.device
                  and edges.is_contiguous() and edges.data_ptr() % 16 == 0)
    with torch.cuda.device(x.device):
        if edges is not None:
            N.check(N.lib.wmm_band_t_edges(band.data_ptr(), N.operand(x), N.operand(o), edges.data_ptr(), edges.shape[1] // 2, int(edge_skip), g,
                                           N.dtype_code(x), _FLAGS if flags is None else flags, N.stream_of(x)))
        else:
            N.check(N.lib.wmm_band_t(band.data_ptr(), N.operand(x), N.operand(o), g, N.dtype_code(x),
                                     _FLAGS if flags is None else flags, N.stream_of(x)))
    return o


# ---- the four native calls of the reference's pybind module ---------------------------------------


def window_matmul_forward(src: torch.Tensor, other: torch.Tensor, window_size: int, out=None) -> torch.Tensor:
    """csrc/window_matmul/window_matmul.cpp:74-78 -> window_matmul_fw_cuda (window_matmul_cuda.cu:224-270).
    src (B,M,N), other (B,N,M) -> (B,M,2w+1)."""
    _mismatch(src.dim() == 3 and other.dim() == 3)
    _mismatch(src.size(0) == other.size(0) and src.size(1) == other.size(2) and src.size(2) == other.size(1))
    return band_nt(src, other.transpose(-1, -2), window_size, out=out)


def window_matmul_backward(src, other, window_size, grad_output, need=(True, True), out=None):
    """window_matmul.cpp:80-85 -> window_matmul_bw_cuda (window_matmul_cuda.cu:272-319).
    Returns (grad_src (B,M,N), grad_other (B,N,M)); like the reference's CUDA path, grad_other is a
    transposed view of a contiguous (B,M,N) buffer (window_matmul_cuda.cu:318).  `out` may give
    preallocated (grad_src (B,M,N), grad_other^T (B,M,N)) buffers."""
    _require_cuda(src, other, grad_output)
    _mismatch(src.dim() == 3 and other.dim() == 3 and grad_output.dim() == 3)
    _mismatch(src.size(0) == other.size(0) and src.size(1) == other.size(2) and src.size(2) == other.size(1))
    _mismatch(grad_output.shape == (src.size(0), src.size(1), 2 * window_size + 1))
    grad_output = grad_output.contiguous()
    kt = _addressable(other.transpose(-1, -2))
    src = _addressable(src)
    B, M, Nn = src.shape
    if need[0] and need[1]:
        gq = torch.empty((B, M, Nn), dtype=src.dtype, device=src.device) if out is None else _check_out(out[0], (B, M, Nn), src, False)
        gkt = torch.empty((B, M, Nn), dtype=src.dtype, device=src.device) if out is None else _check_out(out[1], (B, M, Nn), src, False)
        g = N.geometry(B, M, Nn, window_size)
        with torch.cuda.device(src.device):
            N.check(N.lib.wmm_window_bwd(N.operand(src), N.operand(kt), grad_output.data_ptr(), N.operand(gq),
                                         N.operand(gkt), g, N.dtype_code(src), _FLAGS, N.stream_of(src)))
        return gq, gkt.transpose(-1, -2)
    gq = band_n(grad_output, kt, window_size) if need[0] else None
    gk = band_t(grad_output, src, window_size).transpose(-1, -2) if need[1] else None
    return gq, gk


def unwindow_matmul_forward(src: torch.Tensor, other: torch.Tensor, window_size: int, out=None) -> torch.Tensor:
    """window_matmul.cpp:87-91 -> unwindow_matmul_fw_cuda (window_matmul_cuda.cu:321-358).
    src (B,M,2w+1), other (B,M,N) -> (B,M,N)."""
    _mismatch(src.dim() == 3 and other.dim() == 3)
    _mismatch(src.size(0) == other.size(0) and src.size(1) == other.size(1))
    _mismatch(src.size(2) == window_size * 2 + 1)
    return band_n(src, other, window_size, out=out)


def unwindow_matmul_backward(src, other, window_size, grad_output, need=(True, True), out=None):
    """window_matmul.cpp:93-98 -> unwindow_matmul_bw_cuda (window_matmul_cuda.cu:360-416).
    Returns (grad_src (B,M,2w+1), grad_other (B,M,N))."""
    _require_cuda(src, other, grad_output)
    _mismatch(src.dim() == 3 and other.dim() == 3 and grad_output.dim() == 3)
    _mismatch(src.size(0) == other.size(0) and src.size(1) == other.size(1))
    _mismatch(src.size(2) == window_size * 2 + 1 and grad_output.shape == other.shape)
    src = src.contiguous()
    other, grad_output = _addressable(other), _addressable(grad_output)
    B, M, Nn = other.shape
    if need[0] and need[1]:
        ga = torch.empty((B, M, 2 * window_size + 1), dtype=src.dtype, device=src.device) if out is None \
            else _check_out(out[0], (B, M, 2 * window_size + 1), src, True)
        gv = torch.empty((B, M, Nn), dtype=src.dtype, device=src.device) if out is None else _check_out(out[1], (B, M, Nn), src, False)
        g = N.geometry(B, M, Nn, window_size)
        with torch.cuda.device(src.device):
            N.check(N.lib.wmm_unwindow_bwd(src.data_ptr(), N.operand(other), N.operand(grad_output), ga.data_ptr(),
                                           N.operand(gv), g, N.dtype_code(src), _FLAGS, N.stream_of(src)))
        return ga, gv
    ga = band_nt(grad_output, other, window_size) if need[0] else None
    gv = band_t(src, grad_output, window_size) if need[1] else None
    return ga, gv


# ---- leading dimensions ---------------------------------------------------------------------------
# The reference flattens the leading dimensions with `reshape` (window_matmul/window_matmul.py:36-37, 72-73), which
# silently COPIES an operand whose leading dimensions cannot be merged, e.g. the (B, H, M, N) view of a (B, M, H*N)
# projection.  Here such operands are consumed where they are: the outermost dimensions are looped over until what
# remains of every operand is a view (batch, rows, cols) with element strides, which the kernels take directly.


def _lead(t: torch.Tensor) -> int:
    n = 1
    for d in t.shape[:-2]:
        n *= d
    return n


def _viewable3(t: torch.Tensor) -> bool:
    try:
        t.view(_lead(t), t.shape[-2], t.shape[-1])   # (an explicit size: -1 is ambiguous for empty tensors)
        return True
    except RuntimeError:
        return False


def split_depth(*tensors: torch.Tensor) -> int:
    """Smallest number of outermost dimensions to loop over so that the rest of every tensor is a 3-D view."""
    lead = tensors[0].dim() - 2
    for d in range(lead + 1):
        if all(_viewable3(t[(0,) * d] if d and t.numel() else t) for t in tensors):
            return d
    return lead


def _slices(depth: int, shape) -> list:
    import itertools

    return list(itertools.product(*[range(n) for n in shape[:depth]]))


def _v3(t: torch.Tensor, idx) -> torch.Tensor:
    s = t[idx] if idx else t
    return s.view(_lead(s), s.shape[-2], s.shape[-1])


class _StridedWindowMatmulFunc(torch.autograd.Function):
    """WindowMatmulFunc for operands whose leading dimensions do not merge: same kernels, one call per outer index."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, inp, other, window_size, depth):
        _require_cuda(inp, other)
        *dims, M, Nh = inp.shape
        out = torch.empty((*dims, M, 2 * window_size + 1), dtype=inp.dtype, device=inp.device)
        for idx in _slices(depth, inp.shape):
            window_matmul_forward(_v3(inp, idx), _v3(other, idx), window_size, out=_v3(out, idx))
        ctx.save_for_backward(inp, other)
        ctx.depth = depth
        return out

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        inp, other = ctx.saved_tensors
        window_size = grad_output.shape[-1] // 2
        grad_output = grad_output.contiguous()
        need = tuple(ctx.needs_input_grad[:2])
        gq = torch.empty(inp.shape, dtype=inp.dtype, device=inp.device) if need[0] else None
        gkt = torch.empty(inp.shape, dtype=inp.dtype, device=inp.device) if need[1] else None
        for idx in _slices(ctx.depth, inp.shape):
            if need[0] and need[1]:
                window_matmul_backward(_v3(inp, idx), _v3(other, idx), window_size, _v3(grad_output, idx),
                                       out=(_v3(gq, idx), _v3(gkt, idx)))
            elif need[0]:
                band_n(_v3(grad_output, idx), _addressable(_v3(other, idx).transpose(-1, -2)), window_size, out=_v3(gq, idx))
            elif need[1]:
                band_t(_v3(grad_output, idx), _addressable(_v3(inp, idx)), window_size, out=_v3(gkt, idx))
        return gq, (gkt.transpose(-1, -2) if need[1] else None), None, None


class _StridedUnwindowMatmulFunc(torch.autograd.Function):
    """UnwindowMatmulFunc for operands whose leading dimensions do not merge."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, inp, other, window_size, depth):
        _require_cuda(inp, other)
        out = torch.empty(other.shape, dtype=other.dtype, device=other.device)
        for idx in _slices(depth, other.shape):
            unwindow_matmul_forward(_v3(inp, idx), _v3(other, idx), window_size, out=_v3(out, idx))
        ctx.save_for_backward(inp, other)
        ctx.depth = depth
        return out

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output):
        inp, other = ctx.saved_tensors
        window_size = inp.shape[-1] // 2
        need = tuple(ctx.needs_input_grad[:2])
        ga = torch.empty(inp.shape, dtype=inp.dtype, device=inp.device) if need[0] else None
        gv = torch.empty(other.shape, dtype=other.dtype, device=other.device) if need[1] else None
        depth = max(ctx.depth, split_depth(grad_output))
        for idx in _slices(depth, other.shape):
            a3, v3, g3 = _v3(inp, idx), _v3(other, idx), _v3(grad_output, idx)
            if need[0] and need[1]:
                unwindow_matmul_backward(a3, v3, window_size, g3, out=(_v3(ga, idx), _v3(gv, idx)))
            elif need[0]:
                band_nt(_addressable(g3), _addressable(v3), window_size, out=_v3(ga, idx))
            elif need[1]:
                band_t(a3.contiguous(), _addressable(g3), window_size, out=_v3(gv, idx))
        return ga, gv, None, None


# ---- autograd nodes and the public functions ------------------------------------------------------


class WindowMatmulFunc(torch.autograd.Function):
    """window_matmul/window_matmul.py:7-27."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, inp: torch.Tensor, other: torch.Tensor, window_size: int) -> torch.Tensor:
        _require_cuda(inp, other)
        output = window_matmul_forward(inp, other, window_size)
        ctx.save_for_backward(inp, other)
        return output

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output: torch.Tensor) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], None]:
        window_size = (grad_output.shape[-1]) // 2
        inp, other = ctx.saved_tensors
        inp_grad, other_grad = window_matmul_backward(
            inp, other, window_size, grad_output, need=tuple(ctx.needs_input_grad[:2])
        )
        return inp_grad, other_grad, None


def window_matmul(inp: torch.Tensor, other: torch.Tensor, window_size: int) -> torch.Tensor:
    """Banded Q.K^T.  window_matmul/window_matmul.py:30-40."""
    if not window_size:
        return (inp * other.transpose(-1, -2)).sum(dim=-1, keepdim=True)
    *dims, seq_len, hidden_dim = inp.shape
    if inp.is_cuda and other.is_cuda and other.shape == (*dims, hidden_dim, seq_len):
        depth = split_depth(inp, other)
        if depth:   # leading dimensions that do not merge: no copy, one call per outer index
            return _StridedWindowMatmulFunc.apply(inp, other, window_size, depth)
    inp = inp.reshape(_lead(inp), seq_len, hidden_dim)        # (-1 would be ambiguous for an empty sequence)
    other = other.reshape(_lead(other), hidden_dim, seq_len)
    out = WindowMatmulFunc.apply(inp, other, window_size)
    out = out.reshape(*dims, seq_len, window_size * 2 + 1)
    return out


class UnwindowMatmulFunc(torch.autograd.Function):
    """window_matmul/window_matmul.py:43-63."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, inp: torch.Tensor, other: torch.Tensor, window_size: int) -> torch.Tensor:
        _require_cuda(inp, other)
        output = unwindow_matmul_forward(inp, other, window_size)
        ctx.save_for_backward(inp, other)
        return output

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, grad_output: torch.Tensor) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], None]:
        inp, other = ctx.saved_tensors
        window_size = (inp.shape[-1]) // 2
        inp_grad, other_grad = unwindow_matmul_backward(
            inp, other, window_size, grad_output, need=tuple(ctx.needs_input_grad[:2])
        )
        return inp_grad, other_grad, None


def unwindow_matmul(inp: torch.Tensor, other: torch.Tensor, window_size: int) -> torch.Tensor:
    """Band times V.  window_matmul/window_matmul.py:66-76."""
    if not window_size:
        return inp * other
    *dims, seq_len, hidden_dim = other.shape
    if inp.is_cuda and other.is_cuda and inp.shape == (*dims, seq_len, window_size * 2 + 1):
        depth = split_depth(inp, other)
        if depth:
            return _StridedUnwindowMatmulFunc.apply(inp, other, window_size, depth)
    inp = inp.reshape(_lead(inp), seq_len, window_size * 2 + 1)
    other = other.reshape(_lead(other), seq_len, hidden_dim)
    out = UnwindowMatmulFunc.apply(inp, other, window_size)
    out = out.reshape(*dims, seq_len, hidden_dim)
    return out
