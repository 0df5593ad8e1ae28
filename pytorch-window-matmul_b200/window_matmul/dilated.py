"""Dilated windows on top of the two operators, by views only.

With dilation d a query at position i attends to the positions i + (j - w) * d, j = 0 .. 2w: positions of one residue
class modulo d only ever meet each other.  Splitting the sequence into its d residue classes therefore turns one dilated
problem of length M into d ordinary windowed problems of length M / d, and the split is a VIEW: (*, M, N) ->
(*, d, M/d, N) with strides (N, d*N, 1) inside each batch entry, which the kernels address directly (no copy; see the
leading-dimension handling in window_matmul.py).  The band comes out residue-major, (*, d, M/d, 2w+1): entry
[r, t, j] belongs to query position t*d + r and key position (t + j - w)*d + r.  `window_softmax` and
`dilated_unwindow_matmul` take it in that layout.

The reference has no dilated variant (its README names the sparse-attention models that use one as motivation only).
"""
import torch

from .window_matmul import unwindow_matmul, window_matmul


def _check(seq_len: int, dilation: int) -> None:
    if dilation < 1 or seq_len % dilation != 0:
        raise RuntimeError("Input mismatch: sequence length %d is not a multiple of the dilation %d" % (seq_len, dilation))


def dilate_rows(x: torch.Tensor, dilation: int) -> torch.Tensor:
    """(*, M, N) -> (*, d, M/d, N): residue classes of the sequence positions, as a view."""
    _check(x.shape[-2], dilation)
    return x.unflatten(-2, (x.shape[-2] // dilation, dilation)).transpose(-3, -2)


def undilate_rows(y: torch.Tensor) -> torch.Tensor:
    """(*, d, M/d, N) -> (*, M, N): positions back in sequence order (copies if `y` is not already laid out that way)."""
    return y.transpose(-3, -2).flatten(-3, -2)


def dilated_window_matmul(inp: torch.Tensor, other: torch.Tensor, window_size: int, dilation: int) -> torch.Tensor:
    """inp (*, M, N), other (*, N, M) -> residue-major band (*, d, M/d, 2w+1); out-of-sequence slots are 0."""
    _check(inp.shape[-2], dilation)
    k = other.unflatten(-1, (other.shape[-1] // dilation, dilation)).movedim(-1, -3)   # (*, d, N, M/d), a view
    return window_matmul(dilate_rows(inp, dilation), k, window_size)


def dilated_unwindow_matmul(band: torch.Tensor, other: torch.Tensor, window_size: int, dilation: int) -> torch.Tensor:
    """band (*, d, M/d, 2w+1) residue-major, other (*, M, N) -> (*, M, N)."""
    _check(other.shape[-2], dilation)
    return undilate_rows(unwindow_matmul(band, dilate_rows(other, dilation), window_size))
