"""Masked, scaled softmax over the band, between `window_matmul` and `unwindow_matmul`.

The reference has no such operator: a caller composes it from torch ops (tests/test_attention.py:60-61,
`att_scores / math.sqrt(N)` then `softmax(att_scores, dim=-1)`) and is left to mask the out-of-sequence slots of
the band itself.  Those torch ops read and write the whole band several times in each direction; this operator
does the scale, the mask and the softmax in one pass over HBM forward and one pass backward.

  window_softmax(scores (*,M,2w+1), scale=1.0, mask=True) -> probabilities (*,M,2w+1)

mask=True: slot j of row i takes part only if position i+j-w lies inside the sequence; other slots get probability
exactly 0 (what adding -inf there before a softmax gives).  mask=False: every slot takes part with the score stored
there, which reproduces a plain `torch.softmax(scores * scale, -1)` over the band.
"""
from typing import Optional, Tuple

import torch

from . import _native as N


def _check(t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise RuntimeError("window_softmax: tensor must be CUDA tensor (this package has no CPU path)")
    if t.dim() < 2 or t.shape[-1] % 2 == 0:
        raise RuntimeError("Input mismatch")


def _check_out(out: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    """A caller-supplied output is written as a contiguous, 16-byte aligned band of `like`'s shape and dtype."""
    if not (isinstance(out, torch.Tensor) and out.shape == like.shape and out.dtype == like.dtype
            and out.device == like.device and out.is_contiguous() and out.data_ptr() % 16 == 0):
        raise RuntimeError("Input mismatch")
    return out


def band_softmax(scores, scale=1.0, mask=True, *, other_off=0, seq=None, other_rows=None, out=None):
    """Forward on a (B,M,2w+1) tensor.  `other_off`, `seq`, `other_rows` as in the three primitives: slot j of row i
    is in sequence iff seq[0] <= i + j - w + other_off < seq[1] (a sequence shard passes its halo geometry)."""
    _check(scores)
    scores = scores.contiguous()
    B, M, W = scores.shape
    w = (W - 1) // 2
    probs = torch.empty_like(scores) if out is None else _check_out(out, scores)
    g = N.geometry(B, M, 0, w, M if other_rows is None else other_rows, other_off, seq)
    with torch.cuda.device(scores.device):
        N.check(N.lib.wmm_band_softmax(scores.data_ptr(), probs.data_ptr(), g, N.dtype_code(scores), float(scale),
                                       0 if mask else N.FLAG_SOFTMAX_KEEP_PADDING, N.stream_of(scores)))
    return probs


def band_softmax_backward(probs, grad_probs, scale=1.0, mask=True, *, other_off=0, seq=None, other_rows=None,
                          out=None):
    """grad_scores = scale * probs * (grad_probs - sum_j grad_probs * probs) on (B,M,2w+1) tensors."""
    _check(probs)
    if grad_probs.shape != probs.shape or grad_probs.dtype != probs.dtype or grad_probs.device != probs.device:
        raise RuntimeError("Input mismatch")
    probs, grad_probs = probs.contiguous(), grad_probs.contiguous()
    B, M, W = probs.shape
    w = (W - 1) // 2
    grad_scores = torch.empty_like(probs) if out is None else _check_out(out, probs)
    g = N.geometry(B, M, 0, w, M if other_rows is None else other_rows, other_off, seq)
    with torch.cuda.device(probs.device):
        N.check(N.lib.wmm_band_softmax_bwd(probs.data_ptr(), grad_probs.data_ptr(), grad_scores.data_ptr(), g,
                                           N.dtype_code(probs), float(scale),
                                           0 if mask else N.FLAG_SOFTMAX_KEEP_PADDING, N.stream_of(probs)))
    return grad_scores


class WindowSoftmaxFunc(torch.autograd.Function):
    """Saves only the probabilities (the scores are not needed for the backward)."""

    @staticmethod
    def forward(ctx, scores: torch.Tensor, scale: float, mask: bool) -> torch.Tensor:
        probs = band_softmax(scores, scale, mask)
        ctx.save_for_backward(probs)
        ctx.scale, ctx.mask = scale, mask
        return probs

    @staticmethod
    def backward(ctx, grad_probs: torch.Tensor) -> Tuple[Optional[torch.Tensor], None, None]:
        (probs,) = ctx.saved_tensors
        return band_softmax_backward(probs, grad_probs, ctx.scale, ctx.mask), None, None


def window_softmax(scores: torch.Tensor, scale: float = 1.0, mask: bool = True) -> torch.Tensor:
    """softmax over the last dimension of a band tensor (*, M, 2w+1) of `window_matmul` scores, times `scale` first;
    differentiable in `scores`.  See the module docstring for `mask`."""
    _check(scores)
    if scores.numel() == 0:
        return scores.clone()
    lead = scores.shape[:-2]
    flat = scores.reshape(-1, scores.shape[-2], scores.shape[-1])
    return WindowSoftmaxFunc.apply(flat, float(scale), bool(mask)).reshape(*lead, *scores.shape[-2:])
