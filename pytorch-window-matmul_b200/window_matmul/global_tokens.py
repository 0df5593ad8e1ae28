"""Windowed attention with global tokens (the Longformer / BigBird pattern) on top of the two operators.

A few positions G are global: every query attends to them besides its own window, and the queries AT those positions
attend to the whole sequence.  The windowed part is the two banded contractions of this package; the global part is
dense but thin ((M x |G|) and (|G| x M) blocks) and goes through plain matrix products:

    scores   = [ window_matmul(q, k^T, w) | q . k[G]^T ]                     (*, M, 2w+1 + |G|)
    probs    = softmax over both parts together (out-of-sequence band slots and global columns that already lie in the
               row's window masked out, so that no key is counted twice)
    out      = unwindow_matmul(probs_band, v, w) + probs_glob . v[G]
    out[G]   = softmax(q[G] . k^T) . v                                       (the global queries see every position)

Everything is differentiable through autograd (the banded parts through this package's backward kernels).  The reference
has no such variant; its README names the models that use the pattern as its motivation (README.md:5).
"""
import math
from typing import Optional

import torch

from .window_matmul import unwindow_matmul, window_matmul


def global_window_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window_size: int, global_idx: torch.Tensor,
                            scale: Optional[float] = None) -> torch.Tensor:
    """q, k, v (*, M, N); global_idx: 1-D integer tensor of distinct positions.  Returns (*, M, N)."""
    *_, M, Nh = q.shape
    w = window_size
    if global_idx.dim() != 1 or global_idx.numel() == 0:
        raise RuntimeError("Input mismatch: global_idx must be a non-empty 1-D tensor of positions")
    gidx = global_idx.to(device=q.device, dtype=torch.long)
    scale = 1.0 / math.sqrt(Nh) if scale is None else scale
    kg, vg = k.index_select(-2, gidx), v.index_select(-2, gidx)                      # (*, G, N)
    band = window_matmul(q, k.transpose(-1, -2), w)                                   # (*, M, 2w+1)
    glob = q @ kg.transpose(-1, -2)                                                   # (*, M, G)
    i = torch.arange(M, device=q.device)
    pos = i[:, None] + torch.arange(2 * w + 1, device=q.device)[None, :] - w
    outside = (pos < 0) | (pos >= M)                                                  # band slots beyond the sequence
    in_window = (gidx[None, :] - i[:, None]).abs() <= w                               # global keys the band already holds
    scores = torch.cat([band.float().masked_fill(outside, float("-inf")), glob.float().masked_fill(in_window, float("-inf"))], -1)
    probs = torch.softmax(scores * scale, dim=-1).to(q.dtype)
    p_band, p_glob = probs[..., : 2 * w + 1], probs[..., 2 * w + 1:]
    out = unwindow_matmul(p_band.contiguous(), v, w) + p_glob @ vg
    # the global queries: dense rows over the whole sequence
    qg = q.index_select(-2, gidx)
    dense = torch.softmax((qg @ k.transpose(-1, -2)).float() * scale, dim=-1).to(q.dtype) @ v   # (*, G, N)
    return out.index_copy(-2, gidx, dense)
