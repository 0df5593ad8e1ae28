"""Multi-GPU forms of the two operators: one process per GPU, `torch.distributed` for the plumbing.

Batch sharding needs nothing from this module: every (batch x head) entry is independent in all six
contractions, so each rank calls `window_matmul` / `unwindow_matmul` on its own slice and no data moves.

Sequence sharding (long M): rank r owns rows [r*Ml, (r+1)*Ml) of Q, K, V, A and O.  A band row reaches w
positions to either side, so
  * forward: each rank receives the last w rows of K^T (resp. V) from rank r-1 and the first w rows from
    rank r+1 (zeros at the ends of the global sequence) and runs the primitives on local rows + halo
    (`other_rows = Ml + 2w`, `other_off = w`, and `seq_lo/seq_hi` clipping at the global ends);
  * backward: grad_Q and grad_A reuse those halos; grad_K / grad_V rows within w of a shard edge also
    receive contributions from the neighbour's band rows.  Each rank computes partial rows for its halo
    positions from its own band rows (`band_t` with `other_rows = Ml + 2w`) and SENDS them to the neighbour,
    which adds them (reverse halo).  Band rows never cross ranks.
Only neighbours talk (isend/irecv pairs); there is no collective on the data path and no device-side wait
on a peer.  Requires Ml >= w.

The reference has no multi-GPU code; the single-GPU semantics are those of
window_matmul/window_matmul.py:30-40 and :66-76, and `tests/test_sharded.py` checks that the sharded
operators reproduce them (forward and gradients) on world_size 2 and 3.
"""
import importlib
from typing import Optional, Tuple

import torch
import torch.distributed as dist

# the submodule, not the function of the same name that the package exports
_ops = importlib.import_module(__package__ + ".window_matmul")
_sm = importlib.import_module(__package__ + ".softmax")


class _Primitives:
    """The three primitives the sharded operators are built on.  Tests on CPU ranks replace this object
    with a checker implementation; the product always uses the CUDA kernels."""

    band_nt = staticmethod(_ops.band_nt)
    band_n = staticmethod(_ops.band_n)
    band_t = staticmethod(_ops.band_t)
    band_softmax = staticmethod(_sm.band_softmax)
    band_softmax_backward = staticmethod(_sm.band_softmax_backward)


primitives = _Primitives()


def _neighbours(group) -> Tuple[int, int, Optional[int], Optional[int]]:
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    lo = dist.get_global_rank(group, rank - 1) if (group is not None and rank > 0) else (rank - 1 if rank > 0 else None)
    hi = dist.get_global_rank(group, rank + 1) if (group is not None and rank < world - 1) else (rank + 1 if rank < world - 1 else None)
    return rank, world, lo, hi


def alloc_with_halo(batch: int, rows: int, cols: int, window: int, dtype, device):
    """Storage for a sequence shard WITH room for its halos: returns (local, extended) where `extended` is a
    (batch, rows + 2w, cols) buffer and `local` = extended[:, w:w+rows] is the view to keep the shard's rows in.
    exchange_halo() on such a view fills the margins in place instead of copying the shard into a new buffer
    (the view itself remembers the buffer it was cut from: nothing is registered anywhere)."""
    ext = torch.zeros((batch, rows + 2 * window, cols), dtype=dtype, device=device)
    local = ext[:, window:window + rows]
    return local, ext


def _extended(x: torch.Tensor, window: int) -> torch.Tensor:
    """The (B, Ml + 2w, N) buffer whose middle rows are x: the tensor x is a view of if x was cut from such a buffer
    the way alloc_with_halo() does, else a new zeroed buffer with x copied in."""
    B, Ml, N = x.shape
    held = x._base
    if held is not None and held.dim() == 3 and held.shape == (B, Ml + 2 * window, N) and held.dtype == x.dtype \
            and held.is_contiguous():
        mid = held[:, window:window + Ml]
        if mid.data_ptr() == x.data_ptr() and mid.stride() == x.stride():
            return held
    ext = x.new_zeros((B, Ml + 2 * window, N))
    ext[:, window:window + Ml] = x
    return ext


def _swap_strips(to_lo, to_hi, group):
    """One neighbour exchange: sends `to_lo` to the lower and `to_hi` to the upper neighbour (contiguous
    tensors, or None at a sequence end) and returns what they sent (same shapes), or None."""
    _, _, lo, hi = _neighbours(group)
    ops, from_lo, from_hi = [], None, None
    if lo is not None:
        from_lo = torch.empty_like(to_lo)
        ops += [dist.P2POp(dist.isend, to_lo, lo, group), dist.P2POp(dist.irecv, from_lo, lo, group)]
    if hi is not None:
        from_hi = torch.empty_like(to_hi)
        ops += [dist.P2POp(dist.isend, to_hi, hi, group), dist.P2POp(dist.irecv, from_hi, hi, group)]
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return from_lo, from_hi


def exchange_halo_many(xs, window: int, group=None):
    """exchange_halo() for several tensors of the same shape and dtype in ONE neighbour exchange (their
    boundary rows travel in one message per direction).  Returns the extended tensors."""
    B, Ml, N = xs[0].shape
    if Ml < window:
        raise RuntimeError("sequence shard of %d rows is shorter than the window %d" % (Ml, window))
    _, _, lo, hi = _neighbours(group)
    exts = [_extended(x, window) for x in xs]
    to_lo = torch.stack([x[:, :window] for x in xs]) if lo is not None else None
    to_hi = torch.stack([x[:, Ml - window:] for x in xs]) if hi is not None else None
    from_lo, from_hi = _swap_strips(to_lo, to_hi, group)
    for i, ext in enumerate(exts):
        if from_lo is not None:
            ext[:, :window] = from_lo[i]
        if from_hi is not None:
            ext[:, window + Ml:] = from_hi[i]
    return exts


def exchange_halo(x: torch.Tensor, window: int, group=None) -> torch.Tensor:
    """x (B, Ml, N) local rows -> (B, Ml + 2w, N): [w rows of the lower neighbour | x | w rows of the upper
    neighbour]; zeros where the global sequence ends.  If x lives in storage from alloc_with_halo() only the
    margins are written; otherwise x is copied into a new extended buffer."""
    return exchange_halo_many([x], window, group)[0]


def reduce_halo_many(parts, window: int, group=None):
    """reduce_halo() for several tensors of the same shape and dtype in ONE neighbour exchange."""
    B, Mext, N = parts[0].shape
    Ml = Mext - 2 * window
    _, _, lo, hi = _neighbours(group)
    to_lo = torch.stack([p_[:, :window] for p_ in parts]) if lo is not None else None
    to_hi = torch.stack([p_[:, window + Ml:] for p_ in parts]) if hi is not None else None
    from_lo, from_hi = _swap_strips(to_lo, to_hi, group)
    owns = []
    for i, p_ in enumerate(parts):
        own = p_[:, window:window + Ml]
        if from_lo is not None:
            own[:, :window] += from_lo[i]
        if from_hi is not None:
            own[:, Ml - window:] += from_hi[i]
        owns.append(own)
    return owns


def reduce_halo(part: torch.Tensor, window: int, group=None) -> torch.Tensor:
    """part (B, Ml + 2w, N): this rank's contributions to positions [m0 - w, m0 + Ml + w).  Sends the two
    halo strips to the neighbours that own those positions and adds what they send, in place: returns the
    (B, Ml, N) view part[:, w:w+Ml]."""
    return reduce_halo_many([part], window, group)[0]


def _local_seq(Ml: int, window: int, group) -> Tuple[int, int]:
    """In-sequence range of the extended row space [m0 - w, m0 + Ml + w) of this rank."""
    rank, world, _, _ = _neighbours(group)
    return (window if rank == 0 else 0, Ml + window if rank == world - 1 else Ml + 2 * window)


class _SeqWindowMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, kt, window, group):
        kt_ext = exchange_halo(kt, window, group)
        seq = _local_seq(q.shape[1], window, group)
        a = primitives.band_nt(q, kt_ext, window, other_off=window, seq=seq)
        ctx.save_for_backward(q, kt_ext)
        ctx.window, ctx.group, ctx.seq = window, group, seq
        return a

    @staticmethod
    def backward(ctx, grad_a):
        q, kt_ext = ctx.saved_tensors
        w, seq = ctx.window, ctx.seq
        grad_a = grad_a.contiguous()
        gq = primitives.band_n(grad_a, kt_ext, w, other_off=w, seq=seq)
        part = primitives.band_t(grad_a, q, w, other_rows=kt_ext.shape[1], other_off=w, seq=seq)
        gkt = reduce_halo(part, w, ctx.group)
        return gq, gkt, None, None


class _SeqUnwindowMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, v, window, group):
        v_ext = exchange_halo(v, window, group)
        seq = _local_seq(v.shape[1], window, group)
        a = a.contiguous()
        o = primitives.band_n(a, v_ext, window, other_off=window, seq=seq)
        ctx.save_for_backward(a, v_ext)
        ctx.window, ctx.group, ctx.seq = window, group, seq
        return o

    @staticmethod
    def backward(ctx, grad_o):
        a, v_ext = ctx.saved_tensors
        w, seq = ctx.window, ctx.seq
        grad_o = grad_o.contiguous()
        ga = primitives.band_nt(grad_o, v_ext, w, other_off=w, seq=seq)
        part = primitives.band_t(a, grad_o, w, other_rows=v_ext.shape[1], other_off=w, seq=seq)
        gv = reduce_halo(part, w, ctx.group)
        return ga, gv, None, None


def seq_parallel_window_matmul(inp: torch.Tensor, other: torch.Tensor, window_size: int, group=None) -> torch.Tensor:
    """`window_matmul` on a sequence shard.  inp (*, Ml, N), other (*, N, Ml): this rank's rows of Q and
    columns of K.  Returns this rank's rows of the band, (*, Ml, 2w+1)."""
    if not window_size:
        return (inp * other.transpose(-1, -2)).sum(dim=-1, keepdim=True)
    *dims, seq_len, hidden = inp.shape
    q = inp.reshape(-1, seq_len, hidden)
    kt = other.reshape(-1, hidden, seq_len).transpose(-1, -2)
    out = _SeqWindowMatmul.apply(q, kt, window_size, group)
    return out.reshape(*dims, seq_len, 2 * window_size + 1)


def seq_parallel_unwindow_matmul(inp: torch.Tensor, other: torch.Tensor, window_size: int, group=None) -> torch.Tensor:
    """`unwindow_matmul` on a sequence shard.  inp (*, Ml, 2w+1), other (*, Ml, N) -> (*, Ml, N)."""
    if not window_size:
        return inp * other
    *dims, seq_len, hidden = other.shape
    a = inp.reshape(-1, seq_len, 2 * window_size + 1)
    v = other.reshape(-1, seq_len, hidden)
    out = _SeqUnwindowMatmul.apply(a, v, window_size, group)
    return out.reshape(*dims, seq_len, hidden)


class _SeqWindowSoftmax(torch.autograd.Function):
    """Band rows never cross ranks, so the softmax of a sequence shard needs no communication: only the shard's place
    in the global sequence, for the out-of-sequence slots of the first and last rank."""

    @staticmethod
    def forward(ctx, scores, scale, mask, group):
        Ml, w = scores.shape[1], (scores.shape[2] - 1) // 2
        seq = _local_seq(Ml, w, group)
        probs = primitives.band_softmax(scores, scale, mask, other_off=w, seq=seq, other_rows=Ml + 2 * w)
        ctx.save_for_backward(probs)
        ctx.args = (scale, mask, w, seq, Ml)
        return probs

    @staticmethod
    def backward(ctx, grad_probs):
        (probs,) = ctx.saved_tensors
        scale, mask, w, seq, Ml = ctx.args
        gs = primitives.band_softmax_backward(probs, grad_probs.contiguous(), scale, mask, other_off=w, seq=seq,
                                              other_rows=Ml + 2 * w)
        return gs, None, None, None


def seq_parallel_window_softmax(scores: torch.Tensor, scale: float = 1.0, mask: bool = True, group=None) -> torch.Tensor:
    """`window_softmax` on a sequence shard: scores (*, Ml, 2w+1) = this rank's band rows."""
    lead = scores.shape[:-2]
    flat = scores.reshape(-1, scores.shape[-2], scores.shape[-1])
    return _SeqWindowSoftmax.apply(flat, float(scale), bool(mask), group).reshape(*lead, *scores.shape[-2:])


def shard_batch(t: torch.Tensor, group=None) -> torch.Tensor:
    """This rank's slice of the flattened batch dimension (dim 0), in contiguous blocks of ceil(B / P)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    per = (t.shape[0] + world - 1) // world
    return t[rank * per:(rank + 1) * per]
