"""Sequence- and batch-sharded operators on CPU ranks (gloo, world_size 2 and 3).

The neighbour exchange (forward halo, reverse halo of partial gradients), the sequence-end clipping and the
autograd wiring of window_matmul/sharded.py are host logic; they run here with the three primitives replaced
by a float64 checker, and the assembled result is compared with the oracle on the unsharded problem."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _CheckerPrimitives:
    """The generalised primitives of include/wmm_b200.h in plain torch float64 (checker only)."""

    @staticmethod
    def band_nt(x, y, window, *, other_off=0, seq=None, out=None, flags=None):
        B, M, _ = x.shape
        lo, hi = (0, y.shape[1]) if seq is None else seq
        band = x.new_zeros((B, M, 2 * window + 1))
        i = torch.arange(M)
        for j in range(2 * window + 1):
            p = i + j - window + other_off
            ok = (p >= lo) & (p < hi)
            band[:, i[ok], j] = (x[:, i[ok]] * y[:, p[ok]]).sum(-1)
        return band

    @staticmethod
    def band_n(band, y, window, *, rows_out=None, other_off=0, seq=None, out=None, flags=None):
        B, M, _ = band.shape
        lo, hi = (0, y.shape[1]) if seq is None else seq
        o = y.new_zeros((B, M, y.shape[2]))
        i = torch.arange(M)
        for j in range(2 * window + 1):
            p = i + j - window + other_off
            ok = (p >= lo) & (p < hi)
            o[:, i[ok]] += band[:, i[ok], j].unsqueeze(-1) * y[:, p[ok]]
        return o

    @staticmethod
    def band_t(band, x, window, *, other_rows=None, other_off=0, seq=None, out=None, flags=None):
        B, M, _ = band.shape
        Mo = M if other_rows is None else other_rows
        lo, hi = (0, Mo) if seq is None else seq
        o = x.new_zeros((B, Mo, x.shape[2]))
        i = torch.arange(M)
        for j in range(2 * window + 1):
            p = i + j - window + other_off
            ok = (p >= lo) & (p < hi)
            o.index_add_(1, p[ok], band[:, i[ok], j].unsqueeze(-1) * x[:, i[ok]])
        return o


    @staticmethod
    def band_softmax(scores, scale=1.0, mask=True, *, other_off=0, seq=None, other_rows=None, out=None):
        B, M, W = scores.shape
        w = (W - 1) // 2
        lo, hi = (0, M if other_rows is None else other_rows) if seq is None else seq
        p = torch.arange(M)[:, None] + torch.arange(W)[None, :] - w + other_off
        s = scores * scale
        if mask:
            s = s.masked_fill(~((p >= lo) & (p < hi)), float("-inf"))
        return torch.softmax(s, dim=-1)

    @staticmethod
    def band_softmax_backward(probs, grad_probs, scale=1.0, mask=True, *, other_off=0, seq=None, other_rows=None, out=None):
        return scale * probs * (grad_probs - (grad_probs * probs).sum(-1, keepdim=True))


def _worker(rank, world, port, shape, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import sys

        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        sys.path[:0] = [root, os.path.join(root, "pytorch-window-matmul_b200")]
        from window_matmul import sharded

        sharded.primitives = _CheckerPrimitives()
        B, M, N, w = shape
        g = torch.Generator().manual_seed(5)
        q, k, v = (torch.randn(B, M, N, generator=g, dtype=torch.float64) for _ in range(3))
        go = torch.randn(B, M, N, generator=g, dtype=torch.float64)
        Ml = M // world
        sl = slice(rank * Ml, (rank + 1) * Ml)
        ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
        a = sharded.seq_parallel_window_matmul(ql, kl.transpose(-1, -2), w)
        a.retain_grad()
        o = sharded.seq_parallel_unwindow_matmul(a, vl, w)
        o.backward(go[:, sl])
        # the attention block: scores -> masked softmax -> values, all three sharded operators
        q2, k2, v2 = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
        pr = sharded.seq_parallel_window_softmax(sharded.seq_parallel_window_matmul(q2, k2.transpose(-1, -2), w), 0.5, True)
        ob = sharded.seq_parallel_unwindow_matmul(pr, v2, w)
        ob.backward(go[:, sl])
        np.savez(os.path.join(out_dir, "rank%d.npz" % rank), a=a.detach().numpy(), o=o.detach().numpy(), gq=ql.grad.numpy(),
                 gk=kl.grad.numpy(), gv=vl.grad.numpy(), ga=a.grad.numpy(), ob=ob.detach().numpy(), bq=q2.grad.numpy(),
                 bk=k2.grad.numpy(), bv=v2.grad.numpy())
        # batch sharding: contiguous blocks, no communication
        blk = sharded.shard_batch(torch.arange(7))
        per = -(-7 // world)
        assert blk.tolist() == list(range(rank * per, min(7, (rank + 1) * per)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,shape", [(2, (2, 24, 5, 4)), (3, (1, 36, 4, 12)), (2, (1, 16, 3, 8))])
def test_sequence_sharded_operators_match_the_unsharded_oracle(tmp_path, world, shape):
    from oracle import oracle

    mp.spawn(_worker, args=(world, _free_port(), shape, str(tmp_path)), nprocs=world, join=True)
    B, M, N, w = shape
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(B, M, N, generator=g, dtype=torch.float64).numpy() for _ in range(3))
    go = torch.randn(B, M, N, generator=g, dtype=torch.float64).numpy()
    a, o, gq, gk, ga, gv = oracle.chain_fwd_bwd(q, np.ascontiguousarray(k.transpose(0, 2, 1)), v, w, go)
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    cat = lambda key: np.concatenate([p[key] for p in parts], axis=1)  # noqa: E731
    np.testing.assert_allclose(cat("a"), a, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(cat("o"), o, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(cat("ga"), ga, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(cat("gq"), gq, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(cat("gk"), gk.transpose(0, 2, 1), rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(cat("gv"), gv, rtol=1e-12, atol=1e-12)
    # attention block against the dense formulation on the whole sequence
    qt, kt_, vt = (torch.from_numpy(x).requires_grad_(True) for x in (q, k, v))
    i = torch.arange(M)
    inside = (i[:, None] - i[None, :]).abs() <= w
    dense = torch.softmax((qt @ kt_.transpose(-1, -2) * 0.5).masked_fill(~inside, float("-inf")), -1) @ vt
    dense.backward(torch.from_numpy(go))
    np.testing.assert_allclose(cat("ob"), dense.detach().numpy(), rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(cat("bq"), qt.grad.numpy(), rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(cat("bk"), kt_.grad.numpy(), rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(cat("bv"), vt.grad.numpy(), rtol=1e-10, atol=1e-12)


def test_shard_shorter_than_the_window_is_refused():
    from window_matmul import sharded

    with pytest.raises(RuntimeError, match="shorter than the window"):
        sharded.exchange_halo(torch.zeros(1, 4, 2), 8)
