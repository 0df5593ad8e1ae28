"""Leading dimensions of the operators: operands whose leading dimensions cannot be merged (head-split views) are
consumed without the copy the reference's `reshape` makes (window_matmul/window_matmul.py:36-37, 72-73)."""
import importlib
import math

import pytest
import torch


def _impl():
    return importlib.import_module("window_matmul.window_matmul")


def test_split_depth_finds_the_fewest_outer_dimensions_to_loop_over():
    wm = _impl()
    B, H, M, N = 2, 3, 8, 4
    proj = torch.randn(B, M, H * N)
    heads = proj.view(B, M, H, N).transpose(1, 2)              # (B, H, M, N): B and H do not merge
    assert not heads.is_contiguous()
    assert wm.split_depth(heads) == 1
    assert wm.split_depth(torch.randn(B, H, M, N)) == 0        # contiguous: one call
    assert wm.split_depth(torch.randn(M, N)) == 0
    assert wm.split_depth(torch.randn(B, H, M, N), heads) == 1  # the worst operand decides
    assert wm.split_depth(heads, heads.transpose(-1, -2)) == 1  # a transposed K view changes nothing
    per_b = wm._v3(heads, (1,))
    assert per_b.shape == (H, M, N) and per_b.stride() == (N, H * N, 1) and per_b.data_ptr() == heads[1].data_ptr()
    deep = torch.randn(2, 3, 5, M, N).permute(2, 0, 1, 3, 4)   # (5, 2, 3, M, N): dim 0 is the odd one out
    assert wm.split_depth(deep) == 1
    assert wm._slices(1, deep.shape) == [(i,) for i in range(5)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_head_split_views_give_the_results_of_contiguous_operands(dtype):
    """(B, H, M, N) views of (B, M, H*N) projections through both operators and the band softmax, forward and
    backward: identical to the same call on contiguous copies, with one kernel call per batch entry and no copy."""
    from window_matmul import _native as N_
    from window_matmul import unwindow_matmul, window_matmul, window_softmax

    B, H, M, Nn, w = 3, 2, 256, 64, 64
    g = torch.Generator().manual_seed(3)
    pq, pk, pv = (torch.randn(B, M, H * Nn, generator=g).to(dtype).cuda() for _ in range(3))
    go = torch.randn(B, H, M, Nn, generator=g).to(dtype).cuda()

    def run(strided):
        leaves = [t.clone().requires_grad_(True) for t in (pq, pk, pv)]
        q, k, v = (t.view(B, M, H, Nn).transpose(1, 2) for t in leaves)
        if not strided:
            q, k, v = (t.contiguous() for t in (q, k, v))
        before = N_.launch_count()
        a = window_matmul(q, k.transpose(-1, -2), w)
        launches = N_.launch_count() - before
        o = unwindow_matmul(window_softmax(a, 1.0 / math.sqrt(Nn)), v, w)
        o.backward(go)
        return [a.detach(), o.detach()] + [t.grad for t in leaves], launches

    got, n_strided = run(True)
    want, n_contig = run(False)
    assert n_contig == 1 and n_strided == B
    for name, x, y in zip(("a", "o", "grad_q_proj", "grad_k_proj", "grad_v_proj"), got, want):
        assert torch.equal(x, y), name
