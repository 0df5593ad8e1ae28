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


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,dilation", [(torch.float32, 2), (torch.bfloat16, 4)])
def test_dilated_windows_by_views(dtype, dilation):
    """Dilated windowed attention (scores, masked softmax, values; forward and backward) from the residue-class views
    against the dense formulation with the dilated band mask, in float64."""
    from window_matmul import window_softmax
    from window_matmul.dilated import dilated_unwindow_matmul, dilated_window_matmul

    B, M, Nn, w, d = 2, 512, 64, 16, dilation
    g = torch.Generator().manual_seed(7)
    q, k, v, go = (torch.randn(B, M, Nn, generator=g).to(dtype) for _ in range(4))
    scale = 1.0 / math.sqrt(Nn)

    qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
    i = torch.arange(M)
    diff = i[None, :] - i[:, None]
    allowed = (diff % d == 0) & (diff.abs() <= w * d)
    dense = torch.softmax((qd @ kd.transpose(-1, -2) * scale).masked_fill(~allowed, float("-inf")), -1) @ vd
    dense.backward(go.double())

    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    band = dilated_window_matmul(qc, kc.transpose(-1, -2), w, d)
    assert band.shape == (B, d, M // d, 2 * w + 1)
    # entry [r, t, j] = q[t d + r] . k[(t + j - w) d + r]
    r, t, j = 1, 5, w + 3
    want = (q[0, t * d + r].double() * k[0, (t + j - w) * d + r].double()).sum()
    assert abs(float(band.detach()[0, r, t, j]) - float(want)) <= 2e-2 * (abs(float(want)) + 1)
    out = dilated_unwindow_matmul(window_softmax(band, scale, True), vc, w, d)
    out.backward(go.cuda())
    torch.cuda.synchronize()
    rel = 1e-4 if dtype == torch.float32 else 4e-2
    import helpers as H

    for name, got, ref in (("o", out, dense), ("gq", qc.grad, qd.grad), ("gk", kc.grad, kd.grad), ("gv", vc.grad, vd.grad)):
        H.assert_lowp_close(got, ref.detach().numpy(), name, rel=rel)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_global_tokens_on_top_of_the_window(dtype):
    """Windowed attention with a few global positions (every query sees them, they see everything) against the dense
    formulation with the same mask in float64, forward and backward."""
    from window_matmul.global_tokens import global_window_attention

    B, M, Nn, w = 2, 384, 64, 16
    g = torch.Generator().manual_seed(11)
    q, k, v, go = (torch.randn(B, M, Nn, generator=g).to(dtype) for _ in range(4))
    gidx = torch.tensor([0, 5, 200, 383])
    scale = 1.0 / math.sqrt(Nn)

    qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
    i = torch.arange(M)
    allowed = (i[None, :] - i[:, None]).abs() <= w
    allowed[:, gidx] = True
    allowed[gidx, :] = True
    dense = torch.softmax((qd @ kd.transpose(-1, -2) * scale).masked_fill(~allowed, float("-inf")), -1) @ vd
    dense.backward(go.double())

    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = global_window_attention(qc, kc, vc, w, gidx)
    out.backward(go.cuda())
    torch.cuda.synchronize()
    import helpers as H

    rel = 1e-4 if dtype == torch.float32 else 4e-2
    for name, got, ref in (("o", out, dense), ("gq", qc.grad, qd.grad), ("gk", kc.grad, kd.grad), ("gv", vc.grad, vd.grad)):
        H.assert_lowp_close(got, ref.detach().numpy(), name, rel=rel)


def test_band_row_ranges_are_recognised_without_a_gpu():
    """Which band tensors the wrappers hand over in place: dense ones and row ranges of dense ones (batch stride)."""
    import importlib

    impl = importlib.import_module("window_matmul.window_matmul")
    full = torch.zeros(3, 40, 9)
    assert impl._band_stride(full) == 0
    assert impl._band_stride(full[:, 8:24]) == 40 * 9
    assert impl._band_stride(full[1:]) == 0
    assert impl._band_stride(full[:, :, :5]) is None and impl._band_stride(full[:, ::2]) is None
    t, sb = impl._band_in(full[:, ::2])
    assert sb == 0 and t.is_contiguous()
