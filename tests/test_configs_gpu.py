"""The benchmark configurations at FULL size on one GPU: size-independent properties over the whole tensors
and oracle parity on slices the CPU finishes in seconds.

Config 1 (fp32, full chain, bit-exact) lives in test_parity_gpu.py::test_config1_chain_fp32; config 4's
sequence sharding and config 5's batch sharding are covered by test_sharded*.py / bench.py --gpus N."""
import importlib
import math

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def wm():
    from window_matmul import _native

    impl = importlib.import_module("window_matmul.window_matmul")
    yield impl
    assert _native.device_status() == 0


def _seeded(B, M, N, dtype, seed, dist="normal_scaled"):
    g = torch.Generator().manual_seed(seed)
    if dist == "uniform":
        mk = lambda: torch.rand(B, M, N, generator=g)  # noqa: E731
    else:
        s = 1.0 / math.sqrt(N) if dist == "normal_scaled" else 1.0
        mk = lambda: torch.randn(B, M, N, generator=g) * s  # noqa: E731
    return [mk().to(dtype) for _ in range(4)]  # q, k^T, v, upstream grad


def _oracle_rows(q, kt, v, w, rows):
    """Oracle on the first `rows` rows of one sequence: those rows only see positions < rows + w, so the
    truncated sequence of rows + w positions gives the same values."""
    n = rows + w
    q, kt, v = (t[:, :n].float().numpy() for t in (q, kt, v))
    a = H.oracle.window_matmul_forward(q, np.ascontiguousarray(kt.transpose(0, 2, 1)), w)
    return a[:, :rows]


def _chain(wm, q, kt, v, go, w):
    import window_matmul as pkg

    qd, ktd, vd = (t.cuda().requires_grad_(True) for t in (q, kt, v))
    a = pkg.window_matmul(qd, ktd.transpose(-1, -2), w)
    a.retain_grad()
    o = pkg.unwindow_matmul(a, vd, w)
    o.backward(go.cuda())
    torch.cuda.synchronize()
    return dict(a=a.detach(), o=o.detach(), gq=qd.grad, gk=ktd.grad, gv=vd.grad, ga=a.grad)


def _check_properties(wm, got, q, kt, w, M):
    """Size-independent checks on the whole tensors."""
    from window_matmul import _native as N

    mask = torch.from_numpy(H.out_of_sequence_mask(M, w)).cuda()
    assert (got["a"][:, mask] == 0).all() and (got["ga"][:, mask] == 0).all()
    for t in got.values():
        assert torch.isfinite(t).all()
    # exact homogeneity: scaling Q by 2 scales the band by exactly 2 (a power of two commutes with rounding)
    a2 = wm.band_nt((q * 2).cuda(), kt.cuda(), w)
    assert torch.equal(a2, got["a"] * 2)
    # batch entries are independent: reversing the batch reverses the result bit for bit
    ar = wm.band_nt(q.flip(0).cuda(), kt.flip(0).cuda(), w)
    assert torch.equal(ar, got["a"].flip(0))
    # the tensor-core path really ran where it should
    if q.dtype != torch.float32:
        assert N.lib.wmm_query_path(N.BAND_NT, N.operand(q.cuda()), N.operand(kt.cuda()), got["a"].data_ptr(),
                                    N.geometry(q.shape[0], M, q.shape[2], w), N.dtype_code(q), 0) in (1, 2)


def test_config2_full_size_bf16(wm):
    B, M, Nn, w = 96, 4096, 64, 256
    q, kt, v, go = _seeded(B, M, Nn, torch.bfloat16, 0)
    got = _chain(wm, q, kt, v, go, w)
    _check_properties(wm, got, q, kt, w, M)
    # oracle parity of all six results on the first and the last batch entry
    for b in (0, B - 1):
        sl = slice(b, b + 1)
        d = dict(q=q[sl].float().numpy(), kt=kt[sl].float().numpy(), v=v[sl].float().numpy())
        a, o, gq, gk, ga, gv = H.oracle.chain_fwd_bwd(d["q"], np.ascontiguousarray(d["kt"].transpose(0, 2, 1)), d["v"], w,
                                                      go[sl].float().numpy())
        H.assert_lowp_close(got["a"][sl], a, "a")
        # downstream of A the kernels consume the bf16-rounded band, the oracle the fp32 one
        for key, want in dict(o=o, ga=ga, gq=gq, gk=gk.transpose(0, 2, 1), gv=gv).items():
            H.assert_lowp_close(got[key][sl], want, key, rel=4e-2)


def test_config3_full_size_fp16_small_window(wm):
    B, M, Nn, w = 1024, 2048, 32, 8
    q, kt, v, go = _seeded(B, M, Nn, torch.float16, 1, dist="uniform")
    got = _chain(wm, q, kt, v, go, w)
    _check_properties(wm, got, q, kt, w, M)
    sl = slice(0, 4)
    a, o, gq, gk, ga, gv = H.oracle.chain_fwd_bwd(q[sl].float().numpy(), np.ascontiguousarray(kt[sl].float().numpy().transpose(0, 2, 1)),
                                                  v[sl].float().numpy(), w, go[sl].float().numpy())
    H.assert_lowp_close(got["a"][sl], a, "a")
    for key, want in dict(o=o, ga=ga, gq=gq, gk=gk.transpose(0, 2, 1), gv=gv).items():
        H.assert_lowp_close(got[key][sl], want, key, rel=4e-2)


def test_config4_long_sequence_bf16(wm):
    """B=16, M=65536, N=128, w=512 on ONE GPU (the sharded form is tested in test_sharded_gpu.py)."""
    B, M, Nn, w = 16, 65536, 128, 512
    q, kt, v, go = _seeded(B, M, Nn, torch.bfloat16, 4)
    a = wm.band_nt(q.cuda(), kt.cuda(), w)
    torch.cuda.synchronize()
    mask = torch.from_numpy(H.out_of_sequence_mask(M, w)).cuda()
    assert (a[:, mask] == 0).all() and torch.isfinite(a).all()
    rows = 1024
    want = _oracle_rows(q[:1], kt[:1], v[:1], w, rows)
    H.assert_lowp_close(a[:1, :rows], want, "a, first rows")
    # the rest of the chain against the exact-order CUDA-core kernels on one batch entry
    from window_matmul import _native as N

    vd, gd, ad = v[:1].cuda(), go[:1].cuda(), a[:1].contiguous()
    o = wm.band_n(ad, vd, w)
    gv = wm.band_t(ad, gd, w)
    o_ref = wm.band_n(ad.float(), vd.float(), w, flags=N.FLAG_FORCE_GENERIC)
    gv_ref = wm.band_t(ad.float(), gd.float(), w, flags=N.FLAG_FORCE_GENERIC)
    H.assert_lowp_close(o, o_ref.cpu().numpy(), "o")
    H.assert_lowp_close(gv, gv_ref.cpu().numpy(), "gv")


def test_config5_attention_block_bf16_vs_fp32(wm):
    """a = window_matmul(q,k,w)/sqrt(N); softmax with out-of-sequence slots at -inf; o = unwindow_matmul(p,v,w);
    backward.  At the config's M, N, w and a reduced batch.  Every one of the six contractions of the bf16
    block is compared at 1e-2 with the exact-order fp32 kernels on the SAME (bf16-valued) inputs; the whole
    block is then compared with an all-fp32 block at a looser bound, because bf16 rounding of the
    probabilities and of the N(0,1)-scale scores compounds through the softmax."""
    import window_matmul as pkg
    from window_matmul import _native as N

    B, M, Nn, w = 4, 16384, 64, 384
    q, kt, v, go = _seeded(B, M, Nn, torch.float32, 5, dist="normal")
    mask = torch.from_numpy(H.out_of_sequence_mask(M, w)).cuda()
    G = N.FLAG_FORCE_GENERIC

    # ---- per contraction, identical inputs ----
    bf = torch.bfloat16
    qb, ktb, vb, gob = (t.to(bf).cuda() for t in (q, kt, v, go))
    kb = ktb.transpose(-1, -2)
    a = wm.window_matmul_forward(qb, kb, w)
    H.assert_lowp_close(a, wm.band_nt(qb.float(), ktb.float(), w, flags=G).cpu().numpy(), "a")
    s = (a.float() / math.sqrt(Nn)).masked_fill(mask, float("-inf")).requires_grad_(True)
    pf = torch.softmax(s, dim=-1)
    p = pf.to(bf)
    o = wm.unwindow_matmul_forward(p, vb, w)
    H.assert_lowp_close(o, wm.band_n(p.float(), vb.float(), w, flags=G).cpu().numpy(), "o")
    gp, gv = wm.unwindow_matmul_backward(p, vb, w, gob)
    H.assert_lowp_close(gp, wm.band_nt(gob.float(), vb.float(), w, flags=G).cpu().numpy(), "grad_p")
    H.assert_lowp_close(gv, wm.band_t(p.float(), gob.float(), w, flags=G).cpu().numpy(), "grad_v")
    (gs,) = torch.autograd.grad(pf, s, gp.float())
    gs = (gs / math.sqrt(Nn)).to(bf)
    assert (gs[:, mask] == 0).all()
    gq, gk = wm.window_matmul_backward(qb, kb, w, gs)
    H.assert_lowp_close(gq, wm.band_n(gs.float(), ktb.float(), w, flags=G).cpu().numpy(), "grad_q")
    H.assert_lowp_close(gk.transpose(-1, -2), wm.band_t(gs.float(), qb.float(), w, flags=G).cpu().numpy(), "grad_k")
    del a, s, pf, p, gp, gs

    # ---- the whole block through the public API ----
    def block(dtype):
        qd, ktd, vd = (t.to(dtype).cuda().requires_grad_(True) for t in (q, kt, v))
        sc = pkg.window_matmul(qd, ktd.transpose(-1, -2), w) / math.sqrt(Nn)
        sc = sc.masked_fill(mask, float("-inf"))
        pr = torch.softmax(sc.float(), dim=-1).to(dtype)
        out = pkg.unwindow_matmul(pr, vd, w)
        out.backward(go.to(dtype).cuda())
        return [t.detach().float() for t in (out, qd.grad, ktd.grad, vd.grad)]

    lo = block(torch.bfloat16)
    ref = block(torch.float32)
    for name, x, y in zip(("o", "gq", "gk", "gv"), lo, ref):
        H.assert_lowp_close(x, y.cpu().numpy(), name, rel=1e-1)


def test_config5_attention_block_with_band_softmax(wm):
    """The same block with this library's band softmax between the operators instead of the torch ops: on identical
    bf16 scores its probabilities and score gradients match torch's fp32 softmax of the masked, scaled scores at the
    16-bit bound, and the whole fused block (bf16) stays within the bound of the all-fp32 torch-composed block."""
    import window_matmul as pkg
    from window_matmul import softmax as sm

    B, M, Nn, w = 2, 16384, 64, 384
    q, kt, v, go = _seeded(B, M, Nn, torch.float32, 5, dist="normal")
    mask = torch.from_numpy(H.out_of_sequence_mask(M, w)).cuda()
    bf = torch.bfloat16
    scale = 1.0 / math.sqrt(Nn)

    a = wm.window_matmul_forward(q.to(bf).cuda(), kt.to(bf).cuda().transpose(-1, -2), w)
    s = (a.float() * scale).masked_fill(mask, float("-inf")).requires_grad_(True)
    pf = torch.softmax(s, dim=-1)
    p = sm.band_softmax(a, scale, True)
    assert (p[:, mask] == 0).all()
    H.assert_lowp_close(p, pf.detach().cpu().numpy(), "probabilities")
    gp = torch.randn(p.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)).to(bf)
    (gs_ref,) = torch.autograd.grad(pf, s, gp.float())
    # backward from the same (bf16) probabilities the kernel saved
    pb = p.float().requires_grad_(True)
    gs = sm.band_softmax_backward(p, gp, scale, True)
    assert (gs[:, mask] == 0).all()
    H.assert_lowp_close(gs, (gs_ref * scale).cpu().numpy(), "grad_scores", rel=2e-2)
    del a, s, pf, p, gp, gs, gs_ref, pb

    def fused_block(dtype):
        qd, ktd, vd = (t.to(dtype).cuda().requires_grad_(True) for t in (q, kt, v))
        pr = pkg.window_softmax(pkg.window_matmul(qd, ktd.transpose(-1, -2), w), scale, True)
        out = pkg.unwindow_matmul(pr, vd, w)
        out.backward(go.to(dtype).cuda())
        return [t.detach().float() for t in (out, qd.grad, ktd.grad, vd.grad)]

    def torch_block_fp32():
        qd, ktd, vd = (t.cuda().requires_grad_(True) for t in (q, kt, v))
        sc = (pkg.window_matmul(qd, ktd.transpose(-1, -2), w) * scale).masked_fill(mask, float("-inf"))
        out = pkg.unwindow_matmul(torch.softmax(sc, dim=-1), vd, w)
        out.backward(go.cuda())
        return [t.detach() for t in (out, qd.grad, ktd.grad, vd.grad)]

    ref = torch_block_fp32()
    for name, x, y in zip(("o", "gq", "gk", "gv"), fused_block(torch.float32), ref):
        H.assert_lowp_close(x, y.cpu().numpy(), name + " fp32", rel=1e-4)
    for name, x, y in zip(("o", "gq", "gk", "gv"), fused_block(bf), ref):
        H.assert_lowp_close(x, y.cpu().numpy(), name + " bf16", rel=1e-1)
