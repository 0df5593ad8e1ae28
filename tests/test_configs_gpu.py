"""The benchmark configurations at FULL size on one GPU: size-independent properties over the whole tensors
and oracle parity on slices the CPU finishes in seconds.

Config 1 (fp32, full chain, bit-exact) lives in test_parity_gpu.py::test_config1_chain_fp32; config 4's
sequence sharding and config 5's batch sharding are covered by test_sharded*.py / bench.py --gpus N.

Oracle parity at these sizes works on row slices (helpers.slice_window): rows [r0, r1) of all six results depend on
positions within 2w of the slice only, so the oracle runs on the truncated sequence; and each contraction is checked on
the inputs the GPU actually fed it (the rounded band tensors), which is what holds the 16-bit bound of 1e-2 on every
result, not only on the first."""
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


def _run_boundaries(B, M, sms):
    """(batch entry, first row) of the row tiles at which the one-sweep window backward starts a new CTA run."""
    T = (M + 127) // 128
    total = B * T
    per, rem = divmod(total, sms)
    starts = [k * per + min(k, rem) for k in range(1, min(sms, total))]
    return [(g // T, (g % T) * 128) for g in starts if g % T]


def test_config2_full_size_bf16(wm):
    B, M, Nn, w = 96, 4096, 64, 256
    q, kt, v, go = _seeded(B, M, Nn, torch.bfloat16, 0)
    got = _chain(wm, q, kt, v, go, w)
    _check_properties(wm, got, q, kt, w, M)
    # oracle parity of all six results: the whole first and last batch entry, and slices around starts of CTA runs of
    # the window backward (where a CTA replays the rows before its run), each contraction on the inputs the GPU saw
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    bounds = _run_boundaries(B, M, sms)
    picks = [bounds[i] for i in sorted({0, len(bounds) // 4, len(bounds) // 2, (3 * len(bounds)) // 4, len(bounds) - 1})]
    cases = [(0, 0, M), (B - 1, 0, M)] + [(b, max(0, r - 256), min(M, r + 256)) for b, r in picks]
    H.check_chain_slices(got, q, kt, v, go, w, cases)
    # the one-sweep kernel against the two single-product kernels on the WHOLE tensors (every run boundary): the same
    # products summed in the same order, so they may differ by one rounding of the result at most
    gq2 = wm.band_n(got["ga"], kt.cuda(), w)
    gk2 = wm.band_t(got["ga"], q.cuda(), w)
    for name, x, y in (("gq", got["gq"], gq2), ("gk", got["gk"], gk2)):
        x, y = x.float(), y.float()
        assert ((x - y).abs() <= 2.0 ** -7 * y.abs() + 1e-30).all(), name
        assert (x == y).float().mean() > 0.99, name


def test_config3_full_size_fp16_small_window(wm):
    B, M, Nn, w = 1024, 2048, 32, 8
    q, kt, v, go = _seeded(B, M, Nn, torch.float16, 1, dist="uniform")
    got = _chain(wm, q, kt, v, go, w)
    _check_properties(wm, got, q, kt, w, M)
    H.check_chain_slices(got, q, kt, v, go, w, [(b, 0, M) for b in (0, 1, 511, 1023)])


def test_config4_long_sequence_bf16(wm):
    """B=16, M=65536, N=128, w=512 on ONE GPU (the sharded form is tested in test_sharded_gpu.py): the whole chain, all
    six results against the oracle on the first rows, an interior span that straddles tile boundaries and the last rows
    (the largest offsets) of the first and the last batch entry."""
    B, M, Nn, w = 16, 65536, 128, 512
    q, kt, v, go = _seeded(B, M, Nn, torch.bfloat16, 4)
    got = _chain(wm, q, kt, v, go, w)
    _check_properties(wm, got, q, kt, w, M)
    cases = [(b, r0, r0 + 1024) for b in (0, B - 1) for r0 in (0, 30000, M - 1024)]
    H.check_chain_slices(got, q, kt, v, go, w, cases)


def _block_stage_check(q, kt, v, go, w, scale, st, b, r0, r1):
    """One slice of the attention block, stage by stage against the oracle, each stage on the GPU's own (rounded) inputs.
    st: GPU tensors a (scores), p (probabilities), o, gp, gs (gradient of the scores), gq, gk (of K^T), gv."""
    M = q.shape[1]
    t0, t1 = H.slice_window(M, w, r0, r1)
    f = lambda t: np.ascontiguousarray(t[b:b + 1, t0:t1].float().cpu().numpy())  # noqa: E731
    qs, kts, vs, gos = f(q), f(kt), f(v), f(go)
    ks = np.ascontiguousarray(kts.transpose(0, 2, 1))
    lo, hi = r0 - t0, r1 - t0
    sl = (slice(b, b + 1), slice(r0, r1))
    what = "b=%d rows [%d,%d) " % (b, r0, r1)
    H.assert_lowp_close(st["a"][sl], H.oracle.window_matmul_forward(qs, ks, w)[:, lo:hi], what + "scores")
    a_g, p_g, gp_g, gs_g = f(st["a"]), f(st["p"]), f(st["gp"]), f(st["gs"])
    H.assert_lowp_close(st["p"][sl], H.oracle.band_softmax(a_g, scale, True)[:, lo:hi], what + "probabilities")
    H.assert_lowp_close(st["o"][sl], H.oracle.unwindow_matmul_forward(p_g, vs, w)[:, lo:hi], what + "o")
    gp, gv = H.oracle.unwindow_matmul_backward(p_g, vs, w, gos)
    H.assert_lowp_close(st["gp"][sl], gp[:, lo:hi], what + "grad_p")
    H.assert_lowp_close(st["gv"][sl], gv[:, lo:hi], what + "grad_v")
    gs = H.oracle.band_softmax_backward(p_g, gp_g, scale, True)
    H.assert_lowp_close(st["gs"][sl], gs[:, lo:hi], what + "grad_scores", rel=2e-2)   # a difference of rounded products
    gq, gk = H.oracle.window_matmul_backward(qs, ks, w, gs_g)
    H.assert_lowp_close(st["gq"][sl], gq[:, lo:hi], what + "grad_q")
    H.assert_lowp_close(st["gk"][sl], gk.transpose(0, 2, 1)[:, lo:hi], what + "grad_k")


@pytest.mark.parametrize("softmax", ["torch", "library"])
def test_config5_attention_block_bf16_vs_oracle(wm, softmax):
    """a = window_matmul(q,k,w)/sqrt(N); softmax with out-of-sequence slots at -inf; o = unwindow_matmul(p,v,w);
    backward.  At the config's M, N, w and the batch of one GPU of the 8-way split (B = 8), through the public API, with
    the softmax composed from torch ops as a user of the reference writes it, or with this library's band softmax.
    Every stage is compared with the oracle on slices (first rows, an interior span across tile boundaries, last rows)
    of the first and last batch entry, each stage on the inputs the GPU fed it."""
    import window_matmul as pkg
    from concurrent.futures import ThreadPoolExecutor

    B, M, Nn, w = 8, 16384, 64, 384
    q, kt, v, go = (t.to(torch.bfloat16) for t in _seeded(B, M, Nn, torch.float32, 5, dist="normal"))
    mask = torch.from_numpy(H.out_of_sequence_mask(M, w)).cuda()
    scale = 1.0 / math.sqrt(Nn)
    qd, ktd, vd = (t.cuda().requires_grad_(True) for t in (q, kt, v))
    a = pkg.window_matmul(qd, ktd.transpose(-1, -2), w)
    a.retain_grad()
    if softmax == "torch":
        p = torch.softmax((a.float() * scale).masked_fill(mask, float("-inf")), dim=-1).to(torch.bfloat16)
    else:
        p = pkg.window_softmax(a, scale, True)
    p.retain_grad()
    o = pkg.unwindow_matmul(p, vd, w)
    o.backward(go.cuda())
    torch.cuda.synchronize()
    st = dict(a=a.detach(), p=p.detach(), o=o.detach(), gp=p.grad, gs=a.grad, gq=qd.grad, gk=ktd.grad, gv=vd.grad)
    assert (st["p"][:, mask] == 0).all() and (st["gs"][:, mask] == 0).all()
    for t in st.values():
        assert torch.isfinite(t).all()
    cases = [(b, r0, r0 + 1024) for b in (0, B - 1) for r0 in (0, 7000, M - 1024)]
    H.oracle.band_softmax(np.zeros((1, 2, 3)), 1.0, True)    # (loads the oracle library before the threads start)
    with ThreadPoolExecutor(max_workers=8) as ex:
        for fu in [ex.submit(_block_stage_check, q, kt, v, go, w, scale, st, *c) for c in cases]:
            fu.result()


def test_config5_whole_block_bf16_against_fp32_block(wm):
    """The whole bf16 block against an all-fp32 block through the public API at a looser bound: bf16 rounding of the
    probabilities and of the N(0,1)-scale scores compounds through the softmax (each stage alone is held to 1e-2 in
    test_config5_attention_block_bf16_vs_oracle)."""
    import window_matmul as pkg

    B, M, Nn, w = 4, 16384, 64, 384
    q, kt, v, go = _seeded(B, M, Nn, torch.float32, 5, dist="normal")
    mask = torch.from_numpy(H.out_of_sequence_mask(M, w)).cuda()

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
