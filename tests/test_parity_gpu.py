"""Parity of the CUDA path with the oracle / the reference's golden vectors, through the C ABI."""
import math
import os
import sys

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def wm():
    import importlib

    from window_matmul import _native

    impl = importlib.import_module("window_matmul.window_matmul")  # the module, not the function of that name

    assert torch.cuda.is_available()
    assert os.path.exists(_native.LIB_PATH)
    yield impl
    impl.set_flags(0)
    assert _native.device_status() == 0


def _w(name):
    return int(name.split("_w")[1].split("_")[0])


def _run_all(impl, c, w, dtype, flags):
    """The six contractions through the four native calls, on golden-style inputs (k is (B,N,M))."""
    from window_matmul import _native as N

    q, k, v = (H.to_dev(c[x], dtype) for x in ("q", "k", "v"))
    att, g_band, g_out = (H.to_dev(c[x], dtype) for x in ("att", "g_band", "g_out"))
    old = impl.set_flags(flags)
    try:
        a = impl.window_matmul_forward(q, k, w)
        gq, gk = impl.window_matmul_backward(q, k, w, g_band)
        o = impl.unwindow_matmul_forward(att, v, w)
        gatt, gv = impl.unwindow_matmul_backward(att, v, w, g_out)
    finally:
        impl.set_flags(old)
    torch.cuda.synchronize()
    return dict(a=a, gq=gq, gk=gk, o=o, gatt=gatt, gv=gv)


def test_golden_fp32_fp64_bit_exact_with_split_rounding(wm, golden):
    """Reference CPU results (cpu/window_matmul_cpu.cpp) reproduced bit for bit by the exact-order kernels."""
    from window_matmul import _native as N

    n = 0
    for name, c in golden.items():
        if name.endswith("float16"):
            continue
        dtype = torch.float32 if name.endswith("float32") else torch.float64
        got = _run_all(wm, c, _w(name), dtype, N.FLAG_SPLIT_ROUNDING)
        for key in ("a", "gq", "gk", "o", "gatt", "gv"):
            H.assert_bit_equal(got[key], c[key], name + "/" + key)
        n += 1
    assert n >= 25


def _ref_cuda():
    """The reference's own extension, compiled unmodified (oracle/build_ref.py), CUDA kernels included."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "WITH_CUDA")):
        pytest.skip("compiled reference with CUDA kernels not present")
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    import window_matmul_kernel

    return window_matmul_kernel


def test_golden_fp32_default_fma_close_to_float64_truth(wm, golden):
    """Default fp32 mode (fused multiply-add chains, the order of the reference's CUDA kernels): fused
    and split rounding differ at the 1e-5 level on unit-variance inputs, so the comparand here is the
    float64 oracle, with the error an ascending fp32 chain has; the comparison with the reference's CUDA
    kernels at rtol 1e-5 / atol 1e-6 is test_fp32_default_matches_reference_cuda_kernels."""
    for name, c in golden.items():
        if not name.endswith("float32"):
            continue
        w = _w(name)
        got = _run_all(wm, c, w, torch.float32, 0)
        d = {k: c[k] for k in ("q", "v", "att", "g_band", "g_out")}
        d["kt"] = c["k"].transpose(0, 2, 1)
        want = H.oracle_all(d, w, np.float64)
        for key in ("a", "gq", "gk", "o", "gatt", "gv"):
            H.assert_lowp_close(got[key], want[key], name + "/" + key, rel=2e-5)


@pytest.mark.parametrize("shape", [(2, 16, 3, 4), (2, 130, 64, 64), (2, 257, 128, 32), (4, 1024, 64, 64)])
def test_fp32_default_matches_reference_cuda_kernels(wm, shape):
    """Same seeded inputs through the reference's CUDA kernels (csrc/window_matmul/cuda/window_matmul_cuda.cu)
    and through this library's default fp32 mode: rtol 1e-5 / atol 1e-6, all six results."""
    ref = _ref_cuda()
    B, M, Nn, w = shape
    d = H.rand_inputs(B, M, Nn, w, seed=31)
    q, kt, v, att, g_band, g_out = (H.to_dev(d[x], torch.float32) for x in ("q", "kt", "v", "att", "g_band", "g_out"))
    att = att * torch.from_numpy(~H.out_of_sequence_mask(M, w)).cuda()  # the reference's kernels read those slots
    k = kt.transpose(-1, -2)
    torch.cuda.synchronize()  # the reference launches on the legacy default stream
    want = {}
    want["a"] = ref.window_matmul_forward(q, k, w)
    want["gq"], want["gk"] = ref.window_matmul_backward(q, k, w, g_band)
    want["o"] = ref.unwindow_matmul_forward(att, v, w)
    want["gatt"], want["gv"] = ref.unwindow_matmul_backward(att, v, w, g_out)
    torch.cuda.synchronize()
    got = {}
    got["a"] = wm.window_matmul_forward(q, k, w)
    got["gq"], got["gk"] = wm.window_matmul_backward(q, k, w, g_band)
    got["o"] = wm.unwindow_matmul_forward(att, v, w)
    got["gatt"], got["gv"] = wm.unwindow_matmul_backward(att, v, w, g_out)
    torch.cuda.synchronize()
    for key in got:
        H.assert_fp32_close(got[key], want[key].cpu().numpy(), key)


def test_golden_fp16_inputs_against_fp32_oracle(wm, golden):
    """The reference accumulates fp16 in fp16; these kernels accumulate in fp32, so the comparand is the
    fp32 oracle on the same fp16 inputs, and the reference's own fp16 output must not be closer to it."""
    for name, c in golden.items():
        if not name.endswith("float16"):
            continue
        w = _w(name)
        got = _run_all(wm, c, w, torch.float16, 0)
        d32 = {k: c[k].astype(np.float32) for k in ("q", "v", "att", "g_band", "g_out")}
        d32["kt"] = c["k"].astype(np.float32).transpose(0, 2, 1)
        want = H.oracle_all(d32, w)
        for key in ("a", "gq", "o", "gatt", "gv"):
            H.assert_lowp_close(got[key], want[key], name + "/" + key)
        H.assert_lowp_close(got["gk"], want["gk"], name + "/gk")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64])
@pytest.mark.parametrize("shape", [(2, 1, 3, 1), (2, 4, 3, 16), (3, 100, 20, 7), (2, 130, 64, 64), (1, 300, 32, 8),
                                   (2, 257, 128, 32)])
def test_ops_against_oracle_all_dtypes(wm, shape, dtype):
    B, M, Nn, w = shape
    d = H.rand_inputs(B, M, Nn, w, seed=11)
    if dtype in (torch.float16, torch.bfloat16):
        d = {k: H.round_to(v, dtype) for k, v in d.items()}
    c = dict(d)
    c["k"] = np.ascontiguousarray(d["kt"].transpose(0, 2, 1))
    got = _run_all(wm, c, w, dtype, 0)
    want = H.oracle_all(d, w, np.float64 if dtype == torch.float64 else np.float32)
    for key in ("a", "gq", "gk", "o", "gatt", "gv"):
        if dtype in (torch.float16, torch.bfloat16):
            H.assert_lowp_close(got[key], want[key], key)
        elif dtype == torch.float32:
            # fused multiply-add chains vs the oracle's separately rounded ones: see
            # test_golden_fp32_default_fma_close_to_float64_truth
            H.assert_lowp_close(got[key], want[key], key, rel=2e-5)
        else:
            np.testing.assert_allclose(got[key].cpu().numpy(), want[key], rtol=1e-12, atol=1e-12)
    mask = H.out_of_sequence_mask(M, w)
    for key in ("a", "gatt"):
        assert (got[key].float().cpu().numpy()[:, mask] == 0).all(), key + ": out-of-sequence entries must be exactly 0"


@pytest.mark.parametrize("k_layout", ["transposed_view", "contiguous_bnm"])
def test_k_in_both_memory_orders_and_grad_k_shape(wm, k_layout):
    B, M, Nn, w = 2, 70, 16, 9
    d = H.rand_inputs(B, M, Nn, w, seed=5)
    q = H.to_dev(d["q"], torch.float32)
    kt = H.to_dev(d["kt"], torch.float32)
    k = kt.transpose(-1, -2) if k_layout == "transposed_view" else kt.transpose(-1, -2).contiguous()
    assert k.shape == (B, Nn, M)
    g_band = H.to_dev(d["g_band"], torch.float32)
    want = H.oracle_all(d, w)
    a = wm.window_matmul_forward(q, k, w)
    gq, gk = wm.window_matmul_backward(q, k, w, g_band)
    assert gk.shape == (B, Nn, M)
    H.assert_lowp_close(a, want["a"], "a", rel=2e-5)
    H.assert_lowp_close(gq, want["gq"], "gq", rel=2e-5)
    H.assert_lowp_close(gk, want["gk"], "gk", rel=2e-5)


def test_unwindow_never_reads_out_of_sequence_band_slots(wm):
    B, M, Nn, w = 2, 40, 8, 12
    d = H.rand_inputs(B, M, Nn, w, seed=9)
    mask = H.out_of_sequence_mask(M, w)
    poisoned = d["att"].copy()
    poisoned[:, mask] = np.nan
    v, g_out = H.to_dev(d["v"], torch.float32), H.to_dev(d["g_out"], torch.float32)
    want = H.oracle_all(d, w)
    o = wm.unwindow_matmul_forward(H.to_dev(poisoned, torch.float32), v, w)
    gatt, gv = wm.unwindow_matmul_backward(H.to_dev(poisoned, torch.float32), v, w, g_out)
    H.assert_lowp_close(o, want["o"], "o", rel=2e-5)
    H.assert_lowp_close(gv, want["gv"], "gv", rel=2e-5)
    H.assert_lowp_close(gatt, want["gatt"], "gatt", rel=2e-5)


# ---- the reference's three-way scheme through the public, differentiable API ----------------------

REF_DIMS = [(2, 1, 1, 3), (2, 1, 4, 3), (2, 1, 16, 3), (2, 1, 32, 3), (2, 1, 16, 32)]  # tests/conftest.py:5-11
REF_WINDOWS = [0, 1, 4, 16]  # tests/conftest.py:13


def _head_split(x: torch.Tensor, heads: int) -> torch.Tensor:
    """(B, M, heads*N) -> non-contiguous (B, heads, M, N) view, as the reference's helpers build their
    inputs (tests/utils.py:38-43)."""
    B, M, HN = x.shape
    return x.view(B, M, heads, HN // heads).transpose(-2, -3)


def _strided_windows(x: torch.Tensor, w: int) -> torch.Tensor:
    """Independent torch formulation: zero-pad w rows each side, sliding windows of 2w+1 rows."""
    M, Nn = x.shape[-2:]
    p = torch.nn.functional.pad(x, (0, 0, w, w))
    return p.unfold(-2, 2 * w + 1, 1).transpose(-1, -2)  # (..., M, 2w+1, N)


@pytest.mark.parametrize("dim", REF_DIMS)
@pytest.mark.parametrize("w", REF_WINDOWS)
def test_three_way_window_matmul(wm, dim, w):
    import window_matmul as pkg

    B, Hh, M, Nn = dim
    g = torch.Generator().manual_seed(42)
    q0 = _head_split(torch.randn(B, M, Hh * Nn, generator=g), Hh).cuda()
    k0 = _head_split(torch.randn(B, M, Hh * Nn, generator=g), Hh).cuda()
    outs = {}
    for name in ("custom", "strided"):
        q = q0.detach().clone().requires_grad_(True)
        k = k0.detach().clone().requires_grad_(True)
        if name == "custom":
            att = pkg.window_matmul(q, k.transpose(-1, -2), w)
        else:
            att = torch.matmul(q.unsqueeze(-2), _strided_windows(k, w).transpose(-1, -2)).squeeze(-2)
        assert att.shape == (B, Hh, M, 2 * w + 1)
        (att * torch.arange(att.numel(), device=att.device).to(att).view_as(att)).mean().backward()
        outs[name] = (att.detach(), q.grad, k.grad)
    for x, y in zip(outs["custom"], outs["strided"]):
        assert torch.allclose(x, y, atol=1e-6)
    if w:
        # ... and the oracle (the reference's defining loops) as third leg
        a = H.oracle.window_matmul_forward(
            q0.reshape(-1, M, Nn).cpu().numpy(), k0.reshape(-1, M, Nn).transpose(-1, -2).contiguous().cpu().numpy(), w)
        assert np.allclose(outs["custom"][0].reshape(-1, M, 2 * w + 1).cpu().numpy(), a, atol=1e-6)


@pytest.mark.parametrize("dim", REF_DIMS)
@pytest.mark.parametrize("w", REF_WINDOWS)
def test_three_way_unwindow_matmul(wm, dim, w):
    import window_matmul as pkg

    B, Hh, M, Nn = dim
    g = torch.Generator().manual_seed(43)
    att0 = torch.randn(B, Hh, M, 2 * w + 1, generator=g)
    mask = torch.from_numpy(H.out_of_sequence_mask(M, w))
    att0[..., mask] = 0  # tests/utils.py:79-81 of the reference zeroes the out-of-sequence corners
    att0 = att0.cuda()
    v0 = _head_split(torch.randn(B, M, Hh * Nn, generator=g), Hh).cuda()
    outs = {}
    for name in ("custom", "strided"):
        att = att0.detach().clone().requires_grad_(True)
        v = v0.detach().clone().requires_grad_(True)
        if name == "custom":
            out = pkg.unwindow_matmul(att, v, w)
        else:
            out = torch.matmul(att.unsqueeze(-2), _strided_windows(v, w)).squeeze(-2)
        assert out.shape == (B, Hh, M, Nn)
        (out * torch.arange(out.numel(), device=out.device).to(out).view_as(out)).mean().backward()
        outs[name] = (out.detach(), att.grad, v.grad)
    o1, ga1, gv1 = outs["custom"]
    o2, ga2, gv2 = outs["strided"]
    assert torch.allclose(o1, o2, atol=1e-6) and torch.allclose(gv1, gv2, atol=1e-6)
    # the strided formulation has a (harmless) gradient in the zeroed corners; compare inside the sequence
    assert torch.allclose(ga1[..., ~mask.cuda()], ga2[..., ~mask.cuda()], atol=1e-6)
    assert (ga1[..., mask.cuda()] == 0).all()


@pytest.mark.parametrize("dim", REF_DIMS)
@pytest.mark.parametrize("w", REF_WINDOWS)
def test_window_attention_network(wm, dim, w):
    """tests/test_attention.py:90-140 of the reference: three attention layers chained through both ops,
    outputs and all input gradients at atol 1e-6 against an independent torch formulation."""
    import window_matmul as pkg

    B, Hh, M, Nn = dim
    torch.manual_seed(42)
    linear = torch.nn.Linear(Nn, Nn).cuda()
    g = torch.Generator().manual_seed(44)
    base = [_head_split(torch.randn(B, M, Hh * Nn, generator=g), Hh).cuda() for _ in range(3)]

    def layer(q, k, v, custom):
        kt = k.transpose(-1, -2)
        if custom:
            s = pkg.window_matmul(q, kt, w)
        elif w:
            s = torch.matmul(q.unsqueeze(-2), _strided_windows(k, w).transpose(-1, -2)).squeeze(-2)
        else:
            s = (q * k).sum(-1, keepdim=True)
        p = torch.nn.functional.softmax(s / math.sqrt(Nn), dim=-1)
        if custom:
            o = pkg.unwindow_matmul(p, v, w)
        elif w:
            o = torch.matmul(p.unsqueeze(-2), _strided_windows(v, w)).squeeze(-2)
        else:
            o = p * v
        return torch.sigmoid(linear(o))

    res = {}
    for custom in (True, False):
        q, k, v = (t.detach().clone().requires_grad_(True) for t in base)
        qq, kk, vv = q, k, v
        for _ in range(3):
            out = layer(qq, kk, vv, custom)
            qq = kk = vv = linear(out)
        out.mean().backward()
        res[custom] = (out.detach(), q.grad, k.grad, v.grad)
    for x, y in zip(res[True], res[False]):
        assert torch.allclose(x, y, atol=1e-6)


def test_leading_dims_dtype_rule_and_errors(wm):
    import window_matmul as pkg

    q = torch.randn(2, 3, 24, 8, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(2, 3, 8, 24, device="cuda", dtype=torch.bfloat16)
    a = pkg.window_matmul(q, k, 5)
    assert a.shape == (2, 3, 24, 11) and a.dtype == torch.bfloat16
    o = pkg.unwindow_matmul(a, q, 5)
    assert o.shape == q.shape and o.dtype == torch.bfloat16
    with pytest.raises(RuntimeError, match="Input mismatch"):
        wm.window_matmul_forward(q.reshape(6, 24, 8), k.reshape(6, 8, 24)[:, :, :20], 5)
    with pytest.raises(RuntimeError, match="Input mismatch"):
        wm.unwindow_matmul_forward(a.reshape(6, 24, 11), q.reshape(6, 24, 8), 4)
    with pytest.raises(RuntimeError, match="scalar type"):
        wm.window_matmul_forward(q.reshape(6, 24, 8), k.reshape(6, 8, 24).float(), 5)
    with pytest.raises(RuntimeError, match="not implemented"):
        wm.band_nt(q.reshape(6, 24, 8).to(torch.int32), q.reshape(6, 24, 8).to(torch.int32), 5)


def test_autocast_casts_to_fp16_like_the_reference(wm):
    import window_matmul as pkg

    q = torch.randn(2, 16, 8, device="cuda")
    k = torch.randn(2, 8, 16, device="cuda")
    with torch.autocast("cuda"):
        a = pkg.window_matmul(q, k, 3)
    assert a.dtype == torch.float16  # window_matmul/window_matmul.py:9 of the reference


def test_only_needed_gradients_are_computed(wm):
    import window_matmul as pkg
    from window_matmul import _native as N

    q = torch.randn(2, 16, 8, device="cuda", requires_grad=True)
    k = torch.randn(2, 8, 16, device="cuda")
    a = pkg.window_matmul(q, k, 3)
    before = N.launch_count()
    a.sum().backward()
    assert N.launch_count() - before == 1 and q.grad is not None


# ---- sharded geometry: a slice of the sequence plus halo equals the same slice of the full result ----


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_primitives_on_a_sequence_shard(wm, dtype):
    B, M, Nn, w = 2, 96, 16, 10
    d = H.rand_inputs(B, M, Nn, w, seed=21)
    if dtype != torch.float32:
        d = {k: H.round_to(v, dtype) for k, v in d.items()}
    want = H.oracle_all(d, w)
    close = (lambda g, w_, n: H.assert_lowp_close(g, w_, n, rel=2e-5)) if dtype == torch.float32 else H.assert_lowp_close
    parts = 3
    Ml = M // parts
    gv_sum = np.zeros((B, M + 2 * w, Nn), dtype=np.float64)
    for r in range(parts):
        m0 = r * Ml
        pad = lambda x: np.pad(x, ((0, 0), (w, w), (0, 0)))[:, m0:m0 + Ml + 2 * w]  # rows m0-w .. m0+Ml+w
        seq = (max(0, w - m0), min(Ml + 2 * w, M - m0 + w))
        q, g_out = (H.to_dev(d[x][:, m0:m0 + Ml], dtype) for x in ("q", "g_out"))
        att = H.to_dev(d["att"][:, m0:m0 + Ml], dtype)
        kt_ext, v_ext = H.to_dev(pad(d["kt"]), dtype), H.to_dev(pad(d["v"]), dtype)
        a = wm.band_nt(q, kt_ext, w, other_off=w, seq=seq)
        close(a, want["a"][:, m0:m0 + Ml], "a shard %d" % r)
        o = wm.band_n(att, v_ext, w, other_off=w, seq=seq)
        close(o, want["o"][:, m0:m0 + Ml], "o shard %d" % r)
        part = wm.band_t(att, g_out, w, other_rows=Ml + 2 * w, other_off=w, seq=seq)
        assert (part[:, :seq[0]] == 0).all() and (part[:, seq[1]:] == 0).all()
        gv_sum[:, m0:m0 + Ml + 2 * w] += part.double().cpu().numpy()
    got = torch.from_numpy(gv_sum[:, w:w + M]).float()
    H.assert_lowp_close(got, want["gv"], "gv summed over shards", rel=1e-2 if dtype != torch.float32 else 1e-5)


# ---- full-size configuration 1 (fp32): the whole chain against the oracle ---------------------------


def test_config1_chain_fp32(wm):
    """B=4, M=1024, N=64, w=64, N(0,1) inputs from seed 0, k as contiguous (B,N,M): window -> unwindow ->
    backward.  Split rounding is bit-identical to the reference's CPU loops; the default fused
    multiply-add order is compared against the float64 oracle with the error the fp32 reference itself has."""
    import window_matmul as pkg
    from window_matmul import _native as N

    B, M, Nn, w = 4, 1024, 64, 64
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(B, M, Nn, generator=g), torch.randn(B, Nn, M, generator=g), torch.randn(B, M, Nn, generator=g)
    go = torch.randn(B, M, Nn, generator=g)
    a_ref, o_ref, gq_ref, gk_ref, ga_ref, gv_ref = H.oracle.chain_fwd_bwd(q.numpy(), k.numpy(), v.numpy(), w, go.numpy())
    for flags, exact in ((N.FLAG_SPLIT_ROUNDING, True), (0, False)):
        old = wm.set_flags(flags)
        try:
            qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
            a = pkg.window_matmul(qd, kd, w)
            a.retain_grad()
            o = pkg.unwindow_matmul(a, vd, w)
            o.backward(go.cuda())
        finally:
            wm.set_flags(old)
        got = dict(a=a.detach(), o=o.detach(), gq=qd.grad, gk=kd.grad, ga=a.grad, gv=vd.grad)
        want = dict(a=a_ref, o=o_ref, gq=gq_ref, gk=gk_ref, ga=ga_ref, gv=gv_ref)
        for key in got:
            if exact:
                H.assert_bit_equal(got[key], want[key], "config 1 " + key)
            else:
                # same inputs in float64 = ground truth; the fp32 result must be as close to it as an
                # ascending fp32 chain can be (error grows with the magnitude of the partial sums)
                H.assert_lowp_close(got[key], want[key].astype(np.float64), "config 1 fma " + key, rel=2e-5)
        mask = H.out_of_sequence_mask(M, w)
        assert (got["a"].cpu().numpy()[:, mask] == 0).all() and (got["ga"].cpu().numpy()[:, mask] == 0).all()
        assert abs(mask.mean() - 0.03149) < 1e-4  # 3.149 % of the band is out of sequence at this shape


def test_host_pipeline_matches_direct_calls(wm):
    """Host tensors streamed through the GPU in batch chunks give the same results as one device-resident call."""
    from window_matmul.host_pipeline import batched_host_call

    B, M, Nn, w = 10, 128, 64, 64
    g = torch.Generator().manual_seed(3)
    q, kt, v = (torch.randn(B, M, Nn, generator=g).to(torch.bfloat16).pin_memory() for _ in range(3))

    def fn(qd, ktd, vd):
        a = wm.window_matmul_forward(qd, ktd.transpose(-1, -2), w)
        return a, wm.unwindow_matmul_forward(a, vd, w)

    a_h, o_h = batched_host_call(fn, [q, kt, v], chunks=4)
    a_d, o_d = fn(q.cuda(), kt.cuda(), v.cuda())
    assert not a_h.is_cuda and a_h.shape == (B, M, 2 * w + 1)
    assert torch.equal(a_h, a_d.cpu()) and torch.equal(o_h, o_d.cpu())
    with pytest.raises(RuntimeError, match="host tensors"):
        batched_host_call(fn, [q.cuda(), kt, v])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_empty_single_row_and_window_wider_than_the_sequence(wm, dtype):
    """Edge sizes through the public operators: no batch entries, no rows, one row, a window several times the
    sequence length (every band slot but a few is out of sequence).  Forward and backward, against the oracle."""
    import window_matmul as pkg

    for B, M, Nn, w in [(0, 8, 4, 2), (2, 0, 4, 2)]:
        q = torch.zeros(B, M, Nn, dtype=dtype, device="cuda", requires_grad=True)
        k = torch.zeros(B, Nn, M, dtype=dtype, device="cuda", requires_grad=True)
        a = pkg.window_matmul(q, k, w)
        assert a.shape == (B, M, 2 * w + 1)
        o = pkg.unwindow_matmul(a, torch.zeros(B, M, Nn, dtype=dtype, device="cuda"), w)
        assert o.shape == (B, M, Nn)
        o.sum().backward()
        assert q.grad.shape == q.shape and k.grad.shape == k.shape
    for B, M, Nn, w in [(3, 1, 8, 3), (2, 5, 64, 16), (1, 8, 32, 64)]:
        d = {key: H.round_to(val, dtype) for key, val in H.rand_inputs(B, M, Nn, w, seed=B + M + w).items()}
        want = H.oracle.chain_fwd_bwd(d["q"], np.ascontiguousarray(d["kt"].transpose(0, 2, 1)), d["v"], w, d["g_out"])
        q, kt, v = (H.to_dev(d[key], dtype).requires_grad_(True) for key in ("q", "kt", "v"))
        a = pkg.window_matmul(q, kt.transpose(-1, -2), w)
        a.retain_grad()
        o = pkg.unwindow_matmul(a, v, w)
        o.backward(H.to_dev(d["g_out"], dtype))
        got = (a, o, q.grad, kt.grad.transpose(1, 2), a.grad, v.grad)
        for name, x, y in zip(("a", "o", "gq", "gk", "ga", "gv"), got, want):
            if dtype == torch.float32:
                H.assert_lowp_close(x, y, "%s %s" % (name, (B, M, Nn, w)), rel=2e-5)
            else:
                H.assert_lowp_close(x, y, "%s %s" % (name, (B, M, Nn, w)), rel=4e-2 if name != "a" else 1e-2)
        outside = H.out_of_sequence_mask(M, w)
        assert (a.detach().float().cpu().numpy()[:, outside] == 0).all() and (a.grad.float().cpu().numpy()[:, outside] == 0).all()
