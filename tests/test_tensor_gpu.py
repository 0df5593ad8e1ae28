"""The tcgen05 kernels (16-bit inputs) against the fp32 oracle on the same rounded inputs.  Every call
passes WMM_FLAG_REQUIRE_TENSOR, so a silent fall-back to the CUDA-core kernels fails the test."""
import importlib

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

# (B, M, N, w): the window and hidden sizes of the benchmark configurations at reduced B and M, ragged
# last tiles (M not a multiple of 128), windows that end inside a chunk, one-chunk windows
SHAPES = [
    (2, 512, 64, 64),
    (1, 1024, 64, 256),
    (2, 200, 64, 64),
    (3, 136, 64, 4),
    (1, 640, 64, 12),
    (2, 384, 128, 128),
    (1, 1152, 128, 512),
    (4, 256, 32, 8),
    (1, 768, 64, 384),
    (2, 8, 64, 4),
]


# small-window family (w <= 32): any window, ragged and odd sequence lengths, all three hidden sizes
SMALL_SHAPES = [(2, 300, 32, 1), (3, 129, 64, 5), (2, 100, 128, 16), (1, 1, 32, 3), (2, 257, 64, 32), (5, 77, 32, 17),
                (1, 2048, 32, 8)]


@pytest.fixture(scope="module")
def wm():
    from window_matmul import _native

    impl = importlib.import_module("window_matmul.window_matmul")
    yield impl
    assert _native.device_status() == 0, "a tensor-core kernel abandoned a bounded wait"


def _inputs(shape, dtype, seed=3):
    B, M, Nn, w = shape
    d = H.rand_inputs(B, M, Nn, w, seed=seed, scale=1.0 / np.sqrt(Nn))
    return {k: H.round_to(v, dtype) for k, v in d.items()}


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", SHAPES)
def test_band_nt_tensor(wm, shape, dtype):
    from window_matmul import _native as N

    B, M, Nn, w = shape
    d = _inputs(shape, dtype)
    want = H.oracle.window_matmul_forward(d["q"], np.ascontiguousarray(d["kt"].transpose(0, 2, 1)), w)
    q, kt = H.to_dev(d["q"], dtype), H.to_dev(d["kt"], dtype)
    band = torch.full((B, M, 2 * w + 1), float("nan"), dtype=dtype, device="cuda")  # every entry must be written
    wm.band_nt(q, kt, w, out=band, flags=N.FLAG_REQUIRE_TENSOR)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    H.assert_lowp_close(band, want, "band_nt %s" % (shape,))
    mask = H.out_of_sequence_mask(M, w)
    assert (band.float().cpu().numpy()[:, mask] == 0).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", SHAPES)
def test_band_n_tensor(wm, shape, dtype):
    from window_matmul import _native as N

    B, M, Nn, w = shape
    d = _inputs(shape, dtype)
    want = H.oracle.unwindow_matmul_forward(d["att"], d["v"], w)
    # out-of-sequence band slots hold NaN: they must never reach the product
    att = d["att"].copy()
    att[:, H.out_of_sequence_mask(M, w)] = np.nan
    out = torch.full((B, M, Nn), float("nan"), dtype=dtype, device="cuda")
    wm.band_n(H.to_dev(att, dtype), H.to_dev(d["v"], dtype), w, out=out, flags=N.FLAG_REQUIRE_TENSOR)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    H.assert_lowp_close(out, want, "band_n %s" % (shape,))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [s for s in SHAPES if s[3] % 8 == 0])
def test_band_t_tensor(wm, shape, dtype):
    from window_matmul import _native as N

    B, M, Nn, w = shape
    d = _inputs(shape, dtype)
    _, want = H.oracle.unwindow_matmul_backward(d["att"], d["v"], w, d["g_out"])
    att = d["att"].copy()
    att[:, H.out_of_sequence_mask(M, w)] = np.nan
    out = torch.full((B, M, Nn), float("nan"), dtype=dtype, device="cuda")
    wm.band_t(H.to_dev(att, dtype), H.to_dev(d["g_out"], dtype), w, out=out, flags=N.FLAG_REQUIRE_TENSOR)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    H.assert_lowp_close(out, want, "band_t %s" % (shape,))


@pytest.mark.parametrize("shape", [(2, 256, 64, 64), (1, 384, 64, 256)])
def test_band_n_and_band_t_tensor_on_a_sequence_shard(wm, shape):
    from window_matmul import _native as N

    B, M, Nn, w = shape
    dtype = torch.bfloat16
    d = _inputs(shape, dtype)
    want_o = H.oracle.unwindow_matmul_forward(d["att"], d["v"], w)
    _, want_gv = H.oracle.unwindow_matmul_backward(d["att"], d["v"], w, d["g_out"])
    parts = 2
    Ml = M // parts
    gv = np.zeros((B, M + 2 * w, Nn))
    for r in range(parts):
        m0 = r * Ml
        seq = (max(0, w - m0), min(Ml + 2 * w, M - m0 + w))
        v_ext = np.pad(d["v"], ((0, 0), (w, w), (0, 0)))[:, m0:m0 + Ml + 2 * w].copy()
        v_ext[:, :seq[0]] = np.nan
        v_ext[:, seq[1]:] = np.nan
        att = H.to_dev(d["att"][:, m0:m0 + Ml], dtype)
        o = wm.band_n(att, H.to_dev(v_ext, dtype), w, other_off=w, seq=seq, flags=N.FLAG_REQUIRE_TENSOR)
        H.assert_lowp_close(o, want_o[:, m0:m0 + Ml], "o shard %d" % r)
        part = wm.band_t(att, H.to_dev(d["g_out"][:, m0:m0 + Ml], dtype), w, other_rows=Ml + 2 * w, other_off=w, seq=seq,
                         flags=N.FLAG_REQUIRE_TENSOR)
        assert (part[:, :seq[0]] == 0).all() and (part[:, seq[1]:] == 0).all()
        gv[:, m0:m0 + Ml + 2 * w] += part.double().cpu().numpy()
    H.assert_lowp_close(torch.from_numpy(gv[:, w:w + M]), want_gv, "gv summed over shards")


@pytest.mark.parametrize("shape", [(2, 256, 64, 64), (1, 384, 64, 256)])
def test_band_nt_tensor_on_a_sequence_shard(wm, shape):
    from window_matmul import _native as N

    B, M, Nn, w = shape
    dtype = torch.bfloat16
    d = _inputs(shape, dtype)
    want = H.oracle.window_matmul_forward(d["q"], np.ascontiguousarray(d["kt"].transpose(0, 2, 1)), w)
    parts = 2
    Ml = M // parts
    for r in range(parts):
        m0 = r * Ml
        kt_ext = np.pad(d["kt"], ((0, 0), (w, w), (0, 0)))[:, m0:m0 + Ml + 2 * w]
        # poison the halo rows that lie outside the global sequence: they must be masked, not multiplied
        seq = (max(0, w - m0), min(Ml + 2 * w, M - m0 + w))
        kt_ext = kt_ext.copy()
        kt_ext[:, :seq[0]] = 77.0
        kt_ext[:, seq[1]:] = 77.0
        a = wm.band_nt(H.to_dev(d["q"][:, m0:m0 + Ml], dtype), H.to_dev(kt_ext, dtype), w, other_off=w, seq=seq,
                       flags=N.FLAG_REQUIRE_TENSOR)
        H.assert_lowp_close(a, want[:, m0:m0 + Ml], "shard %d" % r)


@pytest.mark.parametrize("shape", [s for s in SHAPES if s[3] % 8 == 0])
def test_window_backward_fused_tensor(wm, shape):
    """grad_Q and grad_K from one launch over grad_A (both passes share the band tiles through L2)."""
    from window_matmul import _native as N

    B, M, Nn, w = shape
    dtype = torch.bfloat16
    d = _inputs(shape, dtype)
    want_gq, want_gk = H.oracle.window_matmul_backward(d["q"], np.ascontiguousarray(d["kt"].transpose(0, 2, 1)), w, d["g_band"])
    q, kt, g_band = (H.to_dev(d[x], dtype) for x in ("q", "kt", "g_band"))
    old = wm.set_flags(N.FLAG_REQUIRE_TENSOR)
    try:
        before = N.launch_count()
        gq, gk = wm.window_matmul_backward(q, kt.transpose(-1, -2), w, g_band)
        assert N.launch_count() - before == (1 if w > 32 else 2)  # one fused launch in the tcgen05 family
    finally:
        wm.set_flags(old)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    H.assert_lowp_close(gq, want_gq, "grad_q %s" % (shape,))
    H.assert_lowp_close(gk, want_gk, "grad_k %s" % (shape,))


# windows of 128 and 256 with N <= 64 take the one-sweep backward kernel: runs of row tiles that start inside a sequence
# (more row tiles than SMs), sequences shorter than the window, ragged last tiles, one and many sequences per CTA
SWEEP_SHAPES = [(20, 2048, 64, 256), (3, 2048, 64, 256), (2, 1000, 64, 128), (5, 384, 32, 128), (1, 128, 64, 256),
                (2, 256, 64, 256), (7, 640, 64, 256), (160, 128, 32, 128), (40, 520, 64, 128)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", SWEEP_SHAPES)
def test_window_backward_one_sweep(wm, shape, dtype):
    """grad_Q and grad_K from the kernel that brings each box of grad_A into shared memory once.  The out-of-sequence
    slots of grad_A hold NaN: the reference never reads them, so they must not reach either result."""
    from window_matmul import _native as N

    B, M, Nn, w = shape
    d = _inputs(shape, dtype, seed=17)
    want_gq, want_gk = H.oracle.window_matmul_backward(d["q"], np.ascontiguousarray(d["kt"].transpose(0, 2, 1)), w, d["g_band"])
    g_band = d["g_band"].copy()
    g_band[:, H.out_of_sequence_mask(M, w)] = np.nan
    q, kt, gb = H.to_dev(d["q"], dtype), H.to_dev(d["kt"], dtype), H.to_dev(g_band, dtype)
    gq = torch.full((B, M, Nn), float("nan"), dtype=dtype, device="cuda")
    gkt = torch.full((B, M, Nn), float("nan"), dtype=dtype, device="cuda")
    old = wm.set_flags(N.FLAG_REQUIRE_TENSOR | N.FLAG_PREFER_SWEEP)
    try:
        before = N.launch_count()
        wm.window_matmul_backward(q, kt.transpose(-1, -2), w, gb, out=(gq, gkt))
        assert N.launch_count() - before == 1
    finally:
        wm.set_flags(old)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    H.assert_lowp_close(gq, want_gq, "grad_q %s" % (shape,))
    H.assert_lowp_close(gkt, want_gk.transpose(0, 2, 1), "grad_k %s" % (shape,))
    # the library's own choice for the same problem (the two-pass kernel below 8 row tiles per SM) agrees
    gq2, gk2 = wm.window_matmul_backward(q, kt.transpose(-1, -2), w, gb)
    torch.cuda.synchronize()
    H.assert_lowp_close(gq2, want_gq, "grad_q, default choice %s" % (shape,))
    H.assert_lowp_close(gk2.transpose(-1, -2), want_gk.transpose(0, 2, 1), "grad_k, default choice %s" % (shape,))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SMALL_SHAPES)
def test_small_window_family(wm, shape, dtype):
    from window_matmul import _native as N

    B, M, Nn, w = shape
    d = _inputs(shape, dtype, seed=13)
    want = H.oracle_all(d, w)
    q, kt, v, g_out, g_band = (H.to_dev(d[x], dtype) for x in ("q", "kt", "v", "g_out", "g_band"))
    att = d["att"].copy()
    att[:, H.out_of_sequence_mask(M, w)] = np.nan  # never read
    att = H.to_dev(att, dtype)
    geo = N.geometry(B, M, Nn, w)
    assert N.lib.wmm_query_path(N.BAND_NT, N.operand(q), N.operand(kt), 256, geo, N.dtype_code(q), 0) == 2
    F = N.FLAG_REQUIRE_TENSOR
    a = torch.full((B, M, 2 * w + 1), float("nan"), dtype=dtype, device="cuda")
    wm.band_nt(q, kt, w, out=a, flags=F)
    o = wm.band_n(att, v, w, flags=F)
    gv = wm.band_t(att, g_out, w, flags=F)
    gq = wm.band_n(g_band, kt, w, flags=F)
    gk = wm.band_t(g_band, q, w, flags=F)
    gatt = wm.band_nt(g_out, v, w, flags=F)
    torch.cuda.synchronize()
    H.assert_lowp_close(a, want["a"], "a")
    assert (a.float().cpu().numpy()[:, H.out_of_sequence_mask(M, w)] == 0).all()
    H.assert_lowp_close(o, want["o"], "o")
    H.assert_lowp_close(gv, want["gv"], "gv")
    H.assert_lowp_close(gq, want["gq"], "gq")
    H.assert_lowp_close(gk, want["gk"].transpose(0, 2, 1), "gk")
    H.assert_lowp_close(gatt, want["gatt"], "gatt")


def test_small_window_family_on_a_sequence_shard(wm):
    from window_matmul import _native as N

    B, M, Nn, w = 2, 192, 32, 8
    dtype = torch.float16
    d = _inputs((B, M, Nn, w), dtype, seed=17)
    want = H.oracle_all(d, w)
    parts, F = 3, N.FLAG_REQUIRE_TENSOR
    Ml = M // parts
    gv = np.zeros((B, M + 2 * w, Nn))
    for r in range(parts):
        m0 = r * Ml
        seq = (max(0, w - m0), min(Ml + 2 * w, M - m0 + w))
        pad = lambda x: np.pad(x, ((0, 0), (w, w), (0, 0)), constant_values=55.0)[:, m0:m0 + Ml + 2 * w]  # noqa: E731
        att = H.to_dev(d["att"][:, m0:m0 + Ml], dtype)
        a = wm.band_nt(H.to_dev(d["q"][:, m0:m0 + Ml], dtype), H.to_dev(pad(d["kt"]), dtype), w, other_off=w, seq=seq, flags=F)
        H.assert_lowp_close(a, want["a"][:, m0:m0 + Ml], "a shard %d" % r)
        o = wm.band_n(att, H.to_dev(pad(d["v"]), dtype), w, other_off=w, seq=seq, flags=F)
        H.assert_lowp_close(o, want["o"][:, m0:m0 + Ml], "o shard %d" % r)
        part = wm.band_t(att, H.to_dev(d["g_out"][:, m0:m0 + Ml], dtype), w, other_rows=Ml + 2 * w, other_off=w, seq=seq, flags=F)
        assert (part[:, :seq[0]] == 0).all() and (part[:, seq[1]:] == 0).all()
        gv[:, m0:m0 + Ml + 2 * w] += part.double().cpu().numpy()
    H.assert_lowp_close(torch.from_numpy(gv[:, w:w + M]), want["gv"], "gv summed over shards")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [s for s in SHAPES if s[3] % 8 == 0 and s[3] > 32])
def test_k_as_contiguous_bnm_tensor_takes_the_tensor_path(wm, shape, dtype):
    """K given as a contiguous (B, N, M) tensor (as in the reference's README example): consumed in place by the
    tcgen05 kernels (position-major operand), forward and both gradients, no transposing copy."""
    from window_matmul import _native as N

    B, M, Nn, w = shape
    d = _inputs(shape, dtype)
    k_np = np.ascontiguousarray(d["kt"].transpose(0, 2, 1))
    want_a = H.oracle.window_matmul_forward(d["q"], k_np, w)
    want_gq, want_gk = H.oracle.window_matmul_backward(d["q"], k_np, w, d["g_band"])
    q, g_band = H.to_dev(d["q"], dtype), H.to_dev(d["g_band"], dtype)
    k = H.to_dev(k_np, dtype)
    assert k.is_contiguous() and k.shape == (B, Nn, M)
    old = wm.set_flags(N.FLAG_REQUIRE_TENSOR)
    try:
        a = wm.window_matmul_forward(q, k, w)
        before = N.launch_count()
        gq, gk = wm.window_matmul_backward(q, k, w, g_band)
        assert N.launch_count() - before == 1
        gq_only, _ = wm.window_matmul_backward(q, k, w, g_band, need=(True, False))
    finally:
        wm.set_flags(old)
    torch.cuda.synchronize()
    assert N.device_status() == 0 and gk.shape == (B, Nn, M)
    H.assert_lowp_close(a, want_a, "a")
    H.assert_lowp_close(gq, want_gq, "grad_q")
    H.assert_lowp_close(gq_only, want_gq, "grad_q (band_n alone)")
    H.assert_lowp_close(gk, want_gk, "grad_k")


def test_ineligible_problems_are_reported_not_faked(wm):
    from window_matmul import _native as N

    q = torch.randn(2, 64, 24, device="cuda", dtype=torch.bfloat16)  # hidden size 24: no tensor kernel
    with pytest.raises(RuntimeError, match="UNSUPPORTED"):
        wm.band_nt(q, q, 8, flags=N.FLAG_REQUIRE_TENSOR)
    q = torch.randn(2, 64, 64, device="cuda", dtype=torch.float32)  # fp32 stays on the exact-order kernels
    with pytest.raises(RuntimeError, match="UNSUPPORTED"):
        wm.band_nt(q, q, 8, flags=N.FLAG_REQUIRE_TENSOR)


def test_tensor_kernels_from_a_fresh_thread(wm):
    """A thread that has made no CUDA call yet (an autograd worker, a thread pool) has no current context;
    the launcher must bind one before it builds its tensor maps."""
    import threading

    from window_matmul import _native as N

    q = torch.randn(2, 256, 64, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    result = {}

    def work():
        try:
            result["a"] = wm.band_nt(q, q, 64, flags=N.FLAG_REQUIRE_TENSOR)
            result["o"] = wm.band_n(result["a"], q, 64, flags=N.FLAG_REQUIRE_TENSOR)
        except Exception as e:  # noqa: BLE001
            result["error"] = e

    t = threading.Thread(target=work)
    t.start()
    t.join()
    torch.cuda.synchronize()
    assert "error" not in result, result.get("error")
    assert torch.equal(result["a"], wm.band_nt(q, q, 64, flags=N.FLAG_REQUIRE_TENSOR))


# ---- fp32 operands on the tensor cores (WMM_FLAG_TF32) -------------------------------------------------------------
TF32_REL = 2e-3
TF32_SHAPES = [(2, 512, 64, 64), (1, 1024, 64, 256), (2, 200, 64, 64), (3, 136, 64, 4), (1, 640, 64, 12), (4, 256, 32, 8),
               (1, 768, 64, 384), (2, 8, 64, 4), (2, 384, 32, 128), (1, 1152, 64, 100)]


def _assert_tf32_close(got, want, what):
    """2e-3 relative in the norm the target names (largest error against the largest reference value, reported), and
    element by element |err| <= 3e-3 (|x| + rms): the tensor core drops the low 13 mantissa bits of each fp32 operand
    (it truncates, it does not round), so every product is low by up to 2e-3 of itself."""
    g = got.detach().double().cpu().numpy()
    w_ = want.astype(np.float64)
    worst = np.abs(g - w_).max() / max(np.abs(w_).max(), 1e-30)
    assert worst <= TF32_REL, "%s: max abs err / max abs ref = %.3e" % (what, worst)
    H.assert_lowp_close(got, want, what, rel=1.5 * TF32_REL)


@pytest.mark.parametrize("shape", TF32_SHAPES)
def test_band_nt_tf32(wm, shape):
    """fp32 inputs multiplied as tf32 (10-bit mantissas, fp32 sums) against the fp32 oracle on the same inputs: within
    2e-3 relative, exact zeros outside the sequence, every entry written, and the tensor-core kernel really taken."""
    from window_matmul import _native as N

    B, M, Nn, w = shape
    d = H.rand_inputs(B, M, Nn, w, seed=7, scale=1.0 / np.sqrt(Nn))
    want = H.oracle.window_matmul_forward(d["q"], np.ascontiguousarray(d["kt"].transpose(0, 2, 1)), w)
    q, kt = H.to_dev(d["q"], torch.float32), H.to_dev(d["kt"], torch.float32)
    band = torch.full((B, M, 2 * w + 1), float("nan"), dtype=torch.float32, device="cuda")
    flags = N.FLAG_TF32 | N.FLAG_REQUIRE_TENSOR
    assert N.lib.wmm_query_path(N.BAND_NT, N.operand(q), N.operand(kt), band.data_ptr(), N.geometry(B, M, Nn, w), N.F32, flags) == 1
    assert N.lib.wmm_query_path(N.BAND_NT, N.operand(q), N.operand(kt), band.data_ptr(), N.geometry(B, M, Nn, w), N.F32, 0) == 0
    wm.band_nt(q, kt, w, out=band, flags=flags)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    _assert_tf32_close(band, want, "band_nt tf32 %s" % (shape,))
    mask = H.out_of_sequence_mask(M, w)
    assert (band.cpu().numpy()[:, mask] == 0).all()
    # without the flag fp32 stays on the exact-order kernels (rtol 1e-5)
    exact = wm.band_nt(q, kt, w)
    H.assert_lowp_close(exact, want, "band_nt exact", rel=2e-5)


@pytest.mark.parametrize("shape", TF32_SHAPES)
def test_band_n_and_band_t_tf32(wm, shape):
    """The other two contractions on fp32 tensors with WMM_FLAG_TF32, NaN in the out-of-sequence band slots (they must
    never reach a product), against the fp32 oracle; then the two backward entry points, which take the same kernels."""
    from window_matmul import _native as N

    B, M, Nn, w = shape
    d = H.rand_inputs(B, M, Nn, w, seed=8, scale=1.0 / np.sqrt(Nn))
    mask = H.out_of_sequence_mask(M, w)
    flags = N.FLAG_TF32 | N.FLAG_REQUIRE_TENSOR
    att = d["att"].copy()
    att[:, mask] = np.nan
    att_d, v_d, go_d = H.to_dev(att, torch.float32), H.to_dev(d["v"], torch.float32), H.to_dev(d["g_out"], torch.float32)
    want_o = H.oracle.unwindow_matmul_forward(d["att"], d["v"], w)
    want_ga, want_gv = H.oracle.unwindow_matmul_backward(d["att"], d["v"], w, d["g_out"])
    o = torch.full((B, M, Nn), float("nan"), device="cuda")
    wm.band_n(att_d, v_d, w, out=o, flags=flags)
    gv = torch.full((B, M, Nn), float("nan"), device="cuda")
    wm.band_t(att_d, go_d, w, out=gv, flags=flags)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    _assert_tf32_close(o, want_o, "band_n tf32 %s" % (shape,))
    _assert_tf32_close(gv, want_gv, "band_t tf32 %s" % (shape,))
    # the reference-shaped backward calls under the process-wide flag
    old = wm.set_flags(N.FLAG_TF32)
    try:
        q_d, k_d = H.to_dev(d["q"], torch.float32), H.to_dev(np.ascontiguousarray(d["kt"]), torch.float32).transpose(-1, -2)
        gb = d["g_band"].copy()
        gb[:, mask] = 0
        gq, gk = wm.window_matmul_backward(q_d, k_d, w, H.to_dev(gb, torch.float32))
        ga, gv2 = wm.unwindow_matmul_backward(att_d, v_d, w, go_d)
    finally:
        wm.set_flags(old)
    torch.cuda.synchronize()
    want_gq, want_gk = H.oracle.window_matmul_backward(d["q"], np.ascontiguousarray(d["kt"].transpose(0, 2, 1)), w, gb)
    _assert_tf32_close(gq, want_gq, "grad_q tf32")
    _assert_tf32_close(gk, want_gk, "grad_k tf32")
    _assert_tf32_close(ga, want_ga, "grad_a tf32")
    _assert_tf32_close(gv2, want_gv, "grad_v tf32")
    assert (ga.cpu().numpy()[:, mask] == 0).all()
    assert N.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_row_ranges_of_a_band_tensor_in_place(wm, dtype):
    """The tensor-core kernels address a range of rows of a longer band tensor where it lies (a batch stride larger than
    the range): what a sequence shard does when it computes its interior rows before the halo has arrived and the edge
    strips after.  band_nt writes only the range; band_n and band_t read only the range."""
    from window_matmul import _native as N

    B, M, Nn, w = 3, 1024, 64, 128
    flags = N.FLAG_REQUIRE_TENSOR | (N.FLAG_TF32 if dtype == torch.float32 else 0)
    d = _inputs((B, M, Nn, w), dtype if dtype != torch.float32 else torch.float32)
    q, kt, v, go = (H.to_dev(d[k], dtype) for k in ("q", "kt", "v", "g_out"))
    full = wm.band_nt(q, kt, w, flags=flags)
    band = torch.full((B, M, 2 * w + 1), float("nan"), dtype=dtype, device="cuda")
    for r0, r1 in ((w, M - w), (0, w), (M - w, M)):          # interior first, then the two edge strips
        wm.band_nt(q[:, r0:r1], kt, w, other_off=r0, out=band[:, r0:r1], flags=flags)
        torch.cuda.synchronize()
        assert torch.equal(band[:, r0:r1], full[:, r0:r1])
        if r0 == w:
            assert torch.isnan(band[:, :w]).all() and torch.isnan(band[:, M - w:]).all()   # nothing outside the range was touched
    assert torch.equal(band, full)
    o_full = wm.band_n(full, v, w, flags=flags)
    gv_full = wm.band_t(full, go, w, flags=flags)
    r0, r1 = 256, 640
    o = wm.band_n(full[:, r0:r1], v, w, other_off=r0, flags=flags)
    assert torch.equal(o, o_full[:, r0:r1])
    part = wm.band_t(full[:, r0:r1], go[:, r0:r1], w, other_rows=M, other_off=r0, flags=flags)
    rest = full.clone()
    rest[:, r0:r1] = 0
    other = wm.band_t(rest, go, w, flags=flags)
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    H.assert_lowp_close(part.float() + other.float(), gv_full.float().cpu().numpy(), "band_t over a row range", rel=tol)
    assert N.device_status() == 0
    # the other kernel families refuse a strided band instead of misreading it
    with pytest.raises(RuntimeError, match="tensor-core kernels only"):
        wm.band_nt(q[:, :64].float(), kt.float(), w, out=torch.empty(B, M, 2 * w + 1, device="cuda")[:, :64], flags=N.FLAG_FORCE_GENERIC)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_results_do_not_depend_on_a_cta_limit(wm, dtype):
    """wmm_set_cta_limits gives the persistent kernels a smaller grid (SMs left to an exchange on another stream); the
    tiles are the same and so is every output bit, window backward in one launch included."""
    from window_matmul import _native as N

    B, M, Nn, w = 6, 2048, 64, 128            # 96 row tiles: more than one per CTA at 37 CTAs
    flags = N.FLAG_REQUIRE_TENSOR | (N.FLAG_TF32 if dtype == torch.float32 else 0)
    d = _inputs((B, M, Nn, w), torch.float32)
    q, kt, v, go = (H.to_dev(d[k], dtype) for k in ("q", "kt", "v", "g_out"))

    def run():
        band = wm.band_nt(q, kt, w, flags=flags)
        out = [band, wm.band_n(band, v, w, flags=flags), wm.band_t(band, go, w, flags=flags)]
        if dtype == torch.bfloat16:          # both halves of the window backward in one launch
            out += list(wm.window_matmul_backward(q, kt.transpose(-1, -2), w, band))
        torch.cuda.synchronize()
        return out

    free = run()
    with N.cta_limits(37, 0):
        capped = run()
    again = run()
    for a, b, c in zip(free, capped, again):
        assert torch.equal(a, b) and torch.equal(a, c)
    assert N.device_status() == 0
