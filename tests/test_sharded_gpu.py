"""Sequence-sharded operators on real GPUs over NCCL (needs >= 2 GPUs; skipped otherwise).

Child processes, one per GPU; ranks only ever leave between steps.  NVLS is switched off and the kernels use
no peer memory: the exchange is NCCL send/recv between neighbours."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, shape, dtype_name, out_dir):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path[:0] = [ROOT, os.path.join(ROOT, "pytorch-window-matmul_b200")]
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from window_matmul import _native, sharded

        dtype = getattr(torch, dtype_name)
        B, M, N, w = shape
        g = torch.Generator().manual_seed(5)
        q, k, v = (torch.randn(B, M, N, generator=g) / N ** 0.5 for _ in range(3))
        go = torch.randn(B, M, N, generator=g)
        Ml = M // world
        sl = slice(rank * Ml, (rank + 1) * Ml)
        ql, kl, vl = (t[:, sl].to(dtype).to(dev).requires_grad_(True) for t in (q, k, v))
        a = sharded.seq_parallel_window_matmul(ql, kl.transpose(-1, -2), w)
        a.retain_grad()
        o = sharded.seq_parallel_unwindow_matmul(a, vl, w)
        o.backward(go[:, sl].to(dtype).to(dev))
        # the attention block with the band softmax between the sharded operators
        q2, k2, v2 = (t[:, sl].to(dtype).to(dev).requires_grad_(True) for t in (q, k, v))
        pr = sharded.seq_parallel_window_softmax(sharded.seq_parallel_window_matmul(q2, k2.transpose(-1, -2), w), 0.5, True)
        ob = sharded.seq_parallel_unwindow_matmul(pr, v2, w)
        ob.backward(go[:, sl].to(dtype).to(dev))
        torch.cuda.synchronize()
        assert _native.device_status() == 0
        np.savez(os.path.join(out_dir, "rank%d.npz" % rank), **{
            key: t.detach().float().cpu().numpy()
            for key, t in dict(a=a, o=o, gq=ql.grad, gk=kl.grad, gv=vl.grad, ga=a.grad, ob=ob, bq=q2.grad, bk=k2.grad,
                               bv=v2.grad).items()})
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dtype_name,shape", [("float32", (2, 256, 16, 24)), ("bfloat16", (2, 1024, 64, 64)),
                                              ("bfloat16", (1, 2048, 128, 256))])
def test_sequence_sharded_on_gpus(tmp_path, dtype_name, shape):
    import torch.multiprocessing as mp

    import helpers as H

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    mp.spawn(_worker, args=(world, _free_port(), shape, dtype_name, str(tmp_path)), nprocs=world, join=True)
    B, M, N, w = shape
    dtype = getattr(torch, dtype_name)
    g = torch.Generator().manual_seed(5)
    q, k, v = (H.round_to((torch.randn(B, M, N, generator=g) / N ** 0.5).numpy(), dtype) for _ in range(3))
    go = H.round_to(torch.randn(B, M, N, generator=g).numpy(), dtype)
    a, o, gq, gk, ga, gv = H.oracle.chain_fwd_bwd(q, np.ascontiguousarray(k.transpose(0, 2, 1)), v, w, go)
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    cat = lambda key: torch.from_numpy(np.concatenate([p[key] for p in parts], axis=1))  # noqa: E731
    rel = 2e-5 if dtype == torch.float32 else 4e-2  # bf16: the band itself is rounded before it is reused
    for key, want in dict(a=a, o=o, ga=ga, gq=gq, gk=gk.transpose(0, 2, 1), gv=gv).items():
        H.assert_lowp_close(cat(key), want, key, rel=rel if key != "a" else min(rel, 1e-2))
    # attention block (scores * 0.5, masked softmax, values) against the dense float64 formulation
    qt, kt_, vt = (torch.from_numpy(x).double().requires_grad_(True) for x in (q, k, v))
    i = torch.arange(M)
    inside = (i[:, None] - i[None, :]).abs() <= w
    dense = torch.softmax((qt @ kt_.transpose(-1, -2) * 0.5).masked_fill(~inside, float("-inf")), -1) @ vt
    dense.backward(torch.from_numpy(go).double())
    rel_b = 1e-4 if dtype == torch.float32 else 6e-2
    for key, want in dict(ob=dense.detach(), bq=qt.grad, bk=kt_.grad, bv=vt.grad).items():
        H.assert_lowp_close(cat(key), want.numpy(), key, rel=rel_b)


def _peer_worker(rank, world, port, shape, dtype_name, out_dir):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path[:0] = [ROOT, os.path.join(ROOT, "pytorch-window-matmul_b200")]
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from window_matmul import _native
        from window_matmul.peer_halo import PeerHalo

        dtype = getattr(torch, dtype_name)
        B, M, N, w = shape
        Ml = M // world
        g = torch.Generator().manual_seed(11)
        xs = [torch.randn(B, M, N, generator=g).to(dtype) for _ in range(2)]                  # the global operands
        ps = [[torch.randn(B, Ml + 2 * w, N, generator=g).to(dtype) for _ in range(2)] for _ in range(world)]  # partials of every rank
        halo = PeerHalo(2, B, Ml, N, w, dtype, dev)
        for i in range(2):
            halo.local(i).copy_(xs[i][:, rank * Ml:(rank + 1) * Ml])
        # three exchanges; the owners rescale their rows in between, so stale reads would show
        for it in range(3):
            exts = halo.exchange()
            torch.cuda.synchronize()
            for i in range(2):
                padded = torch.nn.functional.pad(xs[i].float() * (2.0 ** it), (0, 0, w, w))
                want = padded[:, rank * Ml:rank * Ml + Ml + 2 * w].to(dtype)
                assert torch.equal(exts[i].cpu(), want), "exchange %d, tensor %d on rank %d" % (it, i, rank)
            for i in range(2):
                halo.local(i).mul_(2.0)
        # reverse halo: own rows += what the neighbours computed for them
        for i in range(2):
            halo.partial(i).copy_(ps[rank][i])
        own = halo.reduce()
        torch.cuda.synchronize()
        for i in range(2):
            want = ps[rank][i][:, w:w + Ml].float().clone()
            if rank > 0:
                want[:, :w] = (want[:, :w].to(dtype).float() + ps[rank - 1][i][:, w + Ml:].float())
            want = want.to(dtype).float()
            if rank < world - 1:
                want[:, Ml - w:] = (want[:, Ml - w:] + ps[rank + 1][i][:, :w].float())
            assert torch.equal(own[i].cpu(), want.to(dtype)), "reduce, tensor %d on rank %d" % (i, rank)
        # the same exchange replayed from a CUDA graph (the hand-shake counts epochs on the device)
        s = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(s):
            halo.exchange()
            s.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                halo.exchange()
            for _ in range(4):
                graph.replay()
            s.synchronize()
        for i in range(2):
            padded = torch.nn.functional.pad(xs[i].float() * 8.0, (0, 0, w, w))
            assert torch.equal(halo.ext(i).cpu(), padded[:, rank * Ml:rank * Ml + Ml + 2 * w].to(dtype))
        assert _native.device_status() == 0
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dtype_name,shape", [("bfloat16", (3, 512, 64, 64)), ("float32", (2, 384, 16, 24))])
def test_peer_memory_halo_exchange(tmp_path, dtype_name, shape):
    """wmm_halo_pull: margins from the neighbours' edge rows, reverse accumulation, repeated epochs, graph replay."""
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    mp.spawn(_peer_worker, args=(world, _free_port(), shape, dtype_name, str(tmp_path)), nprocs=world, join=True)


def test_halo_pull_wait_runs_out_without_hanging():
    """Failure detection of the exchange kernel on ONE GPU: the flag block of a 'neighbour' that never runs is plain local
    memory that nothing sets.  The kernel's bounded waits (about a second for the neighbour to start, about three for its
    acknowledgement) run out, it returns, the status word has bit 5 set, the margins are untouched and the context stays
    usable."""
    import ctypes as C

    sys.path[:0] = [ROOT, os.path.join(ROOT, "pytorch-window-matmul_b200")]
    from window_matmul import _native as N

    dev = torch.device("cuda", 0)
    B, Ml, Nn, w = 2, 64, 8, 16
    mine = torch.full((B, Ml + 2 * w, Nn), 1.0, dtype=torch.bfloat16, device=dev)
    absent = torch.full((B, Ml + 2 * w, Nn), 7.0, dtype=torch.bfloat16, device=dev)   # stands in for the lower neighbour's buffer
    my_flags = torch.zeros(4, dtype=torch.int32, device=dev)
    absent_flags = torch.zeros(4, dtype=torch.int32, device=dev)                       # its ready word stays 0
    counters = torch.zeros(4, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    bufs = (N.HaloBuffer * 1)(N.HaloBuffer(mine.data_ptr(), absent.data_ptr(), None))
    flags = N.HaloFlags(my_flags.data_ptr(), absent_flags.data_ptr(), None, counters.data_ptr())
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    N.check(N.lib.wmm_halo_pull(bufs, 1, C.byref(flags), B, Ml, Nn, w, N.BF16, 0, stream))
    torch.cuda.synchronize()
    assert N.device_status() & 32, "the kernel must report the wait that ran out"
    assert N.device_status() == 0                       # reading cleared it
    assert (mine == 1.0).all()                          # nothing was copied from a neighbour that was not ready
    assert int(my_flags[0]) == 1 and int(counters[0]) == 1 and int(counters[1]) == 0   # epoch advanced, CTA counter reset
    assert int(absent_flags[2]) == 1                    # the acknowledgement went out although the copy was given up
    assert float((mine.float() + 1).sum()) > 0          # the context still works


def test_halo_pull_serves_the_live_side_when_the_other_neighbour_is_absent():
    """ONE GPU, two stand-in neighbours in local memory: the lower one never runs (its flag block stays zero), the upper
    one looks as if it had started and finished (its ready word and its acknowledgement are written by the host before the
    launch).  The kernel reports the lower side (bit 5), leaves the lower margin alone and still fills the upper margin
    from the upper neighbour's first rows."""
    import ctypes as C

    sys.path[:0] = [ROOT, os.path.join(ROOT, "pytorch-window-matmul_b200")]
    from window_matmul import _native as N

    dev = torch.device("cuda", 0)
    B, Ml, Nn, w = 3, 96, 64, 32      # several CTAs
    ext = Ml + 2 * w
    mine = torch.full((B, ext, Nn), 1.0, dtype=torch.bfloat16, device=dev)
    lower = torch.full((B, ext, Nn), 7.0, dtype=torch.bfloat16, device=dev)
    upper = torch.arange(B * ext * Nn, device=dev).remainder(251).to(torch.bfloat16).reshape(B, ext, Nn)
    my_flags = torch.tensor([0, 0, 1, 0], dtype=torch.int32, device=dev)      # word 2: the upper neighbour's ack for epoch 1
    lower_flags = torch.zeros(4, dtype=torch.int32, device=dev)
    upper_flags = torch.tensor([1, 0, 0, 0], dtype=torch.int32, device=dev)   # ready for epoch 1
    counters = torch.zeros(4, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    assert N.device_status() == 0
    bufs = (N.HaloBuffer * 1)(N.HaloBuffer(mine.data_ptr(), lower.data_ptr(), upper.data_ptr()))
    flags = N.HaloFlags(my_flags.data_ptr(), lower_flags.data_ptr(), upper_flags.data_ptr(), counters.data_ptr())
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    N.check(N.lib.wmm_halo_pull(bufs, 1, C.byref(flags), B, Ml, Nn, w, N.BF16, 0, stream))
    torch.cuda.synchronize()
    assert N.device_status() == 32
    assert (mine[:, :w + Ml] == 1.0).all()                        # lower margin and own rows untouched
    assert torch.equal(mine[:, w + Ml:], upper[:, w:2 * w])       # upper margin <- the upper neighbour's first own rows
    assert int(upper_flags[1]) == 1 and int(lower_flags[2]) == 1  # both acknowledgements went out
    assert int(counters[0]) == 1 and int(counters[1]) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("accumulate", [0, 1])
def test_exchange_under_a_cta_limit_moves_the_same_bytes(accumulate):
    """wmm_set_cta_limits picks another grid and another unrolling of the exchange kernel, nothing else.  ONE GPU, the rank
    as its own two neighbours (an exchange then wraps the sequence around)."""
    import ctypes as C

    sys.path[:0] = [ROOT, os.path.join(ROOT, "pytorch-window-matmul_b200")]
    from window_matmul import _native as N

    dev = torch.device("cuda", 0)
    B, Ml, Nn, w = 5, 640, 128, 96          # 5 x 96 x 128 x 2 B per side: more than one sweep of a capped grid
    ext = Ml + 2 * w
    start = torch.randn(B, ext, Nn, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    results = []
    for limit in (0, 3):
        buf = start.to(dev).clone()
        fl = torch.zeros(4, dtype=torch.int32, device=dev)
        counters = torch.zeros(4, dtype=torch.int32, device=dev)
        arr = (N.HaloBuffer * 1)(N.HaloBuffer(buf.data_ptr(), buf.data_ptr(), buf.data_ptr()))
        flags = N.HaloFlags(fl.data_ptr(), fl.data_ptr(), fl.data_ptr(), counters.data_ptr())
        with N.cta_limits(0, limit):
            N.check(N.lib.wmm_halo_pull(arr, 1, C.byref(flags), B, Ml, Nn, w, N.BF16, accumulate, stream))
        torch.cuda.synchronize()
        assert N.device_status() == 0 and int(fl[0]) == 1
        results.append(buf.clone())
    assert torch.equal(results[0], results[1])
    assert not torch.equal(results[0].cpu(), start)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,Nn", [(torch.bfloat16, 64), (torch.float16, 128)])
def test_edge_rows_of_band_t_and_their_reduction(dtype, Nn):
    """wmm_band_t_edges writes output rows near both ends once more as unrounded fp32 (here, as a sequence shard does, the
    first and last w OWN rows: edge_rows = 2w, edge_skip = w); wmm_halo_reduce_edges adds the neighbours' 16-bit margin rows
    to those and rounds once.  ONE GPU: the rank is its own two neighbours, so its first w own rows receive its own upper
    margin and its last w own rows its own lower margin."""
    import ctypes as C
    import importlib

    sys.path[:0] = [ROOT, os.path.join(ROOT, "pytorch-window-matmul_b200")]
    from window_matmul import _native as N

    impl = importlib.import_module("window_matmul.window_matmul")
    dev = torch.device("cuda", 0)
    B, Ml, w = 3, 768, 128
    ext = Ml + 2 * w
    g = torch.Generator().manual_seed(5)
    band = (torch.randn(B, Ml, 2 * w + 1, generator=g) / 4).to(dtype).to(dev)
    x = torch.randn(B, Ml, Nn, generator=g).to(dtype).to(dev)
    flags = N.FLAG_REQUIRE_TENSOR
    plain = impl.band_t(band, x, w, other_rows=ext, other_off=w, flags=flags)
    edges = torch.full((B, 4 * w, Nn), float("nan"), dtype=torch.float32, device=dev)
    out = impl.band_t(band, x, w, other_rows=ext, other_off=w, flags=flags, edges=edges, edge_skip=w)
    torch.cuda.synchronize()
    assert torch.equal(out, plain)                                        # the 16-bit output does not change
    assert torch.isnan(edges[:, :w]).all() and torch.isnan(edges[:, 3 * w:]).all()   # the skipped rows are not written
    own = edges[:, w:3 * w]
    assert torch.equal(own.to(dtype), torch.cat([out[:, w:2 * w], out[:, ext - 2 * w:ext - w]], dim=1))   # the same sums ...
    assert (own != own.to(dtype).float()).float().mean() > 0.5                                            # ... not rounded
    # all 2w rows at each end with edge_skip = 0
    full = torch.empty_like(edges)
    impl.band_t(band, x, w, other_rows=ext, other_off=w, flags=flags, edges=full)
    assert torch.equal(full.to(dtype), torch.cat([out[:, :2 * w], out[:, ext - 2 * w:]], dim=1))
    assert torch.equal(full[:, w:3 * w], own)
    # reduction on a self-ring: own first w rows += own upper margin, own last w rows += own lower margin
    fl = torch.zeros(4, dtype=torch.int32, device=dev)
    counters = torch.zeros(4, dtype=torch.int32, device=dev)
    arr = (N.HaloEdges * 1)(N.HaloEdges(out.data_ptr(), edges.data_ptr(), out.data_ptr(), out.data_ptr()))
    hf = N.HaloFlags(fl.data_ptr(), fl.data_ptr(), fl.data_ptr(), counters.data_ptr())
    want = out.clone()
    want[:, w:2 * w] = (edges[:, w:2 * w] + out[:, ext - w:].float()).to(dtype)
    want[:, Ml:Ml + w] = (edges[:, 2 * w:3 * w] + out[:, :w].float()).to(dtype)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    N.check(N.lib.wmm_halo_reduce_edges(arr, 1, C.byref(hf), B, Ml, Nn, w, N.dtype_code(out), stream))
    torch.cuda.synchronize()
    assert N.device_status() == 0 and int(fl[0]) == 1
    assert torch.equal(out, want)
    # what it buys: against the sum of the unrounded terms, the 16-bit sum is further off
    exact = full[:, w:2 * w].double() + full[:, 3 * w:].double()
    with_edges = (out[:, w:2 * w].double() - exact).abs().max()
    as_16bit = ((plain[:, w:2 * w].float() + plain[:, ext - w:].float()).to(dtype).double() - exact).abs().max()
    assert with_edges <= as_16bit
    # other kernel families have no edge rows
    with pytest.raises(RuntimeError, match="edge rows"):
        impl.band_t(band.float(), x.float(), w, other_rows=ext, other_off=w, edges=edges)


def _peer_chain_worker(rank, world, port, shape, dtype_name, out_dir):
    import importlib

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path[:0] = [ROOT, os.path.join(ROOT, "pytorch-window-matmul_b200")]
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from window_matmul import _native
        from window_matmul.peer_halo import PeerHalo

        impl = importlib.import_module("window_matmul.window_matmul")
        dtype = getattr(torch, dtype_name)
        B, M, N, w = shape
        g = torch.Generator().manual_seed(5)
        q, k, v = (torch.randn(B, M, N, generator=g) / N ** 0.5 for _ in range(3))
        go = torch.randn(B, M, N, generator=g)
        Ml = M // world
        sl = slice(rank * Ml, (rank + 1) * Ml)
        ql, gol = q[:, sl].to(dtype).to(dev), go[:, sl].to(dtype).to(dev)
        halo = PeerHalo(2, B, Ml, N, w, dtype, dev)      # operand 0: K^T rows, operand 1: V rows
        halo.local(0).copy_(k[:, sl].to(dtype))
        halo.local(1).copy_(v[:, sl].to(dtype))
        ext, seq = Ml + 2 * w, halo.seq

        def step():
            kt_ext, v_ext = halo.exchange()
            a = impl.band_nt(ql, kt_ext, w, other_off=w, seq=seq)
            o = impl.band_n(a, v_ext, w, other_off=w, seq=seq)
            ga = impl.band_nt(gol, v_ext, w, other_off=w, seq=seq)
            impl.band_t(a, gol, w, other_rows=ext, other_off=w, seq=seq, out=halo.partial(1))
            gq = impl.band_n(ga, kt_ext, w, other_off=w, seq=seq)
            impl.band_t(ga, ql, w, other_rows=ext, other_off=w, seq=seq, out=halo.partial(0))
            gk, gv = halo.reduce()
            return dict(a=a, o=o, ga=ga, gq=gq, gk=gk, gv=gv)

        step()                 # twice: the second step must not see leftovers of the first in the partial buffers
        out = step()
        torch.cuda.synchronize()
        assert _native.device_status() == 0
        np.savez(os.path.join(out_dir, "rank%d.npz" % rank), **{key: t.detach().float().cpu().numpy() for key, t in out.items()})
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dtype_name,shape", [("bfloat16", (2, 1024, 64, 64)), ("bfloat16", (1, 4096, 128, 512))])
def test_sequence_sharded_chain_through_peer_memory(tmp_path, dtype_name, shape):
    """The six contractions on sequence shards with both halo exchanges done by wmm_halo_pull, against the oracle on the
    whole sequence."""
    import torch.multiprocessing as mp

    import helpers as H

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    mp.spawn(_peer_chain_worker, args=(world, _free_port(), shape, dtype_name, str(tmp_path)), nprocs=world, join=True)
    B, M, N, w = shape
    dtype = getattr(torch, dtype_name)
    g = torch.Generator().manual_seed(5)
    q, k, v = (H.round_to((torch.randn(B, M, N, generator=g) / N ** 0.5).numpy(), dtype) for _ in range(3))
    go = H.round_to(torch.randn(B, M, N, generator=g).numpy(), dtype)
    a, o, gq, gk, ga, gv = H.oracle.chain_fwd_bwd(q, np.ascontiguousarray(k.transpose(0, 2, 1)), v, w, go)
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    cat = lambda key: torch.from_numpy(np.concatenate([p[key] for p in parts], axis=1))  # noqa: E731
    for key, want in dict(a=a, o=o, ga=ga, gq=gq, gk=gk.transpose(0, 2, 1), gv=gv).items():
        H.assert_lowp_close(cat(key), want, key, rel=1e-2 if key == "a" else 4e-2)
