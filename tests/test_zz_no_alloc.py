"""wmm_halo_pull_static: the neighbour exchange for callers that cannot allocate device memory.

Who needs it: a host that gave all device memory to its own pool when it started, code that runs inside a stream capture
or a host callback (where the CUDA runtime refuses to allocate), a latency-critical loop that must stay clear of the
allocator.  wmm_halo_pull wants four scratch words of device memory from its caller; this entry point keeps them in a
static array of the library instead and is otherwise the same exchange.  The test drives both entry points through the C
ABI on the same inputs, twice in a row, and wants identical bytes.

One GPU is enough: the rank is its own lower and upper neighbour (its own buffer and flag block stand in for theirs), so
an exchange wraps the sequence around: lower margin <- own last w rows, upper margin <- own first w rows; a reduction
adds the upper margin to the first w own rows and the lower margin to the last w.

This file sorts last on purpose, so that a run that stops at the first failure has already run every other test.
"""
import ctypes as C
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "pytorch-window-matmul_b200")]


def test_lane_limit_needs_no_gpu():
    """A lane beyond the static array is refused with a clear message before anything touches a device."""
    from window_matmul import _native as N

    arr = (N.HaloBuffer * 1)(N.HaloBuffer(256, 512, 768))
    flags = N.HaloFlags(1024, 2048, 4096, None)
    for lane in (-1, 8, 1000):
        assert N.lib.wmm_halo_pull_static(arr, 1, C.byref(flags), lane, 2, 64, 8, 16, N.BF16, 0, None) == -5
        assert b"8 lanes" in N.lib.wmm_last_error_string()
    before = N.launch_count()
    assert N.lib.wmm_halo_pull_static(arr, 1, C.byref(flags), 0, 0, 64, 8, 16, N.BF16, 0, None) == 0   # empty batch: no launch
    assert N.launch_count() == before


@pytest.mark.gpu
@pytest.mark.parametrize("lane", [0, 7])
def test_static_scratch_exchange_matches_the_caller_scratch_one(lane):
    from window_matmul import _native as N

    dev = torch.device("cuda", 0)
    B, Ml, Nn, w = 3, 160, 64, 32          # several CTAs per launch
    ext = Ml + 2 * w
    g = torch.Generator().manual_seed(11)
    start = torch.randn(2, B, ext, Nn, generator=g).to(torch.bfloat16)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def ring(buf, flag_block, counters):
        """The rank as its own two neighbours."""
        arr = (N.HaloBuffer * 2)(*[N.HaloBuffer(buf[i].data_ptr(), buf[i].data_ptr(), buf[i].data_ptr()) for i in range(2)])
        fl = N.HaloFlags(flag_block.data_ptr(), flag_block.data_ptr(), flag_block.data_ptr(),
                         counters.data_ptr() if counters is not None else None)
        return arr, fl

    # the existing entry point: scratch words from the caller
    want = start.to(dev).clone()
    flags_a = torch.zeros(4, dtype=torch.int32, device=dev)
    counters = torch.zeros(4, dtype=torch.int32, device=dev)
    arr_a, fl_a = ring(want, flags_a, counters)
    # the new one: nothing but inputs, outputs and the flag block
    got = start.to(dev).clone()
    flags_b = torch.zeros(4, dtype=torch.int32, device=dev)
    arr_b, fl_b = ring(got, flags_b, None)
    torch.cuda.synchronize()
    assert N.device_status() == 0

    launches = N.launch_count()
    for step, accumulate in enumerate((0, 1, 0, 1)):       # two exchanges and two reductions, back to back
        N.check(N.lib.wmm_halo_pull(arr_a, 2, C.byref(fl_a), B, Ml, Nn, w, N.BF16, accumulate, stream))
        N.check(N.lib.wmm_halo_pull_static(arr_b, 2, C.byref(fl_b), lane, B, Ml, Nn, w, N.BF16, accumulate, stream))
        torch.cuda.synchronize()
        assert torch.equal(got, want), "step %d (accumulate=%d): the two entry points disagree" % (step, accumulate)
    assert N.launch_count() - launches == 8
    assert N.device_status() == 0
    # the exchanges did something, and what they did is the wrap-around described above
    ref = start.float()
    ref[:, :, :w] = ref[:, :, Ml:Ml + w]
    ref[:, :, w + Ml:] = ref[:, :, w:2 * w]
    first = start.to(dev).clone()
    flags_c = torch.zeros(4, dtype=torch.int32, device=dev)
    arr_c, fl_c = ring(first, flags_c, None)
    N.check(N.lib.wmm_halo_pull_static(arr_c, 2, C.byref(fl_c), lane, B, Ml, Nn, w, N.BF16, 0, stream))
    torch.cuda.synchronize()
    assert torch.equal(first.float().cpu(), ref)
    # epochs are counted in the caller's flag block: 4 exchanges on block b, 1 on the fresh block c, same lane
    assert int(flags_b[3]) == 4 and int(flags_b[0]) == 4 and int(flags_c[3]) == 1 and int(counters[0]) == 4
    assert N.device_status() == 0
