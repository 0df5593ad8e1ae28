"""Operators on HOST tensors: stream the batch through the GPU in chunks.

The reference also runs on CPU tensors (csrc/window_matmul/cpu/window_matmul_cpu.cpp); this package has no CPU
arithmetic, but a caller whose tensors live in host memory can still use the GPU kernels: the batch
dimension is independent in every contraction, so it is cut into chunks and three streams overlap the
host->device copy of chunk i+1, the kernels of chunk i and the device->host copy of chunk i-1.  PCIe is
full duplex, so a step costs about max(upload, download) instead of upload + compute + download.

    outs = batched_host_call(fn, inputs, chunks=8)            # one call
    pipe = HostPipeline(device); outs = pipe(fn, inputs)      # repeated calls: slots and result buffers are kept

`inputs`: CPU tensors (pinned memory for full copy speed) sharing dim 0; `fn(*device_chunks)` returns a tuple
of device tensors whose dim 0 is the chunk's; the results are written into pinned CPU tensors and returned
after a final synchronisation of the download stream.
"""
from typing import Callable, List, Optional, Sequence, Tuple

import torch


class HostPipeline:
    """The streams, device input slots and pinned result buffers of batched_host_call(), allocated once and reused by
    every call with the same shapes (a training loop calls with the same shapes every step)."""

    def __init__(self, device: Optional[torch.device] = None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.up, self.down = torch.cuda.Stream(device=self.device), torch.cuda.Stream(device=self.device)
        self._slots, self._slot_key = None, None
        self._results, self._result_key = None, None

    def _input_slots(self, inputs, per):
        key = (per,) + tuple((tuple(t.shape[1:]), t.dtype) for t in inputs)
        if key != self._slot_key:
            self._slots = [[torch.empty((per,) + tuple(t.shape[1:]), dtype=t.dtype, device=self.device) for t in inputs]
                           for _ in range(2)]
            self._slot_key = key
        return self._slots

    def __call__(self, fn: Callable[..., Sequence[torch.Tensor]], inputs: Sequence[torch.Tensor], chunks: int = 8,
                 outputs: Optional[List[torch.Tensor]] = None) -> Tuple[torch.Tensor, ...]:
        device = self.device
        B = inputs[0].shape[0]
        if any(t.shape[0] != B or t.is_cuda for t in inputs):
            raise RuntimeError("batched_host_call: inputs must be host tensors with a common first dimension")
        chunks = max(1, min(chunks, B))
        per = (B + chunks - 1) // chunks
        bounds = [(i, min(B, i + per)) for i in range(0, B, per)]
        compute = torch.cuda.current_stream(device)
        up, down = self.up, self.down
        up.wait_stream(compute)
        down.wait_stream(compute)
        # two device slots for the inputs: chunk i uploads into slot i % 2 once chunk i - 2 has been computed
        slots = self._input_slots(inputs, per)
        slot_free = [None, None]
        results = outputs
        for i, (lo, hi) in enumerate(bounds):
            slot = slots[i % 2]
            with torch.cuda.stream(up):
                if slot_free[i % 2] is not None:
                    up.wait_event(slot_free[i % 2])
                for dst, src in zip(slot, inputs):
                    dst[: hi - lo].copy_(src[lo:hi], non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(up)
            compute.wait_event(uploaded)
            outs = tuple(fn(*[t[: hi - lo] for t in slot]))
            computed = torch.cuda.Event()
            computed.record(compute)
            slot_free[i % 2] = computed
            if results is None:
                key = (B,) + tuple((tuple(o.shape[1:]), o.dtype) for o in outs)
                if key != self._result_key:
                    self._results = [torch.empty((B,) + tuple(o.shape[1:]), dtype=o.dtype).pin_memory() for o in outs]
                    self._result_key = key
                results = self._results
            with torch.cuda.stream(down):
                down.wait_event(computed)
                for dst, src in zip(results, outs):
                    src.record_stream(down)
                    dst[lo:hi].copy_(src, non_blocking=True)
        down.synchronize()
        # the next call may overwrite the input slots only after this call's kernels: they run on `compute`, which the
        # next call's upload stream waits for
        return tuple(results)


def batched_host_call(fn: Callable[..., Sequence[torch.Tensor]], inputs: Sequence[torch.Tensor], chunks: int = 8,
                      device: Optional[torch.device] = None, outputs: Optional[List[torch.Tensor]] = None) -> Tuple[torch.Tensor, ...]:
    """One-off form: allocates its slots for this call.  Keep a HostPipeline to reuse them across calls."""
    return HostPipeline(device)(fn, inputs, chunks, outputs)
