"""Sequence-shard halos through peer memory: the exchange of `sharded.py` without a host communication library.

`PeerHalo` keeps `count` sharded tensors of one shape in symmetric memory (every rank of the group maps every other
rank's allocation), each as an extended buffer (batch, rows + 2w, cols) = w margin rows | own rows | w margin rows, plus
a second set of the same buffers for partial gradients.  One neighbour exchange is ONE kernel launch of the library
(`wmm_halo_pull`, include/wmm_b200.h): plain peer loads over NVLink and a bounded flag hand-shake, capturable in a CUDA
graph together with the contractions around it.  Only the allocation and the exchange of the mapped pointers (once) go
through `torch.distributed` (`torch.distributed._symmetric_memory`).

    halo = PeerHalo(2, B, Ml, N, w, dtype, device)       # K^T and V of this rank
    halo.local(0).copy_(kt_rows); halo.local(1).copy_(v_rows)
    halo.exchange()                                       # margins <- neighbours' edge rows
    a = band_nt(q, halo.ext(0), w, other_off=w, seq=halo.seq) ...
    band_t(a, grad_o, w, other_rows=Ml + 2 * w, other_off=w, seq=halo.seq, out=halo.partial(1))
    grad_kt, grad_v = halo.reduce()                       # own rows += neighbours' partial rows

Every rank must call exchange() / reduce() in the same order.  The reference has no multi-GPU code.
"""
import ctypes
from typing import List, Tuple

import torch
import torch.distributed as dist

from . import _native as N


class PeerHalo:
    def __init__(self, count: int, batch: int, rows: int, cols: int, window: int, dtype, device, group=None, edges=False):
        import torch.distributed._symmetric_memory as symm_mem

        if not 1 <= count <= 4:
            raise RuntimeError("PeerHalo holds 1 to 4 tensors")
        if rows < 2 * window:
            raise RuntimeError("sequence shard of %d rows is shorter than twice the window %d" % (rows, window))
        self.group = dist.group.WORLD if group is None else group
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.count, self.batch, self.rows, self.cols, self.window = count, batch, rows, cols, window
        self.dtype, self.device = dtype, torch.device(device)
        ext_rows = rows + 2 * window
        # [0, count): operands; [count, 2 count): partial gradients of the same shape
        self.store = symm_mem.empty((2 * count, batch, ext_rows, cols), dtype=dtype, device=self.device)
        self.store.zero_()
        self.flags = symm_mem.empty((64,), dtype=torch.int32, device=self.device)
        self.flags.zero_()
        self.counters = torch.zeros(4, dtype=torch.int32, device=self.device)
        # optional: this rank's own first and last w rows of every partial gradient once more, unrounded (what
        # band_t(..., edges=, edge_skip=w) writes), so that the reduction adds the neighbour's rows before any rounding
        self.with_edges = bool(edges) and dtype in (torch.float16, torch.bfloat16)
        self.edge_store = torch.zeros((count, batch, 4 * window, cols), dtype=torch.float32, device=self.device) if self.with_edges else None
        torch.cuda.synchronize(self.device)
        hdl = symm_mem.rendezvous(self.store, self.group)
        fhdl = symm_mem.rendezvous(self.flags, self.group)
        self._handles = (hdl, fhdl)   # keep the mappings alive
        lo = self.rank - 1 if self.rank > 0 else None
        hi = self.rank + 1 if self.rank < self.world - 1 else None

        def base(h, t, r):
            # address of rank r's copy of tensor t: the handle lists the allocations' base addresses; the tensor sits at
            # the same offset in each
            off = t.data_ptr() - int(h.buffer_ptrs[self.rank])
            return int(h.buffer_ptrs[r]) + off

        per = batch * ext_rows * cols * self.store.element_size()
        self._bufs = []
        for part in (0, 1):
            arr = (N.HaloBuffer * count)()
            for i in range(count):
                o = (part * count + i) * per
                arr[i] = N.HaloBuffer(base(hdl, self.store, self.rank) + o, (base(hdl, self.store, lo) + o) if lo is not None else None,
                                      (base(hdl, self.store, hi) + o) if hi is not None else None)
            self._bufs.append(arr)
        self._edges = None
        if self.with_edges:
            self._edges = (N.HaloEdges * count)()
            for i in range(count):
                o = (count + i) * per
                self._edges[i] = N.HaloEdges(base(hdl, self.store, self.rank) + o, self.edge_store[i].data_ptr(),
                                             (base(hdl, self.store, lo) + o) if lo is not None else None,
                                             (base(hdl, self.store, hi) + o) if hi is not None else None)
        self._flags = N.HaloFlags(base(fhdl, self.flags, self.rank), base(fhdl, self.flags, lo) if lo is not None else None,
                                  base(fhdl, self.flags, hi) if hi is not None else None, self.counters.data_ptr())
        # in-sequence range of the extended row space of this rank (zeros stay in the margins at the global ends)
        self.seq: Tuple[int, int] = (window if self.rank == 0 else 0, rows + window if self.rank == self.world - 1 else ext_rows)
        # nobody starts an exchange before every rank has zeroed its flags and mapped its neighbours
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def ext(self, i: int) -> torch.Tensor:
        """Extended buffer of operand i: (batch, rows + 2w, cols)."""
        return self.store[i]

    def local(self, i: int) -> torch.Tensor:
        """This rank's rows of operand i: a view (batch, rows, cols) into ext(i)."""
        return self.store[i][:, self.window:self.window + self.rows]

    def partial(self, i: int) -> torch.Tensor:
        """Extended buffer for the partial gradient of operand i (what band_t writes with other_rows = rows + 2w)."""
        return self.store[self.count + i]

    def edges(self, i: int):
        """fp32 (batch, 4w, cols) buffer for the unrounded edge rows of partial gradient i (pass it to band_t with
        edge_skip = window), or None."""
        return self.edge_store[i] if self.with_edges else None

    def _pull(self, part: int, accumulate: bool, which=None) -> None:
        with torch.cuda.device(self.device):
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            if accumulate and self.with_edges:
                if which is None:
                    eds, count = self._edges, self.count
                else:
                    eds, count = (N.HaloEdges * 1)(self._edges[which]), 1
                N.check(N.lib.wmm_halo_reduce_edges(eds, count, ctypes.byref(self._flags), self.batch, self.rows, self.cols,
                                                    self.window, N.dtype_code(self.store), stream))
                return
            if which is None:
                bufs, count = self._bufs[part], self.count
            else:   # one tensor only (every rank must then exchange the same one)
                bufs, count = (N.HaloBuffer * 1)(self._bufs[part][which]), 1
            N.check(N.lib.wmm_halo_pull(bufs, count, ctypes.byref(self._flags), self.batch, self.rows, self.cols,
                                        self.window, N.dtype_code(self.store), 1 if accumulate else 0, stream))

    def exchange(self, which=None) -> List[torch.Tensor]:
        """Fills the margins of every operand (or of operand `which`) with the neighbours' edge rows; returns the
        extended buffers.  Runs on torch's current stream: issued on a side stream it overlaps work that needs no halo
        (see interior_rows)."""
        self._pull(0, False, which)
        return [self.ext(i) for i in range(self.count)] if which is None else [self.ext(which)]

    def reduce(self, which=None) -> List[torch.Tensor]:
        """Adds the neighbours' partial rows for this rank's edge positions; returns this rank's gradient rows."""
        self._pull(1, True, which)
        idx = range(self.count) if which is None else [which]
        return [self.partial(i)[:, self.window:self.window + self.rows] for i in idx]

    def interior_rows(self) -> Tuple[int, int]:
        """Rows [lo, hi) of this rank whose window touches no margin: a contraction over them needs no halo and can run
        while the exchange is still in flight; rows [0, lo) and [hi, rows) wait for it.  (A row i reads the extended rows
        i .. i + 2w; the margins are the first and last w of them.)"""
        return self.window, self.rows - self.window
