#!/usr/bin/env python
"""Benchmark of the banded-contraction hot path: forward + backward of window_matmul -> unwindow_matmul.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c3|c4|c5]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one pass of the six contractions (window fwd, unwindow fwd, unwindow bwd {grad_A, grad_V},
window bwd {grad_Q, grad_K}) over the workload.  The default workload is the configuration the headline
metric is quoted on: B = 96 (8 batch x 12 heads), M = 4096, N = 64, w = 256, bf16, seeded N(0,1)/sqrt(N)
inputs.  On N > 1 GPUs the batch is split evenly over the ranks (no data-path communication; strong
scaling: the job is the same 96 sequences) and the time is the maximum over ranks.

Prints ONE JSON line (rank 0).  `value` is microseconds per step with inputs resident in HBM, the six
kernels replayed from a CUDA graph; `e2e` is the same step through the package's public, differentiable
API with pinned HOST buffers, host->device and device->host copies inside the timed region.
`--impl reference` times the reference's own CPU implementation (oracle/_ref, else the CPU oracle port)
on a bounded sample of the same workload and extrapolates to the full size.
"""
import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "pytorch-window-matmul_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

WORKLOADS = {
    # name: (B, M, N, w, dtype, distribution)
    "c1": (4, 1024, 64, 64, "fp32", "normal"),
    "c2": (96, 4096, 64, 256, "bf16", "normal_scaled"),
    "c2_fp32": (96, 4096, 64, 256, "fp32", "normal_scaled"),
    "c3": (1024, 2048, 32, 8, "fp16", "uniform"),
    "c4": (16, 65536, 128, 512, "bf16", "normal_scaled"),
    "c5": (64, 16384, 64, 384, "bf16", "normal"),
}
METRIC = "fwd+bwd window+unwindow us at B=96 M=4096 N=64 w=256"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, per band row, from an ncu capture of each kernel at
# B=48 (196608 rows per launch).
# (bytes per band row, bytes per launch).  The window backward (one sweep over grad_A) re-reads a fixed number of boxes at
# the start of every CTA's run: 59.7 MB per launch whatever the batch, on top of 1461.8 B per band row.
NCU_DRAM_BYTES_PER_ROW = {"c2": {"band_nt": (990.9, 0.0), "band_n+band_t": (1449.8, 59.7e6), "band_n": (1245.4, 0.0),
                                 "band_t": (1226.9, 0.0)}}


def algorithmic(B, M, N, w, e):
    """Bytes and flops of one step: each distinct input read once and each output written once per
    autograd node; 6 contractions of 2*B*M*(2w+1)*N flops."""
    W = 2 * w + 1
    return e * (11 * B * M * N + 5 * B * M * W), 12 * B * M * W * N


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.004)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {
            "sm_mhz": s[len(s) // 2] if s else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(s),
        }


def make_inputs(B, M, N, w, dist, seed, torch):
    g = torch.Generator(device="cpu").manual_seed(seed)
    if dist == "uniform":
        mk = lambda: torch.rand(B, M, N, generator=g)  # noqa: E731
    else:
        s = (1.0 / N ** 0.5) if dist == "normal_scaled" else 1.0
        mk = lambda: torch.randn(B, M, N, generator=g) * s  # noqa: E731
    q, kt, v = mk(), mk(), mk()
    go = torch.randn(B, M, N, generator=g)
    return q, kt, v, go


# ---------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's CPU implementation on a bounded sample
# ---------------------------------------------------------------------------------------------------


def _cpu_reference_module():
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if os.path.exists(os.path.join(ref_dir, "window_matmul_kernel.so")):
        sys.path.insert(0, ref_dir)
        try:
            import window_matmul_kernel

            return window_matmul_kernel, "reference"
        except Exception:
            pass
    from oracle import oracle

    return oracle, "port"


def cpu_chain_seconds(mod, kind, q, kt, v, go, w, torch):
    """One fwd+bwd chain on the CPU (fp32, one thread as the reference ships it).  Returns seconds."""
    k = kt.transpose(1, 2).contiguous()
    t0 = time.perf_counter()
    if kind == "reference":
        a = mod.window_matmul_forward(q, k, w)
        mod.unwindow_matmul_forward(a, v, w)
        ga, _gv = mod.unwindow_matmul_backward(a, v, w, go)
        mod.window_matmul_backward(q, k, w, ga)
    else:
        mod.chain_fwd_bwd(q.numpy(), k.numpy(), v.numpy(), w, go.numpy())
    return time.perf_counter() - t0


def cpu_sample_plan(B, M, N, w, budget_s, steps):
    """Chooses (batch entries, rows) of the per-step CPU sample so that `steps` of them fit the budget.
    Cost model: ~1.2e-9 s per multiply-add of the six single-threaded loops (measured on this image)."""
    per_row = 6 * (2 * w + 1) * N * 1.2e-9 * 2
    rows_budget = max(1.0, budget_s / max(1, steps) / per_row)
    Ms = M
    while Ms > 4 * w and Ms > 512 and Ms > rows_budget:
        Ms //= 2
    Bs = int(max(1, min(B, rows_budget // Ms)))
    return Bs, Ms


def run_reference(args, torch):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    B, M, N, w, dt, dist = WORKLOADS[args.workload]
    mod, kind = _cpu_reference_module()
    torch.set_num_threads(1)
    Bs, Ms = cpu_sample_plan(B, M, N, w, 150.0, args.steps + args.warmup)
    q, kt, v, go = make_inputs(Bs, Ms, N, w, dist, 0, torch)
    if dt != "fp32":  # the reference has no bf16 and accumulates fp16 in fp16: run fp32 on the rounded inputs
        lowp = torch.bfloat16 if dt == "bf16" else torch.float16
        q, kt, v, go = (t.to(lowp).float() for t in (q, kt, v, go))
    for _ in range(args.warmup):
        cpu_chain_seconds(mod, kind, q, kt, v, go, w, torch)
    t = [cpu_chain_seconds(mod, kind, q, kt, v, go, w, torch) for _ in range(args.steps)]
    scale = (B * M) / float(Bs * Ms)
    step_s = sum(t) / len(t)
    value = step_s * scale * 1e6
    sample = "B=%d M=%d of B=%d M=%d (N=%d w=%d, fp32 on %s-rounded inputs), x%.1f extrapolated" % (Bs, Ms, B, M, N, w, dt, scale)
    line = {
        "impl": "reference", "metric": METRIC if args.workload == "c2" else "fwd+bwd window+unwindow us (%s)" % args.workload,
        "value": value, "unit": "us", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": value / 1e3, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.workload), "reference_cpu_step_s_on_sample": step_s},
        "cpu_baseline": {"value": value, "unit": "us", "cores": 1, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def reference_cuda_summary(args, torch, steps=None):
    """The reference's own CUDA kernels (csrc/window_matmul/cuda/window_matmul_cuda.cu, compiled unmodified by
    oracle/build_ref.py) on this GPU, same workload, through its four pybind entry points.  The reference has
    no bf16: bf16 workloads run in fp16 (same bytes).  Reported beside our numbers, not part of the contract's
    two arms.  Returns a dict."""
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "WITH_CUDA")):
        return {"unavailable": "oracle/_ref was built without the reference's CUDA sources"}
    sys.path.insert(0, ref_dir)
    try:
        import window_matmul_kernel as ref
    except Exception as ex:
        return {"unavailable": "the compiled reference does not import: %s" % ex}
    steps = steps or max(2, min(args.steps, 5))
    B, M, N, w, dt, dist = WORKLOADS[args.workload]
    dtype = {"bf16": torch.float16, "fp16": torch.float16, "fp32": torch.float32}[dt]
    e = 2 if dt != "fp32" else 4
    q, kt, v, go = (t.to(dtype).cuda() for t in make_inputs(B, M, N, w, dist, 0, torch))
    k = kt.transpose(-1, -2)  # a view: the reference's transposing copy (window_matmul_cuda.cu:236) is then free

    def step():
        a = ref.window_matmul_forward(q, k, w)
        ref.unwindow_matmul_forward(a, v, w)
        ga, _ = ref.unwindow_matmul_backward(a, v, w, go)
        ref.window_matmul_backward(q, k, w, ga)

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / steps
    total_bytes, total_flops = algorithmic(B, M, N, w, e)
    return {"us": round(us, 1), "steps": steps, "dtype": "f16" if dt != "fp32" else "f32",
            "note": "reference CUDA kernels (unmodified, sm_100), legacy default stream, zero-filled outputs, K as a transposed view",
            "achieved_GBps": round(total_bytes / (us * 1e-6) / 1e9, 1), "TFLOPs": round(total_flops / (us * 1e-6) / 1e12, 2)}


def run_reference_cuda(args, torch):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    r = reference_cuda_summary(args, torch, steps=args.steps)
    line = {"impl": "reference_cuda", "metric": "fwd+bwd window+unwindow us (%s)" % args.workload, "unit": "us", "n_gpus": 1,
            "warmup": 2, "data": "synthetic", "config": {"workload": workload_name(args.workload)}}
    line.update(r)
    if "us" in r:
        line["value"] = r["us"]
    print(json.dumps(line), flush=True)


def workload_name(key):
    B, M, N, w, dt, dist = WORKLOADS[key]
    return "%s: B=%d M=%d N=%d w=%d %s fwd+bwd window_matmul->unwindow_matmul, %s inputs" % (key, B, M, N, w, dt, dist)


# ---------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------


def run_ours(args, torch):
    import importlib

    import window_matmul as pkg
    from window_matmul import _native as N_

    impl = importlib.import_module("window_matmul.window_matmul")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist_on = world > 1
    if dist_on:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    B, M, N, w, dt, distn = WORKLOADS[args.workload]
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[dt]
    e = 2 if dt != "fp32" else 4
    if args.tf32:
        impl.set_flags(N_.FLAG_TF32)
    if args.shard == "seq" or (args.shard == "auto" and args.workload == "c4" and world > 1):
        return run_seq_sharded(args, torch, impl, N_, rank, world, dev)
    # strong scaling: the same B sequences, split evenly over the ranks (the last rank may get fewer)
    per = (B + world - 1) // world
    b0, b1 = min(B, rank * per), min(B, (rank + 1) * per)
    Bl = b1 - b0
    q, kt, v, go = make_inputs(B, M, N, w, distn, 0, torch)
    q, kt, v, go = (t[b0:b1].to(dtype).contiguous() for t in (q, kt, v, go))
    host = [t.pin_memory() for t in (q, kt, v, go)]
    qd, ktd, vd, god = (t.to(dev) for t in host)
    if args.k_layout == "bnm":  # K stored as a contiguous (B, N, M) tensor; ktd is its (B, M, N) view
        ktd = ktd.transpose(-1, -2).contiguous().transpose(-1, -2)
    W = 2 * w + 1
    a = torch.empty(Bl, M, W, dtype=dtype, device=dev)
    ga = torch.empty_like(a)
    o, gv, gq, gkt = (torch.empty(Bl, M, N, dtype=dtype, device=dev) for _ in range(4))

    kd = ktd.transpose(-1, -2)  # K as the (B,N,M) tensor the operators take
    # the four native calls of the reference's module = one step (5 kernel launches)
    ops = [
        lambda: impl.band_nt(qd, ktd, w, out=a),                                        # window forward
        lambda: impl.band_n(a, vd, w, out=o),                                           # unwindow forward
        lambda: impl.unwindow_matmul_backward(a, vd, w, god, out=(ga, gv)),             # grad_A, grad_V
        lambda: impl.window_matmul_backward(qd, kd, w, ga, out=(gq, gkt)),              # grad_Q, grad_K (one launch)
    ]
    launches_per_step = 5
    # (name, call, algorithmic bytes per band row / e): per-kernel durations for the roofline
    kernels = [
        ("window_fwd band_nt", ops[0], 2 * N + W),
        ("unwindow_fwd band_n", ops[1], 2 * N + W),
        ("unwindow_bwd grad_A band_nt", lambda: impl.band_nt(god, vd, w, out=ga), 2 * N + W),
        ("unwindow_bwd grad_V band_t", lambda: impl.band_t(a, god, w, out=gv), 2 * N + W),
        ("window_bwd grad_Q+grad_K band_n+band_t", ops[3], 4 * N + W),
    ]

    def step():
        for fn in ops:
            fn()

    # SMs per kernel of the DAG: [window fwd, grad_A, unwindow fwd, grad_V, window bwd]; 0 = all of them
    sms_total = torch.cuda.get_device_properties(dev).multi_processor_count
    tiles_per_sm = Bl * ((M + 127) // 128) / float(sms_total)
    if args.sm_split == "auto":
        split_on = args.branches == 2 and 0 < tiles_per_sm < 16.0
        caps = [sms_total // 2, sms_total // 2, sms_total // 4, sms_total // 4, sms_total // 2] if split_on else [0] * 5
    elif args.sm_split == "off":
        caps = [0] * 5
    else:
        caps = [int(x) for x in args.sm_split.split(",")]
        assert len(caps) == 5, "--sm-split takes five CTA caps"
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        for _ in range(max(3, args.warmup)):
            step()
        stream.synchronize()
        graph = None
        if Bl > 0 and not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                if args.branches == 2:
                    # The step is a small DAG, not a chain: window fwd feeds unwindow fwd and grad_V (both only
                    # read A); grad_A needs only the upstream gradient and feeds the window backward.  Captured
                    # with its real dependencies, the tail of one kernel (SMs running out of tiles) is filled
                    # by another branch's kernel.
                    # With few tiles per SM (a batch shard of a multi-GPU run) the fixed cost of a launch -- first loads,
                    # the epilogue's first pass, the last wave -- is paid five times in a row, because every kernel asks
                    # for all SMs and so runs alone.  `caps` gives the kernels of one level of the DAG a share of the
                    # SMs each (wmm_set_cta_limits, read at capture), so they start together and pay it side by side.
                    s1, s2 = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

                    def capped(cap, fn):
                        with N_.cta_limits(cap, 0):
                            fn()

                    s1.wait_stream(stream)
                    with torch.cuda.stream(s1):
                        capped(caps[1], lambda: impl.band_nt(god, vd, w, out=ga))
                        capped(caps[4], ops[3])
                    capped(caps[0], ops[0])
                    s2.wait_stream(stream)
                    with torch.cuda.stream(s2):
                        capped(caps[3], lambda: impl.band_t(a, god, w, out=gv))
                    capped(caps[2], ops[1])
                    stream.wait_stream(s1)
                    stream.wait_stream(s2)
                else:
                    step()
            for _ in range(2):
                graph.replay()
            stream.synchronize()

        def barrier():
            torch.cuda.synchronize(dev)
            if dist_on:
                dist.barrier()
            torch.cuda.synchronize(dev)

        # ---- device-resident timing: blocks of exactly K steps, each between two events on the launching stream.
        # `value` is the MEDIAN block (min and max are reported beside it): the blocks together span about a second, so
        # the number is a sustained one and its spread is on record.
        def run_steps(n):
            for _ in range(n):
                if graph is not None:
                    graph.replay()
                else:
                    step()

        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record(stream)
        run_steps(3)
        p1.record(stream)
        stream.synchronize()
        est_ms = max(1e-3, p0.elapsed_time(p1) / 3) * args.steps
        blocks = args.blocks if args.blocks > 0 else int(min(400, max(50, math.ceil(1000.0 / est_ms))))
        if dist_on:   # every rank times the same number of blocks
            nb = torch.tensor([blocks], device=dev)
            dist.all_reduce(nb, op=dist.ReduceOp.MAX)
            blocks = int(nb[0])
        launches0 = N_.launch_count()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
        barrier()
        with ClockSampler(local_rank) as clocks:
            evs[0].record(stream)
            for i in range(blocks):
                run_steps(args.steps)
                evs[i + 1].record(stream)
            stream.synchronize()
        barrier()
        block_ms = sorted(evs[i].elapsed_time(evs[i + 1]) for i in range(blocks))
        elapsed_ms, block_min_ms, block_max_ms = block_ms[len(block_ms) // 2], block_ms[0], block_ms[-1]
        launches = (N_.launch_count() - launches0) if graph is None else blocks * args.steps * launches_per_step

        # ---- per-kernel durations (for the roofline of the dominant kernel) ----
        per_kernel = {}
        reps = 10
        for name, fn, cols in kernels:
            if Bl == 0:
                continue
            fn()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            stream.synchronize()
            kgraph = None
            if not args.no_graph:  # replayed from a graph so that host launch overhead cannot hide in the number
                kgraph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(kgraph, stream=stream):
                    for _ in range(reps):
                        fn()
                stream.synchronize()
            k0.record(stream)
            if kgraph is not None:
                kgraph.replay()
            else:
                for _ in range(reps):
                    fn()
            k1.record(stream)
            stream.synchronize()
            us = k0.elapsed_time(k1) * 1e3 / reps
            nbytes = e * Bl * M * cols
            per_kernel[name] = {"us": round(us, 2), "alg_MB": round(nbytes / 1e6, 1), "GBps": round(nbytes / us / 1e3, 1)}

        # ---- the attention block the two operators are written for: window fwd -> scale, mask, softmax -> unwindow
        # fwd, and its backward, with the band softmax of this library between the operators (7 launches).  Reported
        # beside the headline (which stays the reference's own four calls), with the same block using torch ops for
        # the softmax as the reference's users compose it.
        block = None
        if Bl > 0 and (args.block == "on" or (args.block == "auto" and args.workload == "c5")):
            from window_matmul import softmax as sm_

            scale = 1.0 / math.sqrt(N)

            def block_step():
                impl.band_nt(qd, ktd, w, out=a)
                sm_.band_softmax(a, scale, True, out=a)                       # probabilities, in place
                impl.band_n(a, vd, w, out=o)
                impl.unwindow_matmul_backward(a, vd, w, god, out=(ga, gv))    # grad_P, grad_V
                sm_.band_softmax_backward(a, ga, scale, True, out=ga)         # grad_scores, in place
                impl.window_matmul_backward(qd, kd, w, ga, out=(gq, gkt))

            def timed(fn, reps):
                fn()
                stream.synchronize()
                g = None
                if not args.no_graph:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        for _ in range(reps):
                            fn()
                    stream.synchronize()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record(stream)
                if g is not None:
                    g.replay()
                else:
                    for _ in range(reps):
                        fn()
                t1.record(stream)
                stream.synchronize()
                return t0.elapsed_time(t1) * 1e3 / reps

            block_us = timed(block_step, 5)
            sm_f = timed(lambda: sm_.band_softmax(a, scale, True, out=ga), 5)
            sm_b = timed(lambda: sm_.band_softmax_backward(a, ga, scale, True, out=ga), 5)
            band_bytes = e * Bl * M * W
            ii = torch.arange(M, device=dev)[:, None]
            jj = torch.arange(W, device=dev)[None, :]
            outside = ((ii + jj - w) < 0) | ((ii + jj - w) >= M)
            a_req = a.detach().clone().requires_grad_()

            def torch_softmax_fwd_bwd():
                pr = torch.softmax((a_req * scale).masked_fill(outside, float("-inf")), dim=-1)
                pr.backward(ga)
                a_req.grad = None

            torch_us = timed(torch_softmax_fwd_bwd, 2) if args.no_graph else None
            if torch_us is None:   # torch's autograd ops are timed from the stream, not from a graph
                torch_softmax_fwd_bwd()
                stream.synchronize()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record(stream)
                for _ in range(3):
                    torch_softmax_fwd_bwd()
                t1.record(stream)
                stream.synchronize()
                torch_us = t0.elapsed_time(t1) * 1e3 / 3
            del a_req
            block_bytes = e * Bl * M * (11 * N + 10 * W)
            block = {
                "us": round(block_us, 1), "launches": 7, "alg_MB": round(block_bytes / 1e6, 1),
                "GBps": round(block_bytes / block_us / 1e3, 1),
                "softmax_fwd": {"us": round(sm_f, 1), "GBps": round(2 * band_bytes / sm_f / 1e3, 1)},
                "softmax_bwd": {"us": round(sm_b, 1), "GBps": round(3 * band_bytes / sm_b / 1e3, 1)},
                "torch_softmax_fwd_bwd_us": round(torch_us, 1),
            }

        # ---- end to end through the public API, host buffers, copies inside the timed region ----
        e2e_steps = max(3, min(args.steps, 20))
        outs_host = [torch.empty(Bl, M, N, dtype=dtype).pin_memory() for _ in range(4)]

        from window_matmul.host_pipeline import HostPipeline

        pipe = HostPipeline(dev)

        def chain(qh, kth, vh, goh):
            """What a user of the package writes: the two differentiable operators and .backward() on one device-resident
            chunk of the batch.  Returns the output and the three gradients."""
            qd_, ktd_, vd_ = (t.detach().requires_grad_(True) for t in (qh, kth, vh))
            att = pkg.window_matmul(qd_, ktd_.transpose(-1, -2), w)
            out = pkg.unwindow_matmul(att, vd_, w)
            out.backward(goh)
            return out.detach(), qd_.grad, ktd_.grad, vd_.grad

        # a handful of chunks: enough for uploads, kernels and downloads to overlap, few enough that the host-side cost
        # per chunk (autograd, ~10 launches: ~0.45 ms measured) stays below the copies of a chunk (12 sequences = 25 MB each
        # way = ~0.5 ms): one chunk per 12 sequences, at most 8 (12 sequences per GPU: 1.09 / 1.29 / 1.72 / 2.18 ms with
        # 1 / 2 / 3 / 4 chunks)
        e2e_chunks = args.e2e_chunks if args.e2e_chunks > 0 else max(1, min(8, Bl // 12))

        def e2e_step():
            # host tensors in, host tensors out; uploads, kernels and downloads of batch chunks overlap
            pipe(chain, host, chunks=e2e_chunks, outputs=outs_host)

        run_e2e = Bl > 0 and not args.skip_e2e
        if run_e2e:
            for _ in range(2):
                e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        if run_e2e:
            for _ in range(e2e_steps):
                e2e_step()
        e1.record(stream)
        stream.synchronize()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps

    status = N_.device_status()
    if status != 0:
        raise SystemExit("bench.py: a kernel abandoned a bounded wait (device status %d); numbers are void" % status)

    # max over ranks, on the device clock
    t = torch.tensor([elapsed_ms, e2e_ms, block_min_ms, block_max_ms], dtype=torch.float64, device=dev)
    if dist_on:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, block_min_ms, block_max_ms = (float(x) for x in t)
    us_per_step = elapsed_ms * 1e3 / args.steps

    if rank == 0:
        peak, peak_kind = measured_peaks()
        total_bytes, total_flops = algorithmic(B, M, N, w, e)
        dom = max(per_kernel.items(), key=lambda kv: kv[1]["us"]) if per_kernel else (None, None)
        traffic = None
        if dom[0] and args.workload in NCU_DRAM_BYTES_PER_ROW:
            per_row = NCU_DRAM_BYTES_PER_ROW[args.workload].get(dom[0].split()[-1])
            if per_row:  # captured at B=48; traffic grows in proportion to the band rows of a launch
                traffic = per_row[0] * Bl * M + per_row[1]
        line = {
            "metric": METRIC if args.workload == "c2" and not args.batch and not args.rows else "fwd+bwd window+unwindow us (%s)" % args.workload,
            "value": us_per_step, "unit": "us", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "blocks": {"n": blocks, "steps_each": args.steps, "value_is": "median block, max over ranks",
                       "min_us": round(block_min_ms * 1e3 / args.steps, 2), "median_us": round(us_per_step, 2),
                       "max_us": round(block_max_ms * 1e3 / args.steps, 2),
                       "timed_s": round(sum(block_ms) / 1e3, 3)},
            "ms_per_step": us_per_step / 1e3, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": dt.replace("fp", "f"), "data": "synthetic",
            "config": {
                "workload": workload_name(args.workload), "batch_per_gpu": per,
                "l2": "no flush: one step touches %.0f MB per GPU, larger than the 126 MB L2" % (total_bytes / world / 1e6),
                "launch": ("cuda graph of %d kernels, %s" % (launches_per_step, ("dependency DAG" + (", CTAs per kernel %s" % caps if any(caps) else "")) if args.branches == 2 else "one chain")) if graph is not None else "%d stream launches" % launches_per_step,
                "k_layout": "contiguous (B,N,M)" if args.k_layout == "bnm" else "transposed view of (B,M,N)",
                **({"fp32_mode": "tf32 products on the tensor cores (WMM_FLAG_TF32)" if args.tf32 else "exact-order fp32"} if dt == "fp32" else {}),
            },
            "step_roofline": {
                "alg_MB": round(total_bytes / 1e6, 1), "alg_GFLOP": round(total_flops / 1e9, 1),
                "achieved_GBps": round(total_bytes / world / (us_per_step * 1e-6) / 1e9, 1) * world,
                "frac_of_%s_hbm" % peak_kind: round(total_bytes / world / (us_per_step * 1e-6) / 1e9 / peak, 4),
                "TFLOPs": round(total_flops / (us_per_step * 1e-6) / 1e12, 1),
            },
            "roofline": {
                "bound": "hbm", "kernel": dom[0], "achieved": dom[1]["GBps"] if dom[0] else None, "peak": peak,
                "unit": "GB/s", "frac": round(dom[1]["GBps"] / peak, 4) if dom[0] else None, "peak_kind": peak_kind,
                "traffic": traffic,
            },
            "per_kernel": per_kernel,
            "attention_block": block,
            "e2e": {
                "value": e2e_ms * 1e3 if run_e2e else None, "unit": "us", "h2d_bytes_per_step": 4 * Bl * M * N * e * world,
                "d2h_bytes_per_step": 4 * Bl * M * N * e * world, "steps": e2e_steps, "chunks_per_gpu": e2e_chunks,
                "api": "window_matmul.window_matmul -> window_matmul.unwindow_matmul -> .backward() per batch chunk, pinned host buffers",
            },
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            mod, kind = _cpu_reference_module()
            torch.set_num_threads(1)
            Bs, Ms = cpu_sample_plan(B, M, N, w, 15.0, 2)
            cq, ckt, cv, cgo = make_inputs(Bs, Ms, N, w, distn, 0, torch)
            if dt != "fp32":
                cq, ckt, cv, cgo = (x.to(dtype).float() for x in (cq, ckt, cv, cgo))
            cpu_chain_seconds(mod, kind, cq, ckt, cv, cgo, w, torch)  # the first call carries one-off warm-up
            secs = cpu_chain_seconds(mod, kind, cq, ckt, cv, cgo, w, torch)
            scale = (B * M) / float(Bs * Ms)
            line["cpu_baseline"] = {
                "value": secs * scale * 1e6, "unit": "us", "cores": 1, "kind": kind,
                "sample": "B=%d M=%d of B=%d M=%d, fp32 on %s-rounded inputs, %.2f s measured, x%.1f extrapolated; host has %d cores, "
                          "the reference's loops use one" % (Bs, Ms, B, M, dt, secs, scale, os.cpu_count()),
            }
        if world == 1 and not args.no_reference_cuda and not args.batch:
            line["reference_cuda"] = reference_cuda_summary(args, torch)
    if dist_on and args.workload == "c2" and not args.no_seq_extra and not args.batch:
        # the other multi-GPU partitioning, on the same ranks: config 4 split along the sequence with halo exchange
        try:
            seq = measure_seq_sharded(args, torch, impl, N_, rank, world, dev, "c4", max(5, min(args.steps, 20)))
        except Exception as ex:   # reported, never hides the headline
            seq = {"error": "%s: %s" % (type(ex).__name__, ex)}
        if rank == 0:
            line["seq_sharded"] = seq
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist_on:
        dist.destroy_process_group()


def _seq_rank_inputs(torch, r, B, Ml, N, distn, dtype):
    """The rows rank r owns, from a CPU generator seeded by r: any rank can regenerate a neighbour's rows."""
    g = torch.Generator(device="cpu").manual_seed(1000 + r)
    s = 1.0 / N ** 0.5 if distn == "normal_scaled" else 1.0
    q, kt, v = ((torch.randn(B, Ml, N, generator=g) * s).to(dtype) for _ in range(3))
    go = torch.randn(B, Ml, N, generator=g).to(dtype)
    return q, kt, v, go


def _seq_parity(torch, impl, dev, workload, world, got, mine):
    """Rank 0's rows of all six results against the UNSHARDED kernels of this library on the same seeded rows: rows
    [0, Ml) of a sequence depend on positions below Ml + 2w only, so the plain operators run on rank 0's rows plus the
    first 2w rows of rank 1 (regenerated from rank 1's seed).  Returns, per tensor, max |x - y| / (1e-2 (|y| + rms(y)));
    <= 1 means within the 16-bit bound.  The sharded grad_K / grad_V edge rows are sums of two partial rows: summed from
    this rank's unrounded fp32 rows and the neighbour's 16-bit rows (--edges 1) they carry one rounding more than the
    unsharded rows; summed as 16-bit rows (--edges 0) two more, which can pass the bound where the partial rows cancel."""
    B, M, N, w, dt, distn = WORKLOADS[workload]
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[dt]
    Ml = M // world
    q, kt, v, go = mine
    if world > 1:
        nq, nkt, nv, ngo = _seq_rank_inputs(torch, 1, B, Ml, N, distn, dtype)
        q, kt, v, go = (torch.cat([x, y[:, :2 * w]], dim=1) for x, y in ((q, nq), (kt, nkt), (v, nv), (go, ngo)))
    q, kt, v, go = (t.to(dev) for t in (q, kt, v, go))
    ra = impl.band_nt(q, kt, w)
    ro = impl.band_n(ra, v, w)
    rga = impl.band_nt(go, v, w)
    rgv = impl.band_t(ra, go, w)
    rgq = impl.band_n(rga, kt, w)
    rgk = impl.band_t(rga, q, w)
    out = {}
    for name, x, y in (("a", got["a"], ra), ("o", got["o"], ro), ("ga", got["ga"], rga), ("gq", got["gq"], rgq),
                       ("gk", got["gk"], rgk), ("gv", got["gv"], rgv)):
        y = y[:, :Ml].float()
        x = x.float()
        rms = float(y.pow(2).mean().sqrt())
        out[name] = round(float(((x - y).abs() / (1e-2 * (y.abs() + rms) + 1e-30)).max()), 4)
    out["max_err_over_bound"] = max(out.values())
    return out


def measure_seq_sharded(args, torch, impl, N_, rank, world, dev, workload, steps, parity=True):
    """Sequence-sharded step (config 4): rank r owns rows [r*M/P, (r+1)*M/P) of every tensor; K^T and V rows within w
    of a shard edge are exchanged with the neighbours before the forward contractions, partial grad_K / grad_V rows
    after the backward ones.  Same six contractions, same job at every P (strong scaling); time = max over ranks on
    device clocks.  Returns a dict (the same on every rank).  Needs an initialised process group when world > 1."""
    import torch.distributed as dist

    from window_matmul import sharded

    B, M, N, w, dt, distn = WORKLOADS[workload]
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[dt]
    e = 2 if dt != "fp32" else 4
    Ml = M // world
    qc, ktc, vc, goc = _seq_rank_inputs(torch, rank, B, Ml, N, distn, dtype)
    q, go = qc.to(dev), goc.to(dev)
    # K^T and V live in storage with halo margins, so the exchange writes only the margins
    kt, _ = sharded.alloc_with_halo(B, Ml, N, w, dtype, dev)
    v, _ = sharded.alloc_with_halo(B, Ml, N, w, dtype, dev)
    kt.copy_(ktc)
    v.copy_(vc)
    W = 2 * w + 1
    a = torch.empty(B, Ml, W, dtype=dtype, device=dev)
    ga = torch.empty_like(a)
    o, gq = torch.empty_like(q), torch.empty_like(q)
    seq = sharded._local_seq(Ml, w, None) if world > 1 else (0, Ml)
    ext = Ml + 2 * w if world > 1 else Ml
    off = w if world > 1 else 0
    halo = (lambda xs: sharded.exchange_halo_many(xs, w)) if world > 1 else (lambda xs: xs)
    unhalo = (lambda xs: sharded.reduce_halo_many(xs, w)) if world > 1 else (lambda xs: xs)

    # Two neighbour exchanges per step: the K^T and V halos together before the forward contractions, the partial
    # grad_K and grad_V rows together after the backward ones.
    #   --exchange peer (default): each exchange is ONE kernel of the library reading the neighbours' rows through peer
    #     memory (window_matmul/peer_halo.py); the whole step, exchanges included, replays as one CUDA graph.
    #   --exchange nccl: torch.distributed send/recv pairs (window_matmul/sharded.py) around a graph of the six
    #     contractions; each exchange costs ~120 us of host time per rank, which binds the step at 8 ranks.
    peer = world > 1 and args.exchange == "peer"
    parts = {}
    ph = None
    if peer:
        from window_matmul.peer_halo import PeerHalo

        ph = PeerHalo(2, B, Ml, N, w, dtype, dev, edges=args.edges)
        ph.local(0).copy_(kt)
        ph.local(1).copy_(v)

    launch_list = [
        ("window_fwd band_nt", lambda k_, v_: impl.band_nt(q, k_, w, other_off=off, seq=seq, out=a)),
        ("unwindow_fwd band_n", lambda k_, v_: impl.band_n(a, v_, w, other_off=off, seq=seq, out=o)),
        ("unwindow_bwd grad_A band_nt", lambda k_, v_: impl.band_nt(go, v_, w, other_off=off, seq=seq, out=ga)),
        ("unwindow_bwd grad_V band_t", lambda k_, v_: parts.__setitem__("gv", impl.band_t(
            a, go, w, other_rows=ext, other_off=off, seq=seq, out=ph.partial(1) if peer else None,
            edges=ph.edges(1) if peer else None, edge_skip=w))),
        ("window_bwd grad_Q band_n", lambda k_, v_: impl.band_n(ga, k_, w, other_off=off, seq=seq, out=gq)),
        ("window_bwd grad_K band_t", lambda k_, v_: parts.__setitem__("gk", impl.band_t(
            ga, q, w, other_rows=ext, other_off=off, seq=seq, out=ph.partial(0) if peer else None,
            edges=ph.edges(0) if peer else None, edge_skip=w))),
    ]

    def contractions(kt_ext, v_ext):
        for _, fn in launch_list:
            fn(kt_ext, v_ext)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    stream = torch.cuda.Stream(device=dev)
    graph = None
    result = {}
    with torch.cuda.stream(stream):
        side = torch.cuda.Stream(device=dev) if peer and args.overlap > 0 else None

        free_sms = max(0, args.overlap_sms)
        sms_total = torch.cuda.get_device_properties(dev).multi_processor_count
        seq_tiles_per_sm = B * ((Ml + 127) // 128) / float(sms_total)
        seq_split = peer and not args.no_graph and args.overlap == 0 and (
            args.sm_split != "off" and (args.sm_split != "auto" or seq_tiles_per_sm < 16.0))

        def beside(exchange_fn, contraction_fn):
            """An exchange on the side stream beside a contraction on the main one.  The contraction leaves `free_sms` SMs,
            the exchange is capped at one CTA for each of them (wmm_set_cta_limits): without the caps the exchange's
            CTAs find no SM with room and run after the contraction."""
            ready = torch.cuda.Event()
            ready.record(stream)
            with N_.cta_limits(sms_total - free_sms if free_sms else 0, free_sms):
                with torch.cuda.stream(side):
                    side.wait_event(ready)
                    r = exchange_fn()
                    done = torch.cuda.Event()
                    done.record(side)
                contraction_fn()
            stream.wait_event(done)
            return r

        def overlapped_step():
            """Exchanges beside contractions that do not need them.  Level 1: K^T margins first (nothing to hide them
            under), V margins beside the window forward, the grad_V reduction beside the grad_K contraction, the grad_K
            reduction beside the grad_Q one.  Level 2: also the K^T exchange is hidden, beside the window forward of the
            interior rows (whose windows touch no margin); the two edge strips follow."""
            lo_r, hi_r = ph.interior_rows()
            kt_ext, v_ext = ph.ext(0), ph.ext(1)
            if args.overlap >= 2:
                beside(lambda: ph.exchange(),
                       lambda: impl.band_nt(q[:, lo_r:hi_r], kt_ext, w, other_off=off + lo_r, seq=seq, out=a[:, lo_r:hi_r]))
                impl.band_nt(q[:, :lo_r], kt_ext, w, other_off=off, seq=seq, out=a[:, :lo_r])
                impl.band_nt(q[:, hi_r:], kt_ext, w, other_off=off + hi_r, seq=seq, out=a[:, hi_r:])
            else:
                ph.exchange(0)
                beside(lambda: ph.exchange(1), lambda: launch_list[0][1](kt_ext, v_ext))
            for _, fn in launch_list[1:4]:      # unwindow forward, grad_A, grad_V partial rows
                fn(kt_ext, v_ext)
            gv_rows = beside(lambda: ph.reduce(1)[0], lambda: launch_list[5][1](kt_ext, v_ext))   # grad_K partial rows
            gk_rows = beside(lambda: ph.reduce(0)[0], lambda: launch_list[4][1](kt_ext, v_ext))   # grad_Q
            return [gk_rows, gv_rows]

        def raw_step():
            if peer and side is not None:
                return overlapped_step()
            if peer:
                kt_ext, v_ext = ph.exchange()
                if seq_split:
                    # The six contractions as their DAG, the kernels of a level side by side on a share of the SMs each
                    # (a rank of an 8-GPU run has 7 row tiles per SM: the fixed cost of a launch counts):
                    #   level 1: window forward | grad_A          (half of the SMs each)
                    #   level 2: unwindow forward, grad_V | grad_Q, grad_K   (a quarter each)
                    la, lb, lc = (torch.cuda.Stream(device=dev) for _ in range(3))
                    half, quarter = sms_total // 2, sms_total // 4
                    la.wait_stream(stream)
                    with N_.cta_limits(half, 0):
                        with torch.cuda.stream(la):
                            launch_list[2][1](kt_ext, v_ext)        # grad_A
                        launch_list[0][1](kt_ext, v_ext)            # window forward
                    lb.wait_stream(stream)
                    lc.wait_stream(la)
                    with N_.cta_limits(quarter, 0):
                        with torch.cuda.stream(lb):
                            launch_list[3][1](kt_ext, v_ext)        # grad_V partial rows
                        launch_list[1][1](kt_ext, v_ext)            # unwindow forward
                        with torch.cuda.stream(lc):
                            launch_list[5][1](kt_ext, v_ext)        # grad_K partial rows
                        with torch.cuda.stream(la):
                            launch_list[4][1](kt_ext, v_ext)        # grad_Q
                    for x in (la, lb, lc):
                        stream.wait_stream(x)
                else:
                    contractions(kt_ext, v_ext)
                return ph.reduce()
            kt_ext, v_ext = halo([kt, v])   # views of the same storage every step: only the margins are written
            if graph is not None:
                graph.replay()
            else:
                contractions(kt_ext, v_ext)
            return unhalo([parts["gv"], parts["gk"]])

        def step():
            if peer and graph is not None:
                graph.replay()
                return None
            return raw_step()

        for _ in range(max(3, args.warmup)):
            step()
        stream.synchronize()
        l0 = N_.launch_count()
        grads = step()
        launches_per_step = N_.launch_count() - l0
        stream.synchronize()

        # ---- parity, outside the timed region: rank 0's rows against the unsharded kernels on the same seeded rows ----
        if parity and rank == 0:
            gk_l, gv_l = (grads[0], grads[1]) if peer else (grads[1], grads[0])
            result["parity"] = _seq_parity(torch, impl, dev, workload, world, dict(a=a, o=o, ga=ga, gq=gq, gk=gk_l, gv=gv_l),
                                           (qc, ktc, vc, goc))
        if not args.no_graph:
            g_ = torch.cuda.CUDAGraph()
            if peer:
                barrier()
                with torch.cuda.graph(g_, stream=stream):
                    raw_step()
            else:
                kt_ext, v_ext = halo([kt, v])
                stream.synchronize()
                with torch.cuda.graph(g_, stream=stream):
                    contractions(kt_ext, v_ext)
            graph = g_
            for _ in range(2):
                step()
            stream.synchronize()
        barrier()
        # five blocks of `steps` steps each, every block between two events; the MEDIAN block counts (a step is half a
        # millisecond and the ranks meet in every exchange: one late rank stretches a whole block)
        nblk = 5
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nblk)]
        with ClockSampler(dev.index) as clocks:
            for b0, b1 in evs:
                b0.record(stream)
                for _ in range(steps):
                    step()
                b1.record(stream)
            stream.synchronize()
        block_ms = sorted(b0.elapsed_time(b1) for b0, b1 in evs)
        barrier()

        # ---- per-launch durations: every rank issues the same launch, `reps` times, between two barriers ----
        per_launch = []
        reps = 5
        if peer:
            kt_ext, v_ext = ph.exchange()
            seq_launches = ([("halo_pull K^T+V margins", lambda k_, v_: ph.exchange())] + launch_list +
                            [("halo_pull grad_K+grad_V reduction", lambda k_, v_: ph.reduce())])
        else:
            kt_ext, v_ext = halo([kt, v])
            seq_launches = launch_list
        for name, fn in seq_launches:
            fn(kt_ext, v_ext)
            barrier()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record(stream)
            for _ in range(reps):
                fn(kt_ext, v_ext)
            k1.record(stream)
            stream.synchronize()
            per_launch.append(k0.elapsed_time(k1) * 1e3 / reps)
        barrier()
    status = N_.device_status()
    t = torch.tensor([block_ms[nblk // 2], float(status)] + per_launch + [block_ms[0], block_ms[-1]], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us = float(t[0]) * 1e3 / steps
    blocks_us = {"n": nblk, "steps_each": steps, "value_is": "median block, max over ranks",
                 "min_us": round(float(t[-2]) * 1e3 / steps, 1), "max_us": round(float(t[-1]) * 1e3 / steps, 1)}
    t = t[:-2]
    total_bytes, total_flops = algorithmic(B, M, N, w, e)
    peak, peak_kind = measured_peaks()
    result.update({
        "value_us": us, "n_gpus": world, "steps": steps, "workload": workload_name(workload), "rows_per_gpu": Ml,
        "partial_rows": ("own rows unrounded (fp32) until the neighbour's 16-bit rows are added (wmm_band_t_edges, wmm_halo_reduce_edges)"
                         if (peer and ph is not None and ph.with_edges) else "summed as 16-bit rows"),
        "contractions": ("DAG, kernels of a level side by side on a share of the SMs each (wmm_set_cta_limits)" if seq_split
                         else "one after the other, all SMs each"),
        "overlap": ("none: exchanges in stream order" if not (peer and side is not None) else
                    ("V exchange beside the window forward, grad_V / grad_K reductions beside the grad_K / grad_Q contractions"
                     if args.overlap == 1 else
                     "K^T and V exchange beside the window forward of the interior rows, reductions beside grad_K / grad_Q")
                    + "; %d SMs left to each exchange" % max(0, args.overlap_sms)),
        "exchange": ("peer memory: one kernel of the library per exchange" if peer else
                     "NCCL send/recv (torch.distributed)" if world > 1 else "none"),
        "halo_bytes_per_rank_step": 0 if world == 1 else 4 * 2 * B * w * N * e,  # K^T, V margins in; grad_K, grad_V partials in
        "launch": ("stream launches" if graph is None else "one cuda graph per step (exchanges and contractions)" if peer
                   else "cuda graph of the six contractions between two NCCL exchanges"),
        "launches_per_step": int(launches_per_step),
        "blocks": blocks_us,
        "per_launch_us_max_over_ranks": {name: round(float(x), 1) for (name, _), x in zip(seq_launches, t[2:].tolist())},
        "alg_MB": round(total_bytes / 1e6, 1),
        "frac_of_%s_hbm" % peak_kind: round(total_bytes / world / (us * 1e-6) / 1e9 / peak, 4),
        "device_status": int(t[1]), "clocks": clocks.summary(),
    })
    if world > 1:   # every rank returns the same dict (rank 0 holds the parity figures)
        box = [result if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        result = box[0]
    del ph
    return result

def run_seq_sharded(args, torch, impl, N_, rank, world, dev):
    """bench.py --shard seq (the default for --workload c4 on several GPUs): prints the sequence-sharded step as its own line."""
    r = measure_seq_sharded(args, torch, impl, N_, rank, world, dev, args.workload, args.steps)
    if r["device_status"] != 0:
        raise SystemExit("bench.py: a kernel abandoned a bounded wait; numbers are void")
    if rank == 0:
        B, M, N, w, dt, distn = WORKLOADS[args.workload]
        e = 2 if dt != "fp32" else 4
        total_bytes, total_flops = algorithmic(B, M, N, w, e)
        us = r["value_us"]
        line = {
            "metric": "fwd+bwd window+unwindow us (%s, sequence-sharded)" % args.workload, "value": us, "unit": "us", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": us / 1e3, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": dt.replace("fp", "f"), "data": "synthetic",
            "config": {"workload": r["workload"], "parallelism": "sequence-sharded x%d, w-row halo exchange" % world,
                       "rows_per_gpu": r["rows_per_gpu"], "halo_bytes_per_rank_step": r["halo_bytes_per_rank_step"],
                       "exchange": r["exchange"], "launch": r["launch"],
                       "l2": "no flush: one step touches %.0f MB per GPU" % (total_bytes / world / 1e6)},
            "step_roofline": {"alg_MB": r["alg_MB"], "alg_GFLOP": round(total_flops / 1e9, 1),
                              "achieved_GBps": round(total_bytes / (us * 1e-6) / 1e9, 1),
                              **{k: v for k, v in r.items() if k.startswith("frac_of_")}},
            "per_launch_us_max_over_ranks": r["per_launch_us_max_over_ranks"], "parity_vs_unsharded": r.get("parity"),
            "gpu_launches": int(r["launches_per_step"] * args.steps * r["blocks"]["n"]), "clocks": r["clocks"],
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_cuda"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--blocks", type=int, default=0, help="timed blocks of --steps steps each (0: enough for about a second, at least 50)")
    ap.add_argument("--no-reference-cuda", action="store_true", help="skip the short run of the reference's CUDA kernels beside the headline")
    ap.add_argument("--overlap", type=int, default=0, choices=[0, 1, 2],
                    help="sequence-sharded step: 0 = exchanges in stream order (default: fastest measured); 1 = the V exchange "
                         "and both reductions on a side stream beside contractions that do not need them; 2 = also the K^T "
                         "exchange, beside the window forward of the interior rows")
    ap.add_argument("--edges", type=int, default=1, choices=[0, 1],
                    help="sequence-sharded step: 1 = add the neighbour's partial grad_K / grad_V rows to this rank's unrounded fp32 "
                         "rows; 0 = sum 16-bit rows (one rounding more)")
    ap.add_argument("--overlap-sms", type=int, default=8,
                    help="SMs a contraction leaves to the exchange that runs beside it (0: no caps)")
    ap.add_argument("--no-seq-extra", action="store_true", help="on several GPUs: skip the sequence-sharded config 4 step reported beside the headline")
    ap.add_argument("--tf32", action="store_true", help="fp32 workloads: multiply on the tensor cores as tf32 (WMM_FLAG_TF32) instead of the exact-order kernels")
    ap.add_argument("--sm-split", default="auto",
                    help="CTA caps for the five kernels of the step's DAG (window fwd, grad_A, unwindow fwd, grad_V, window bwd), "
                         "'off', or 'auto': kernels of one level share the SMs when a GPU has fewer than 16 row tiles per SM")
    ap.add_argument("--branches", type=int, default=2, choices=[1, 2], help="capture the step as one chain (1) or with its real dependencies (2)")
    ap.add_argument("--no-graph", action="store_true", help="launch the six kernels on the stream instead of a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override B of the workload (small cases for profiling)")
    ap.add_argument("--rows", type=int, default=0, help="override M of the workload (e.g. the rows of a shard of a larger run)")
    ap.add_argument("--k-layout", default="view", choices=["view", "bnm"],
                    help="K as a transposed view of a (B,M,N) tensor (default) or as a contiguous (B,N,M) tensor")
    ap.add_argument("--shard", default="auto", choices=["auto", "batch", "seq"],
                    help="multi-GPU partitioning: batch entries (default) or sequence rows with halo exchange (default for c4)")
    ap.add_argument("--e2e-chunks", type=int, default=0, help="batch chunks of the host-buffer leg (0: from the batch per GPU)")
    ap.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="sequence-sharded mode: halo exchange through peer memory (one library kernel) or NCCL send/recv")
    ap.add_argument("--block", default="auto", choices=["auto", "on", "off"],
                    help="also time the attention block with the band softmax between the operators (auto: config 5)")
    args = ap.parse_args()
    import torch

    if args.batch > 0:
        B, M, N, w, dt, dist = WORKLOADS[args.workload]
        WORKLOADS[args.workload] = (args.batch, M, N, w, dt, dist)
    if args.rows > 0:
        B, M, N, w, dt, dist = WORKLOADS[args.workload]
        WORKLOADS[args.workload] = (B, args.rows, N, w, dt, dist)
    if args.impl == "reference":
        run_reference(args, torch)
    elif args.impl == "reference_cuda":
        run_reference_cuda(args, torch)
    else:
        run_ours(args, torch)


if __name__ == "__main__":
    main()
