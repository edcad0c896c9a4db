"""Benchmark of the indexed delta matmul path (sbmm) on synthetic Llama-shaped data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload at N = 1 (`config.workload` = "sbmm-decode-64x4096x4096-g128"): 64 int4 2:4 deltas of
4096 x 4096 with group-128 fp16 scales resident in HBM; one step = one batch of 128 fp16 tokens
~N(0,1), one int32 delta index per token uniform over [0, 64) with 10% set to -1, pushed
through `sbmm_4bit_2_4_native` (router + row gather + grouped kernel).  At N > 1 every rank holds
its own 64-delta shard of a 64*N-delta set and 128 tokens whose indices range over the whole set;
tokens are exchanged with all-to-all (weak scaling).

Prints ONE JSON line: tokens/s with inputs resident on the device (`value`), the same through the
public API from pinned host buffers (`e2e`), the roofline of the grouped kernel measured with CUDA
events on the launching stream, the CPU baseline (the torch fp32 dequantise-then-matmul path on
the host cores, bounded sample), and the clocks sampled during the timed region.
`--impl reference` times only that CPU path and prints it in the same format.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

D_PER_GPU, K, N_OUT, TOKENS, GROUP = 64, 4096, 4096, 128, 128
BYTES_PER_DELTA = K * N_OUT // 4 + K * N_OUT // 8 + (K // GROUP) * N_OUT * 2   # codes + metadata + scales
METRIC, UNIT = "sbmm_tokens_per_s", "tokens/s"
WORKLOAD = "sbmm-decode-64x4096x4096-g128"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def describe_parallelism(world, exchange_kind):
    if world == 1:
        return "single GPU"
    how = ("rows and results stored straight into the owner's symmetric-memory buffers over NVLink by the pack kernel "
           "and the grouped kernel's epilogue, two cross-GPU barriers per step" if exchange_kind == "p2p" else
           "two equal-split NCCL all-to-alls per step (rows + ids out, result rows back)")
    return f"deltas sharded by id over {world} GPUs; {how}; no host synchronisation"


def make_indices(seed, tokens, num_deltas):
    rng = np.random.default_rng(seed)
    idx = rng.integers(0, num_deltas, tokens)
    idx[rng.choice(tokens, size=tokens // 10, replace=False)] = -1
    return idx.astype(np.int32)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms while running."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU baseline
class CpuPath:
    """The reference has no CPU kernel for this path; its torch check path is
    `sbmm_16bit_forloop` on dequantised weights (triteia/python/ops/matmul/sbmm.py:7-23).  Here: fp32
    torch matmul with all host threads on a bounded sample of the workload — `num_sample_deltas`
    deltas with the tokens that select them.  The sample is dequantised once by the oracle's
    decoder (untimed); one pass = one per-delta matmul loop over the sample."""

    def __init__(self, num_sample_deltas=6, seed=0):
        from oracle import delta_format as fmt
        from triteia_b200.ops.utils.generator import random_packed_deltas

        torch.set_num_threads(os.cpu_count() or 1)
        self.cores = torch.get_num_threads()
        self.n = num_sample_deltas
        qs, metas, ss = random_packed_deltas(self.n, K, N_OUT, groupsize=GROUP, device="cpu", seed=seed)
        self.weights = [torch.from_numpy(fmt.dequantize(qs[d].numpy(), metas[d].numpy(), ss[d].numpy())
                                         .astype(np.float32)) for d in range(self.n)]
        idx = make_indices(seed, TOKENS, D_PER_GPU)
        self.x = torch.randn(TOKENS, K, generator=torch.Generator().manual_seed(seed)).half().float()
        self.rows = [np.flatnonzero(idx == d) for d in range(self.n)]
        self.tokens = int(sum(len(r) for r in self.rows))
        self.y = torch.zeros(TOKENS, N_OUT)

    def one_pass(self):
        for d, r in enumerate(self.rows):
            if len(r):
                self.y[r] += self.x[r] @ self.weights[d]

    def timed(self, passes, warmup=1):
        for _ in range(warmup):
            self.one_pass()
        t0 = time.perf_counter()
        for _ in range(passes):
            self.one_pass()
        dt = (time.perf_counter() - t0) / passes
        return {"value": self.tokens / dt, "unit": UNIT, "cores": self.cores, "kind": "port",
                "sample": f"{self.n} of {D_PER_GPU} deltas with their {self.tokens} tokens, fp32 torch matmul on "
                          f"dequantised weights, mean of {passes} passes ({dt * 1e3:.1f} ms each), dequantisation untimed",
                "seconds_per_pass": dt, "tokens_in_sample": self.tokens}


def cpu_baseline():
    return CpuPath(num_sample_deltas=16).timed(passes=600, warmup=3)   # about 10 s of host work


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    path = CpuPath()
    base = path.timed(passes=max(1, args.steps), warmup=max(1, args.warmup))
    v = base["value"]
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": base["seconds_per_pass"] * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": "the reference ships no CPU kernel for this path; this is its "
                       "torch check path (dequantised weights, per-delta fp32 matmul) on the host cores, one step = "
                       "one pass over a bounded sample"},
            "cpu_baseline": base,
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# --------------------------------------------------------------------------- GPU arm
def time_steps(fn, steps, flush):
    """Per-step CUDA-event timing on the current stream, L2 flushed (untimed) before every step."""
    times = []
    for _ in range(steps):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return times


def run_gpu_arm(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    import triteia_b200.ops as ops
    from triteia_b200 import _lib, sharded
    from triteia_b200.ops.matmul.sbmm import sbmm_indexed, _segments

    total_deltas = D_PER_GPU * world
    qs, metas, ss = ops.random_packed_deltas(D_PER_GPU, K, N_OUT, groupsize=GROUP, device=dev, seed=1000 + rank)
    idx_np = make_indices(rank, TOKENS, total_deltas)
    x_host = torch.randn(TOKENS, K, generator=torch.Generator().manual_seed(rank)).half().pin_memory()
    idx_host = torch.from_numpy(idx_np).pin_memory()
    y_host = torch.empty(TOKENS, N_OUT, dtype=torch.float16).pin_memory()
    x_dev, idx_dev = x_host.to(dev), idx_host.to(dev)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flush_src = torch.zeros(64 << 20, dtype=torch.int32, device=dev)

    def flush():
        # Write 256 MiB (evicts everything), then read another 256 MiB so that the lines left in
        # L2 are clean: a timed step must not pay for writing back the flush's own dirty lines.
        flush_buf.zero_()
        flush_src.sum()

    if world == 1:
        step_resident = lambda: ops.sbmm_4bit_2_4_native(qs, x_dev, metas, ss, idx_dev)
        launches_per_step = 3   # router, row gather, grouped kernel
    else:
        # Peer-to-peer exchange over CUDA symmetric memory when the box offers it, else NCCL all-to-all.
        exchange_kind = os.environ.get("TRB_EXCHANGE", "p2p")
        try:
            exchange = sharded.FixedCapacityExchange(TOKENS, K, N_OUT, dev, backend=exchange_kind, qweights=qs,
                                                     metas=metas, scales=ss)
        except Exception as e:   # symmetric memory unavailable
            if rank == 0:
                print(f"bench.py: p2p exchange unavailable ({e}); using NCCL all-to-all", file=sys.stderr)
            exchange_kind = "cuda"
            exchange = sharded.FixedCapacityExchange(TOKENS, K, N_OUT, dev, backend="cuda", qweights=qs, metas=metas,
                                                     scales=ss)
        step_resident = lambda: exchange(x_dev, idx_dev)
        launches_per_step = 5 if exchange_kind == "p2p" else 6   # plan + pack, router + gather + grouped kernel (+ combine)

    def step_e2e():
        xd = x_host.to(dev, non_blocking=True)
        idd = idx_host.to(dev, non_blocking=True)
        if world == 1:
            y = ops.sbmm_4bit_2_4_native(qs, xd, metas, ss, idd)
        else:
            y = exchange(xd, idd)
        y_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step_resident()
        step_e2e()
    barrier()

    class E2ESlot:
        """One in-flight end-to-end step: pinned host buffers, device staging, a stream and a CUDA
        graph of [copy x and ids in, the public op, copy y out]."""

        def __init__(self):
            self.x_host, self.idx_host = x_host.clone().pin_memory(), idx_host.clone().pin_memory()
            self.y_host = torch.empty(TOKENS, N_OUT, dtype=torch.float16).pin_memory()
            self.x_dev, self.idx_dev = torch.empty_like(x_dev), torch.empty_like(idx_dev)
            self.stream = torch.cuda.Stream()
            self.graph = None

        def body(self):
            self.x_dev.copy_(self.x_host, non_blocking=True)
            self.idx_dev.copy_(self.idx_host, non_blocking=True)
            if world == 1:
                y = ops.sbmm_4bit_2_4_native(qs, self.x_dev, metas, ss, self.idx_dev)
            else:
                y = exchange(self.x_dev, self.idx_dev)
            self.y_host.copy_(y, non_blocking=True)
            return y

        def capture(self):
            with torch.cuda.stream(self.stream):
                self.body()
            self.stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream):
                self.keep = self.body()
            self.graph = g

        def launch(self):
            with torch.cuda.stream(self.stream):
                if self.graph is not None:
                    self.graph.replay()
                else:
                    self.body()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_wall0 = time.perf_counter()
    # Timed region of `value`: exactly K steps bracketed by barrier + synchronize, CUDA events on the
    # launching stream, max over ranks below.  No flush inside the bracket: every step streams the
    # touched deltas (~360 MB per GPU), far more than the 126 MB L2, and they carry an evict-first hint.
    # One step is captured into a CUDA graph (the library calls neither allocate nor synchronise) and
    # replayed K times, so the host's launch cost is off the device timeline; --eager disables this.
    launch_mode = "eager"
    run_step = step_resident
    if not args.eager:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_resident()
            torch.cuda.current_stream().wait_stream(side)
            barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_out = step_resident()
            barrier()
            graph.replay()
            barrier()
            run_step, launch_mode = graph.replay, "cuda-graph replay of one captured step"
        except Exception as e:   # capture not possible: keep the eager path
            if rank == 0:
                print(f"bench.py: graph capture failed ({e}); timing eager launches", file=sys.stderr)
            run_step = step_resident
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        run_step()
    ev1.record()
    ev1.synchronize()
    barrier()
    times = [ev0.elapsed_time(ev1) / args.steps]
    # end-to-end latency of one step: host buffers in, host buffer out, wall clock around a stream sync
    e2e_times = []
    for _ in range(args.steps):
        flush()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        step_e2e()
        e2e_times.append((time.perf_counter() - t0) * 1e3)
    barrier()
    # end-to-end throughput: K steps, every one copying its inputs in from pinned host memory and its
    # result back; at N = 1 three steps are in flight on three streams so the copies of one overlap the
    # kernels of the other (the host waits for a slot's previous result before it reuses the slot).
    # With the cross-GPU exchange one step is in flight: its buffers and barriers are single.
    # No flush: every step streams the touched deltas, far more than the L2.
    slots = [E2ESlot() for _ in range(int(os.environ.get("TRB_E2E_SLOTS", "3")) if world == 1 else 1)]
    e2e_mode = "eager"
    if not args.eager:
        try:
            for sl in slots:
                sl.capture()
            e2e_mode = "cuda-graph replay"
        except Exception as e:
            if rank == 0:
                print(f"bench.py: e2e graph capture failed ({e}); eager e2e steps", file=sys.stderr)
            for sl in slots:
                sl.graph = None
    barrier()
    for i in range(2 * len(slots)):
        slots[i % len(slots)].launch()
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        sl = slots[i % len(slots)]
        sl.stream.synchronize()      # the slot's previous result is in host memory
        sl.launch()
    for sl in slots:
        sl.stream.synchronize()
    t_e2e_pipe = (time.perf_counter() - t0) * 1e3 / args.steps
    barrier()

    # dominant kernel alone (grouped kernel through the segment-list entry point), rank-local
    order = torch.argsort(idx_dev.long() % world if world > 1 else idx_dev, stable=True)
    if world == 1:
        idx_sorted = idx_dev[order].contiguous()
        x_sorted = x_dev[order].contiguous()
        uniq, starts, counts = _segments(idx_sorted)
        touched = int(uniq.numel())
    else:
        # what this rank's grouped kernel sees in a step: the tokens of EVERY rank whose delta it owns
        # (all ranks draw their ids from seed = rank, so they can be restated here without a collective)
        all_idx = torch.from_numpy(np.concatenate([make_indices(r, TOKENS, total_deltas) for r in range(world)])).to(dev)
        mine = (all_idx >= 0) & (all_idx % world == rank)
        loc = torch.div(all_idx[mine], world, rounding_mode="floor")
        o2 = torch.argsort(loc, stable=True)
        idx_sorted = loc[o2].int().contiguous()
        x_sorted = x_dev.repeat(world, 1)[mine][o2].contiguous()
        uniq, starts, counts = _segments(idx_sorted)
        touched = int(uniq.numel())
    y_k = torch.empty(x_sorted.shape[0], N_OUT, dtype=torch.float16, device=dev)
    ws = torch.zeros(max(touched, 1), N_OUT // 8, dtype=torch.int32, device=dev)
    # the segment-list entry point with working memory for the tail K split (what the fused step's
    # grouped kernel runs with); TRB_KSPLIT=0 in the environment turns the split off
    ks_bytes = _lib.lib.trb_sbmm_ksplit_bytes()
    ks_buf = torch.zeros(ks_bytes, dtype=torch.uint8, device=dev)

    def kern():
        if touched:
            _lib.check(_lib.lib.trb_sbmm_2_4_ksplit(
                _lib.ptr(x_sorted), _lib.ptr(qs), _lib.ptr(metas), _lib.ptr(y_k), _lib.ptr(ss), _lib.ptr(uniq),
                _lib.ptr(starts), _lib.ptr(counts), N_OUT, x_sorted.shape[0], K, touched, GROUP, _lib.dev_of(y_k),
                _lib.stream_of(y_k), _lib.ptr(ks_buf), ks_bytes), "sbmm_2_4_ksplit")
    for _ in range(3):
        kern()
    k_times = time_steps(kern, args.steps, flush)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    wall_s = time.perf_counter() - t_wall0

    t_step = statistics.mean(times)
    t_e2e = statistics.mean(e2e_times)
    t_kern = statistics.mean(k_times)
    if world > 1:
        t = torch.tensor([t_step, t_e2e, t_e2e_pipe], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_step, t_e2e, t_e2e_pipe = t.tolist()
    status = _lib.device_status(local_rank)

    if rank == 0:
        peak, peak_src = peaks()
        alg_bytes = touched * BYTES_PER_DELTA + x_sorted.numel() * 2 + y_k.numel() * 2 + touched * 12
        achieved = alg_bytes / (t_kern * 1e-3) / 1e9
        tokens_total = TOKENS * world
        line = {
            "metric": METRIC, "value": tokens_total / (t_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": t_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "deltas_per_gpu": D_PER_GPU, "tokens_per_gpu": TOKENS, "k": K, "n": N_OUT,
                       "groupsize": GROUP, "index_law": "uniform over all deltas, 10% -1, unsorted",
                       "distinct_local_deltas_touched_rank0": touched, "launch": launch_mode,
                       "l2": f"inputs larger than L2: every step streams {touched * BYTES_PER_DELTA / 1e6:.0f} MB of packed "
                             "deltas (126 MB L2, evict-first loads); the kernel-alone roofline leg and the e2e leg "
                             "additionally flush L2 before every step (256 MiB memset + 256 MiB read, untimed)",
                       "parallelism": describe_parallelism(world, exchange_kind if world > 1 else None)},
            "e2e": {"value": tokens_total / (t_e2e_pipe * 1e-3), "unit": UNIT, "ms_per_step": t_e2e_pipe,
                    "h2d_bytes_per_step": int(x_host.numel() * 2 + idx_host.numel() * 4),
                    "d2h_bytes_per_step": int(y_host.numel() * 2),
                    "steps_in_flight": len(slots), "launch": e2e_mode,
                    "latency_ms_one_step": t_e2e, "latency_tokens_per_s": tokens_total / (t_e2e * 1e-3),
                    "note": "sbmm_4bit_2_4_native from pinned host buffers, every step copies x and ids in and y "
                            "out; packed deltas stay resident (model state); latency_* is one step alone after "
                            "an L2 flush"},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_src, "kernel": "delta_gemm_kernel", "kernel_ms": t_kern,
                         "algorithmic_bytes": alg_bytes,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this
                         # launch (profiles/delta_gemm_kernel_sbmm-decode-64x4096x4096-g128.md);
                         # only known for the single-GPU seed (56 deltas touched).
                         "traffic": 374398720 if (world == 1 and touched == 56) else None},
            "clocks": clocks, "device_status": status, "wall_s": wall_s,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- other workloads (1 GPU)
def _event_time(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / steps


def _e2e_time(fn, host_inputs, dev, steps):
    """Wall-clock ms per step of fn(*device copies of host_inputs) with the copies in from pinned host
    memory and the copy of the result back inside the timed region (one step in flight)."""
    pinned = [t.cpu().pin_memory() for t in host_inputs]
    out_host = None

    def one():
        nonlocal out_host
        ins = [t.to(dev, non_blocking=True) for t in pinned]
        y = fn(*ins)
        if out_host is None:
            out_host = torch.empty(y.shape, dtype=y.dtype).pin_memory()
        out_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(2):
        one()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) * 1e3 / steps
    return dt, int(sum(t.numel() * t.element_size() for t in pinned)), int(out_host.numel() * out_host.element_size())


def run_prefill(args):
    """The prefill configuration: 32 deltas 5120x13824 (or 13824x5120 with --shape down), group 128, 8192 tokens in
    16 contiguous segments of 512 (deltas 0..15); optional SGMV rank-64 LoRA on the same segments.
    Tensor-bound: flops are dense-equivalent 2*T*K*N (the reference's convention, bench_sbmm.py:17)."""
    import triteia_b200.ops as ops
    from triteia_b200 import _lib
    from triteia_b200.capi import sbmm_2_4

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    k, n = (5120, 13824) if args.shape == "up" else (13824, 5120)
    T, D, SEG, R = 8192, 32, 16, 64
    qs, metas, ss = ops.random_packed_deltas(D, k, n, groupsize=128, device=dev, seed=1)
    g = torch.Generator(dev).manual_seed(0)
    x = torch.randn(T, k, device=dev, generator=g).half()
    idx = torch.arange(SEG, device=dev, dtype=torch.int32).repeat_interleave(T // SEG)
    A = (torch.randn(SEG, k, R, device=dev, generator=g) / k ** 0.5).half()
    B = (torch.randn(SEG, R, n, device=dev, generator=g) / R ** 0.5).half()
    uniq = torch.arange(SEG, device=dev, dtype=torch.int32)
    counts = torch.full((SEG,), T // SEG, device=dev, dtype=torch.int32)
    starts = (uniq * (T // SEG)).int()
    yk = torch.empty(T, n, dtype=torch.float16, device=dev)
    ws = torch.zeros(SEG, n // 8, dtype=torch.int32, device=dev)
    sampler = ClockSampler(0)
    sampler.start()
    t_step = _event_time(lambda: ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx), args.steps, max(3, args.warmup))
    t_kern = _event_time(lambda: sbmm_2_4(x, qs, metas, yk, ss, uniq, ws, starts, counts), args.steps, 3)
    t_lora = _event_time(lambda: ops.lora_sgmv(A, B, x, idx), max(1, args.steps // 4), 2)
    t_e2e, h2d, d2h = _e2e_time(lambda xd, idd: ops.sbmm_4bit_2_4_native(qs, xd, metas, ss, idd), [x, idx], dev,
                                max(2, args.steps // 4))
    clocks = sampler.stop()
    flops = 2.0 * T * k * n
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    dense = float(json.load(open(path))["bf16_tflops"]) if os.path.exists(path) else 1590.0
    ach = flops / (t_kern * 1e-3) / 1e12
    line = {"metric": METRIC, "value": T / (t_step * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": t_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"sbmm-prefill-32x{k}x{n}-g128-8192tok-16seg", "sgmv_rank64_ms": t_lora,
                       "l2": "inputs larger than L2 (442 MB of packed deltas touched, 84-226 MB of activations)"},
            "e2e": {"value": T / (t_e2e * 1e-3), "unit": UNIT, "ms_per_step": t_e2e, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "note": "one step in flight; bound by the host link (x in, y out)"},
            "gpu_launches": 3 * args.steps,
            "roofline": {"bound": "tensor", "achieved": ach, "peak": 2 * dense, "unit": "TFLOP/s", "frac": ach / (2 * dense),
                         "peak_source": "2 x measured dense bf16 burst (MEASURED_PEAKS.json has no sparse entry)",
                         "frac_of_dense_peak": ach / dense, "kernel": ("delta_gemm_tc_kernel" if os.environ.get("TRB_TC_DENSE") == "1" else "delta_gemm_tcsp_kernel"), "kernel_ms": t_kern,
                         "algorithmic_flops": flops, "traffic": None},
            "clocks": clocks, "device_status": _lib.device_status(0)}
    print(json.dumps(line))


def run_ldmm(args):
    """The ldmm configuration: fp16 base [11008, 4096] ~N(0, 0.02), 32 per-channel deltas 4096 -> 11008, 32 LoRA
    adapters of rank 16, 256 decode tokens, ids Zipf(1.2) over the 64 ids through a seeded permutation."""
    import triteia_b200.ops as ops
    from triteia_b200 import _lib

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    k, n, T, M, D, R = 4096, 11008, 256, 32, 32, 16
    qs, metas, ss = ops.random_packed_deltas(D, k, n, groupsize=-1, device=dev, seed=2)
    g = torch.Generator(dev).manual_seed(0)
    base = (torch.randn(n, k, device=dev, generator=g) * 0.02).half()
    A = (torch.randn(M, k, R, device=dev, generator=g) / k ** 0.5).half()
    B = (torch.randn(M, R, n, device=dev, generator=g) / R ** 0.5).half()
    x = torch.randn(T, k, device=dev, generator=g).half()
    rng = np.random.default_rng(0)
    p = np.arange(1, M + D + 1, dtype=np.float64) ** -1.2
    ids = rng.permutation(M + D)[rng.choice(M + D, T, p=p / p.sum())].astype(np.int32)
    idx = torch.from_numpy(ids).to(dev)
    touched_d = len({int(i) for i in ids if i >= M})
    touched_l = len({int(i) for i in ids if 0 <= i < M})
    sampler = ClockSampler(0)
    sampler.start()
    t_step = _event_time(lambda: ops.ldmm(idx, x, A, B, qs, metas, ss, base_weight=base), args.steps, max(3, args.warmup))
    t_base = _event_time(lambda: torch.matmul(x, base.t()), args.steps, 3)
    t_e2e, h2d, d2h = _e2e_time(lambda idd, xd: ops.ldmm(idd, xd, A, B, qs, metas, ss, base_weight=base), [idx, x], dev,
                                args.steps)
    clocks = sampler.stop()
    alg = (n * k * 2 + touched_d * (k * n // 4 + k * n // 8 + n * 2) + touched_l * (k * R + R * n) * 2 + T * k * 2 + T * n * 2)
    peak, peak_src = peaks()
    ach = alg / (t_step * 1e-3) / 1e9
    line = {"metric": "ldmm_tokens_per_s", "value": T / (t_step * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": t_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "ldmm-256tok-4096x11008-32deltas-32lora-r16-zipf1.2", "deltas_touched": touched_d,
                       "adapters_touched": touched_l, "base_gemm_ms": t_base,
                       "l2": f"inputs larger than L2 ({alg / 1e6:.0f} MB streamed per step)"},
            "e2e": {"value": T / (t_e2e * 1e-3), "unit": UNIT, "ms_per_step": t_e2e, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "note": "one step in flight"},
            "gpu_launches": 4 * args.steps,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "peak_source": peak_src, "kernel": "whole step (library base GEMM + LoRA + router + gather + grouped kernel)",
                         "algorithmic_bytes": alg, "traffic": None},
            "clocks": clocks, "device_status": _lib.device_status(0)}
    print(json.dumps(line))


def run_stack(args):
    """The linear-stack configuration: L layers of the seven Llama-2-7B linears, 128 deltas sharded by
    id over the ranks, 512 tokens in all (512 / N per rank), delta id ~ Zipf(1.5); one dispatch and one
    combine per pass.  Strong scaling: the total work is fixed as N grows."""
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev) if world > 1 else dist.init_process_group(
        "nccl", init_method="tcp://127.0.0.1:%d" % (29700 + os.getpid() % 200), rank=0, world_size=1, device_id=dev)
    from triteia_b200 import _lib, stack

    D, T_total, L, group = 128, 512, args.layers, 128
    T = T_total // world
    t0 = time.perf_counter()
    shard = stack.random_stack_shard(D, rank, world, L, groupsize=group, device=dev, seed=3)
    local = stack.DeltaStackShard(shard)
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t0
    rng = np.random.default_rng(7)
    p = np.arange(1, D + 1, dtype=np.float64) ** -1.5
    ids_all = rng.choice(D, T_total, p=p / p.sum()).astype(np.int32)          # the same batch for every N
    g = torch.Generator().manual_seed(7)
    x4096_all = torch.randn(T_total, 4096, generator=g).half()
    x11008_all = torch.randn(T_total, 11008, generator=g).half()
    sl = slice(rank * T, (rank + 1) * T)
    host = {4096: x4096_all[sl].contiguous().pin_memory(), 11008: x11008_all[sl].contiguous().pin_memory()}
    idx_host = torch.from_numpy(ids_all[sl].copy()).pin_memory()
    xs = {k: v.to(dev) for k, v in host.items()}
    idx = idx_host.to(dev)
    y_host = torch.empty(T, 4096, dtype=torch.float16).pin_memory()
    cs_host = torch.empty(T, dtype=torch.float32).pin_memory()

    def step():
        return stack.stack_sharded(xs, idx, local, 4096)

    def step_e2e():
        xd = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
        idd = idx_host.to(dev, non_blocking=True)
        y, cs = stack.stack_sharded(xd, idd, local, 4096)
        y_host.copy_(y, non_blocking=True)
        cs_host.copy_(cs, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    step_e2e()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    ev1.synchronize()
    barrier()
    t_step = ev0.elapsed_time(ev1) / args.steps
    tw = time.perf_counter()
    for _ in range(args.steps):
        step_e2e()
    t_e2e = (time.perf_counter() - tw) * 1e3 / args.steps
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    mine = set(range(rank, D, world))
    touched_local = len({int(i) for i in ids_all if int(i) in mine})
    per_layer = sum(k * n // 4 + k * n // 8 + (k // group) * n * 2 for _, k, n in stack.LLAMA_7B_LINEARS)
    t = torch.tensor([t_step, t_e2e, float(touched_local)], device=dev, dtype=torch.float64)
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        t_step, t_e2e, touched_max = tmax.tolist()
    else:
        touched_max = touched_local
    status = _lib.device_status(local_rank)
    if rank == 0:
        peak, peak_src = peaks()
        alg = touched_max * per_layer * L          # the busiest rank's delta bytes: what bounds the pass
        ach = alg / (t_step * 1e-3) / 1e9
        print(json.dumps({
            "metric": "stack_tokens_per_s", "value": T_total / (t_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": t_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"stack-llama7b-linears-{L}layers-128deltas-512tok-zipf1.5-g128", "layers": L,
                       "tokens_total": T_total, "linears_per_pass": 7 * L, "ms_per_layer": t_step / L,
                       "distinct_deltas_touched": len(set(int(i) for i in ids_all)),
                       "touched_on_busiest_rank": int(touched_max), "build_s": t_build,
                       "l2": "inputs larger than L2 (every linear streams its touched deltas: 6-17 MB each, all distinct)",
                       "parallelism": "single GPU" if world == 1 else
                       f"deltas sharded by id over {world} GPUs; one NCCL all-to-all dispatch of [x4096|x11008] rows + ids "
                       "and one combine (last output + checksums) per pass; one host read of the counts per pass"},
            "e2e": {"value": T_total / (t_e2e * 1e-3), "unit": UNIT, "ms_per_step": t_e2e,
                    "h2d_bytes_per_step": int(T * (4096 + 11008) * 2 + T * 4), "d2h_bytes_per_step": int(T * 4096 * 2 + T * 4)},
            "gpu_launches": 14 * L * args.steps,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "peak_source": peak_src, "kernel": "whole pass on the busiest rank (grouped kernel + row checksum per linear)",
                         "algorithmic_bytes": alg, "traffic": None},
            "clocks": clocks, "device_status": status}))
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (profiling runs)")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of CUDA-graph replays")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "ldmm", "stack"],
                    help="decode = the headline sbmm configuration (default); prefill / ldmm: 1-GPU extra legs; "
                         "stack = the sharded linear stack (any number of GPUs, strong scaling)")
    ap.add_argument("--layers", type=int, default=8, help="stack: number of layers (8 fits one GPU: 78 GB of deltas)")
    ap.add_argument("--shape", default="up", choices=["up", "down"], help="prefill: 5120x13824 (up) or 13824x5120")
    args = ap.parse_args()
    if args.workload == "prefill":
        return run_prefill(args)
    if args.workload == "ldmm":
        return run_ldmm(args)
    if args.workload == "stack":
        return run_stack(args)
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
