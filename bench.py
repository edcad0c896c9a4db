"""Benchmark of the indexed delta matmul path (sbmm / ldmm) on synthetic Llama-shaped data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (`config.workload` = "sbmm-decode-64x4096x4096-g128"): 64 int4 2:4 deltas of
4096 x 4096 with group-128 fp16 scales resident in HBM; one step = one batch of 128 fp16 tokens
~N(0,1), one int32 delta index per token uniform over [0, 64) with 10% set to -1, pushed
through `sbmm_4bit_2_4_native` (router + row gather + grouped kernel).  At N > 1 every rank holds
its own 64-delta shard of a 64*N-delta set and 128 tokens whose indices range over the whole set;
tokens are exchanged between the ranks (weak scaling).

Prints ONE JSON line: tokens/s with inputs resident on the device (`value`; the K-step bracket is
repeated and the median reported, with p10 / p90), the same through the public API from pinned
host buffers (`e2e`, results compared with the CPU oracle after the timed loop), the roofline of
the grouped kernel measured with CUDA events on the launching stream, the CPU baseline (the torch
fp32 dequantise-then-matmul path on the host cores, bounded sample), the clocks sampled during the
timed region, and `legs`: the other configurations of the path, each with its own roofline —
`ldmm` (base + LoRA + delta, 256 decode tokens), `prefill_up` / `prefill_down` (8192 tokens, tensor
bound) at N = 1, and `stack` (the sharded Llama-2-7B linear stack, strong scaling) at every N.
`--impl reference` times only the CPU path and prints it in the same format; that arm imports
nothing of the product.
"""
import argparse
import gc
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
TOL = 1e-2          # max_n |y - ref| / max_n |ref| per output row against the fp32 oracle


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, 1590.0, "fallback (6.65 TB/s, 1.59 PFLOP/s: earlier measurement on this pool)"


def recorded_traffic(key, units):
    """DRAM bytes per launch of a kernel from the ncu capture recorded in profiles/traffic.json,
    scaled by the units (touched deltas) of this launch; None if no capture is recorded."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        rec = json.load(f).get(key)
    if not rec:
        return None
    return int(round(rec["dram_bytes_per_launch"] * units / rec["units_in_capture"]))


def make_indices(seed, tokens, num_deltas):
    rng = np.random.default_rng(seed)
    idx = rng.integers(0, num_deltas, tokens)
    idx[rng.choice(tokens, size=tokens // 10, replace=False)] = -1
    return idx.astype(np.int32)


def spread(times):
    """median / p10 / p90 / mean of a list of per-step times (ms)."""
    s = sorted(times)
    pick = lambda q: s[min(len(s) - 1, max(0, int(round(q * (len(s) - 1)))))]
    return {"median_ms": statistics.median(s), "p10_ms": pick(0.1), "p90_ms": pick(0.9), "mean_ms": statistics.mean(s),
            "brackets": len(s)}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms while running."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,utilization.gpu")

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
        sm, sm_load, mx, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            try:
                if len(r) > 6 and float(r[6]) >= 50:
                    sm_load.append(float(r[0]))
            except ValueError:
                pass
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        under = sm_load if sm_load else sm
        return {"sm_mhz": statistics.median(under) if under else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "samples_under_load": len(sm_load), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU baseline
class CpuPath:
    """The reference has no CPU kernel for this path; its torch check path is
    `sbmm_16bit_forloop` on dequantised weights (triteia/python/ops/matmul/sbmm.py:7-23).  Here: the
    oracle's fp32 statement of it (oracle.ops.sbmm_dense_f32, torch matmul with all host threads) on a
    bounded sample of the workload — `num_sample_deltas` deltas with the tokens that select them.
    The sample's packed deltas are drawn in the wire format with numpy and dequantised once by the
    oracle's decoder (untimed).  Nothing of the product is imported."""

    def __init__(self, num_sample_deltas=6, seed=0):
        from oracle import delta_format as fmt
        from oracle import ops as oracle_ops

        torch.set_num_threads(os.cpu_count() or 1)
        self.cores = torch.get_num_threads()
        self.n = num_sample_deltas
        self.run = oracle_ops.sbmm_dense_f32
        self.weights = []
        for d in range(self.n):
            q, m, s = fmt.random_packed(K, N_OUT, groupsize=GROUP, seed=seed * 1000 + d)
            self.weights.append(torch.from_numpy(fmt.dequantize(q, m, s).astype(np.float32)))
        idx = make_indices(seed, TOKENS, D_PER_GPU)
        self.x = torch.randn(TOKENS, K, generator=torch.Generator().manual_seed(seed)).half().float()
        self.rows = [np.flatnonzero(idx == d) for d in range(self.n)]
        self.tokens = int(sum(len(r) for r in self.rows))

    def timed(self, passes, warmup=1):
        for _ in range(warmup):
            self.run(self.weights, self.x, self.rows)
        t0 = time.perf_counter()
        for _ in range(passes):
            self.run(self.weights, self.x, self.rows)
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
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "product_library_loaded": any("triteia_b200" in m for m in sys.modules)}
    print(json.dumps(line))


# --------------------------------------------------------------------------- helpers of the GPU arm
class Flusher:
    """Write 256 MiB (evicts everything), then read another 256 MiB so that the lines left in L2 are
    clean: a timed step must not pay for writing back the flush's own dirty lines."""

    def __init__(self, dev):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        self.src = torch.zeros(64 << 20, dtype=torch.int32, device=dev)

    def __call__(self):
        self.buf.zero_()
        self.src.sum()


def time_each(fn, reps, flush):
    """Per-launch CUDA-event timing on the current stream, L2 flushed (untimed) before every launch."""
    times = []
    for _ in range(reps):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return times


def time_brackets(run_step, steps, reps, barrier):
    """`reps` brackets of exactly `steps` steps, each bracketed by barrier + synchronize on both sides
    and timed with CUDA events on the launching stream; ms per step of every bracket."""
    out = []
    for _ in range(reps):
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            run_step()
        ev1.record()
        ev1.synchronize()
        barrier()
        out.append(ev0.elapsed_time(ev1) / steps)
    return out


def graph_of(step, barrier):
    """One step captured in a CUDA graph (the library calls neither allocate nor synchronise); returns
    (replay, output of the captured step)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):   # the stream of the warm-up run: its scratch exists already
        out = step()
    barrier()
    graph.replay()
    barrier()
    return graph, out


def check_rows(y, ref_fn, rows, blk0, nblk):
    """max row-relative error of y[rows, 64*blk0 : 64*(blk0+nblk)] against the oracle (fp32)."""
    from oracle import ops as oracle_ops

    if len(rows) == 0:
        return 0.0
    got = y[np.asarray(rows)][:, 64 * blk0:64 * (blk0 + nblk)].float().cpu().numpy()
    return float(oracle_ops.row_rel_err(got, ref_fn(rows, blk0, nblk)).max())


def sample_rows(idx_np, want, seed):
    """Up to `want` rows spread over the distinct ids of the batch (at least one row of -1 if any)."""
    rng = np.random.default_rng(seed)
    rows = []
    for d in rng.permutation(np.unique(idx_np)):
        cand = np.flatnonzero(idx_np == d)
        rows.append(int(rng.choice(cand)))
        if len(rows) >= want:
            break
    return sorted(rows)


# --------------------------------------------------------------------------- headline leg (decode)
def run_decode(args, world, rank, dev, barrier, dist):
    import triteia_b200.ops as ops
    from oracle import ops as oracle_ops
    from triteia_b200 import _lib, sharded
    from triteia_b200.ops.matmul.sbmm import _segments

    total_deltas = D_PER_GPU * world
    qs, metas, ss = ops.random_packed_deltas(D_PER_GPU, K, N_OUT, groupsize=GROUP, device=dev, seed=1000 + rank)
    idx_np = make_indices(rank, TOKENS, total_deltas)
    x_host = torch.randn(TOKENS, K, generator=torch.Generator().manual_seed(rank)).half().pin_memory()
    idx_host = torch.from_numpy(idx_np).pin_memory()
    x_dev, idx_dev = x_host.to(dev), idx_host.to(dev)
    flush = Flusher(dev)
    exchange_kind = None

    def new_exchange():
        kind = os.environ.get("TRB_EXCHANGE", "p2p")
        try:
            return kind, sharded.FixedCapacityExchange(TOKENS, K, N_OUT, dev, backend=kind, qweights=qs, metas=metas,
                                                       scales=ss)
        except Exception as e:   # symmetric memory unavailable
            if rank == 0:
                print(f"bench.py: p2p exchange unavailable ({e}); using NCCL all-to-all", file=sys.stderr)
            return "cuda", sharded.FixedCapacityExchange(TOKENS, K, N_OUT, dev, backend="cuda", qweights=qs,
                                                         metas=metas, scales=ss)

    if world == 1:
        op = lambda xd, idd: ops.sbmm_4bit_2_4_native(qs, xd, metas, ss, idd)
        make_op = lambda: op
        launches_per_step = 3   # router, row gather, grouped kernel
    else:
        exchange_kind, exchange = new_exchange()
        op = lambda xd, idd: exchange(xd, idd)

        def make_op():
            """An exchange of its own (buffers, barriers) for a step that runs beside other steps."""
            _, ex = new_exchange()
            return lambda xd, idd: ex(xd, idd)
        launches_per_step = 5 if exchange_kind == "p2p" else 6   # plan + pack, router + gather + grouped kernel (+ combine)
    step_resident = lambda: op(x_dev, idx_dev)

    for _ in range(max(3, args.warmup)):
        step_resident()
    barrier()

    # ---- `value`: K resident steps per bracket, the bracket repeated; one step is a CUDA-graph replay
    launch_mode, run_step, graph_out = "eager", step_resident, None
    if not args.eager:
        try:
            graph, graph_out = graph_of(step_resident, barrier)
            run_step, launch_mode = graph.replay, "cuda-graph replay of one captured step"
        except Exception as e:   # capture not possible: keep the eager path
            if rank == 0:
                print(f"bench.py: graph capture failed ({e}); timing eager launches", file=sys.stderr)
    for _ in range(3):
        run_step()
    times = time_brackets(run_step, args.steps, args.brackets, barrier)
    value_out = (graph_out if graph_out is not None else step_resident()).clone()
    torch.cuda.synchronize()

    # ---- end-to-end: host buffers in, host buffer out
    class E2ESlot:
        """One in-flight end-to-end step: its own seeded inputs in pinned host buffers, device staging,
        a stream (hence its own scratch inside the op) and a CUDA graph of [copy x and ids in, the
        public op, copy y out]."""

        def __init__(self, number):
            seed = 100 + 10 * number + rank
            self.idx_np = idx_np if number == 0 else make_indices(seed, TOKENS, total_deltas)
            self.x_host = (x_host if number == 0 else
                           torch.randn(TOKENS, K, generator=torch.Generator().manual_seed(seed)).half().pin_memory())
            self.idx_host = torch.from_numpy(self.idx_np).pin_memory()
            self.y_host = torch.zeros(TOKENS, N_OUT, dtype=torch.float16).pin_memory()
            self.x_dev, self.idx_dev = torch.empty_like(x_dev), torch.empty_like(idx_dev)
            self.stream = torch.cuda.Stream()
            self.graph = None
            self.op = op if number == 0 else make_op()

        def body(self):
            self.x_dev.copy_(self.x_host, non_blocking=True)
            self.idx_dev.copy_(self.idx_host, non_blocking=True)
            y = self.op(self.x_dev, self.idx_dev)
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

    # one step alone (latency): L2 flushed before it, wall clock around a stream synchronise
    lat_slot = E2ESlot(0)
    e2e_lat = []
    for i in range(args.steps + 2):
        flush()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        lat_slot.launch()
        lat_slot.stream.synchronize()
        if i >= 2:
            e2e_lat.append((time.perf_counter() - t0) * 1e3)
    barrier()
    # throughput: eight steps in flight on eight streams (at 8 GPUs a step alone takes 230 us of cross-GPU
    # latency against 105 us of device time: 3 / 5 / 8 in flight gave 6.0 / 7.4 / 8.2 M tokens/s there, and
    # 8 is no worse than 3 at 1 and 2 GPUs), every slot with its own inputs, its own scratch
    # and (N > 1) its own exchange buffers and barriers, so the copies and the exchange of one step
    # overlap the kernels of another (the host waits for a slot's previous result before it reuses
    # the slot; every rank launches the slots in the same order).  With the NCCL exchange one step is
    # in flight (one communicator).  No flush: every step streams the touched deltas, far more than L2.
    n_slots = int(os.environ.get("TRB_E2E_SLOTS", "8")) if (world == 1 or exchange_kind == "p2p") else 1
    slots = [lat_slot] + [E2ESlot(i) for i in range(1, n_slots)]
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
    e2e_pipe = []
    for _ in range(args.brackets):
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            sl = slots[i % len(slots)]
            sl.stream.synchronize()      # the slot's previous result is in host memory
            sl.launch()
        for sl in slots:
            sl.stream.synchronize()
        e2e_pipe.append((time.perf_counter() - t0) * 1e3 / args.steps)
    barrier()

    # ---- results against the oracle (outside every timed region): sampled rows x 128 columns of every
    # slot's host result and of the resident leg's output; rows with id -1 must be exactly zero.
    if world == 1:
        fetch = lambda d: (qs[d], metas[d], ss[d])
    else:
        # a rank needs column slices of deltas other ranks own: every rank publishes the slices of its
        # local deltas that anybody's sampled rows select
        need = {}
        for r in range(world):
            for number in range(n_slots):
                seed = 100 + 10 * number + r
                inp = make_indices(r, TOKENS, total_deltas) if number == 0 else make_indices(seed, TOKENS, total_deltas)
                for t in sample_rows(inp, 10, seed):
                    if inp[t] >= 0:
                        need.setdefault(int(inp[t]), set()).add(3 * number)
        mine = {}
        from oracle import delta_format as fmt
        for d, blks in need.items():
            if d % world == rank:
                for b in blks:
                    mine[(d, b)] = fmt.column_blocks(qs[d // world], metas[d // world], ss[d // world], b, 2)
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        slices = {k: v for part in gathered for k, v in part.items()}
        fetch = None

    def oracle_rows(x_t, idx_arr, number):
        def ref(rows, blk0, nblk):
            if world == 1:
                return oracle_ops.sbmm_rows(qs, x_t, metas, ss, idx_arr, rows, blk0, nblk)
            from oracle import delta_format as fmt
            x32 = x_t[np.asarray(rows)].float().cpu().numpy()
            out = np.zeros((len(rows), 64 * nblk), np.float32)
            for i, t in enumerate(rows):
                d = int(idx_arr[t])
                if d >= 0:
                    out[i] = x32[i] @ fmt.dequantize(*slices[(d, blk0)]).astype(np.float32)
            return out
        return ref

    errs, zero_ok = [], True
    for number, sl in enumerate(slots):
        seed = 100 + 10 * number + rank
        rows = sample_rows(sl.idx_np, 10, seed)
        errs.append(check_rows(sl.y_host, oracle_rows(sl.x_host, sl.idx_np, number), rows, 3 * number, 2))
        zero_ok = zero_ok and bool((sl.y_host[sl.idx_np == -1] == 0).all())
    rows0 = sample_rows(idx_np, 10, 100 + rank)
    value_err = check_rows(value_out.cpu(), oracle_rows(x_host, idx_np, 0), rows0, 0, 2)
    zero_ok = zero_ok and bool((value_out[idx_dev == -1] == 0).all())

    # ---- dominant kernel alone (grouped kernel through the segment-list entry point), rank-local
    if world == 1:
        order = torch.argsort(idx_dev, stable=True)
        idx_sorted = idx_dev[order].contiguous()
        x_sorted = x_dev[order].contiguous()
    else:
        # what this rank's grouped kernel sees in a step: the tokens of EVERY rank whose delta it owns
        # (all ranks draw their ids from seed = rank, so they can be restated here without a collective)
        all_idx = torch.from_numpy(np.concatenate([make_indices(r, TOKENS, total_deltas) for r in range(world)])).to(dev)
        mine_mask = (all_idx >= 0) & (all_idx % world == rank)
        loc = torch.div(all_idx[mine_mask], world, rounding_mode="floor")
        o2 = torch.argsort(loc, stable=True)
        idx_sorted = loc[o2].int().contiguous()
        x_sorted = x_dev.repeat(world, 1)[mine_mask][o2].contiguous()
    uniq, starts, counts = _segments(idx_sorted)
    touched = int(uniq.numel())
    y_k = torch.empty(x_sorted.shape[0], N_OUT, dtype=torch.float16, device=dev)
    # the segment-list entry point with working memory for the tail K split (what the fused step's
    # grouped kernel runs with)
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
    k_times = time_each(kern, max(args.steps, 30), flush)
    barrier()

    t_vec = torch.tensor(times + e2e_pipe + [statistics.median(e2e_lat), max(errs + [value_err]), 0.0 if zero_ok else 1.0],
                         device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_vec, op=dist.ReduceOp.MAX)
    t_all = t_vec.tolist()
    times, e2e_pipe = t_all[:len(times)], t_all[len(times):len(times) + len(e2e_pipe)]
    t_e2e_lat, max_err, zero_bad = t_all[-3], t_all[-2], t_all[-1]
    t_step, t_e2e_pipe, t_kern = statistics.median(times), statistics.median(e2e_pipe), statistics.median(k_times)

    if rank != 0:
        return None
    peak, _, peak_src = peaks()
    alg_bytes = touched * BYTES_PER_DELTA + x_sorted.numel() * 2 + y_k.numel() * 2 + touched * 12
    achieved = alg_bytes / (t_kern * 1e-3) / 1e9
    tokens_total = TOKENS * world
    how = None
    if world > 1:
        how = ("rows and results stored straight into the owner's symmetric-memory buffers over NVLink by the pack kernel "
               "and the grouped kernel's epilogue, two cross-GPU barriers per step" if exchange_kind == "p2p" else
               "two equal-split NCCL all-to-alls per step (rows + ids out, result rows back)")
    return {
        "metric": METRIC, "value": tokens_total / (t_step * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": t_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "timing": dict(spread(times), note=f"{args.brackets} brackets of exactly {args.steps} steps, each bracketed by barrier + "
                       "synchronize, CUDA events, max over ranks per bracket; value uses the median bracket"),
        "config": {"workload": WORKLOAD, "deltas_per_gpu": D_PER_GPU, "tokens_per_gpu": TOKENS, "k": K, "n": N_OUT,
                   "groupsize": GROUP, "index_law": "uniform over all deltas, 10% -1, unsorted",
                   "distinct_local_deltas_touched_rank0": touched, "launch": launch_mode,
                   "l2": f"inputs larger than L2: every step streams {touched * BYTES_PER_DELTA / 1e6:.0f} MB of packed "
                         "deltas (126 MB L2, evict-first loads); the kernel-alone roofline leg and the e2e latency leg "
                         "additionally flush L2 before every step (256 MiB memset + 256 MiB read, untimed)",
                   "parallelism": "single GPU" if world == 1 else
                   f"deltas sharded by id over {world} GPUs; {how}; no host synchronisation"},
        "e2e": dict({"value": tokens_total / (t_e2e_pipe * 1e-3), "unit": UNIT, "ms_per_step": t_e2e_pipe,
                     "h2d_bytes_per_step": int(x_host.numel() * 2 + idx_host.numel() * 4),
                     "d2h_bytes_per_step": int(TOKENS * N_OUT * 2),
                     "steps_in_flight": len(slots), "launch": e2e_mode,
                     "latency_ms_one_step": t_e2e_lat, "latency_tokens_per_s": tokens_total / (t_e2e_lat * 1e-3),
                     "e2e_checked": bool(max_err <= TOL and zero_bad == 0.0), "max_row_rel_err": max_err,
                     "note": "sbmm_4bit_2_4_native from pinned host buffers, every step copies x and ids in and y "
                             "out; packed deltas stay resident (model state); every slot has its own seeded inputs, stream "
                             "and scratch; after the timed loop sampled rows (x 128 columns) of every slot's host result "
                             "and of the resident leg's output are compared with the fp32 oracle (bound 1e-2 per row) and "
                             "rows with id -1 must be zero; latency_* is one step alone after an L2 flush"},
                    **{k: v for k, v in spread(e2e_pipe).items() if k != "brackets"}),
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_src, "kernel": "delta_gemm_kernel", "kernel_ms": t_kern,
                     "kernel_ms_p10_p90": [spread(k_times)["p10_ms"], spread(k_times)["p90_ms"]],
                     "algorithmic_bytes": alg_bytes,
                     # dram__bytes_read.sum + dram__bytes_write.sum of the recorded ncu capture of this
                     # launch, scaled by the touched deltas (traffic is proportional to them)
                     "traffic": recorded_traffic("delta_gemm_kernel/" + WORKLOAD, touched)},
    }


# --------------------------------------------------------------------------- ldmm leg (1 GPU)
def run_ldmm(args, dev):
    """fp16 base [11008, 4096] ~N(0, 0.02), 32 per-channel deltas 4096 -> 11008, 32 LoRA adapters of rank 16,
    256 decode tokens, ids Zipf(1.2) over the 64 ids through a seeded permutation."""
    import triteia_b200.ops as ops
    from oracle import ops as oracle_ops

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
    step = lambda: ops.ldmm(idx, x, A, B, qs, metas, ss, base_weight=base)
    for _ in range(max(3, args.warmup)):
        step()
    sync = torch.cuda.synchronize
    run, mode = step, "eager"
    if not args.eager:
        try:
            graph, _ = graph_of(step, sync)
            run, mode = graph.replay, "cuda-graph replay"
        except Exception as e:
            print(f"bench.py: ldmm graph capture failed ({e})", file=sys.stderr)
    times = time_brackets(run, args.steps, max(5, args.brackets // 2), sync)
    y = step()
    # e2e: ids and x in from pinned host memory, y out, one step in flight
    pin = [idx.cpu().pin_memory(), x.cpu().pin_memory()]
    y_host = torch.empty(T, n, dtype=torch.float16).pin_memory()

    def one():
        idd, xd = (t.to(dev, non_blocking=True) for t in pin)
        y_host.copy_(ops.ldmm(idd, xd, A, B, qs, metas, ss, base_weight=base), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    for _ in range(2):
        one()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one()
    t_e2e = (time.perf_counter() - t0) * 1e3 / args.steps
    # oracle: sampled rows over the distinct ids x 128 columns
    rows = sample_rows(ids, 24, 5)
    blk0 = 40

    def ref(rows_, b0, nb):
        from oracle import delta_format as fmt
        xr = x[np.asarray(rows_)].float().cpu().numpy()
        c0, c1 = 64 * b0, 64 * (b0 + nb)
        out = xr @ base[c0:c1].float().cpu().numpy().T
        for i, t in enumerate(rows_):
            d = int(ids[t])
            if 0 <= d < M:
                out[i] += (xr[i] @ A[d].float().cpu().numpy()) @ B[d][:, c0:c1].float().cpu().numpy()
            elif d >= M:
                out[i] += xr[i] @ fmt.dequantize(*fmt.column_blocks(qs[d - M], metas[d - M], ss[d - M], b0, nb)).astype(np.float32)
        return out
    err = check_rows(y_host, ref, rows, blk0, 2)
    t_step = statistics.median(times)
    alg = (n * k * 2 + touched_d * (k * n // 4 + k * n // 8 + n * 2) + touched_l * (k * R + R * n) * 2 + T * k * 2 + T * n * 2)
    peak, _, peak_src = peaks()
    ach = alg / (t_step * 1e-3) / 1e9
    return {"metric": "ldmm_tokens_per_s", "value": T / (t_step * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "ms_per_step": t_step, "timing": spread(times), "higher_is_better": True, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "ldmm-256tok-4096x11008-32deltas-32lora-r16-zipf1.2", "deltas_touched": touched_d,
                       "adapters_touched": touched_l, "launch": mode,
                       "l2": f"inputs larger than L2 ({alg / 1e6:.0f} MB streamed per step)"},
            "e2e": {"value": T / (t_e2e * 1e-3), "unit": UNIT, "ms_per_step": t_e2e,
                    "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in pin)),
                    "d2h_bytes_per_step": int(y_host.numel() * 2), "steps_in_flight": 1,
                    "e2e_checked": bool(err <= TOL), "max_row_rel_err": err},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "peak_source": peak_src, "kernel": "whole ldmm step (every launch of the call)",
                         "algorithmic_bytes": alg, "traffic": None}}


# --------------------------------------------------------------------------- prefill leg (1 GPU)
def run_prefill(args, dev, shape):
    """32 deltas 5120x13824 ("up") or 13824x5120 ("down"), group 128, 8192 tokens in 16 contiguous segments of
    512 (deltas 0..15); SGMV rank-64 LoRA on the same segments timed beside it.  Tensor-bound: flops are
    dense-equivalent 2*T*K*N (the reference's convention, meta/benchmarks/bench_sbmm.py:17)."""
    import triteia_b200.ops as ops
    from oracle import ops as oracle_ops
    from triteia_b200.capi import sbmm_2_4

    k, n = (5120, 13824) if shape == "up" else (13824, 5120)
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
    sync = torch.cuda.synchronize
    step = lambda: ops.sbmm_4bit_2_4_native(qs, x, metas, ss, idx)
    kern = lambda: sbmm_2_4(x, qs, metas, yk, ss, uniq, ws, starts, counts)
    lora = lambda: ops.lora_sgmv(A, B, x, idx)
    for _ in range(max(3, args.warmup)):
        step()
        kern()
    lora()
    reps = max(5, args.brackets // 3)
    steps = max(4, args.steps // 4)
    times = time_brackets(step, steps, reps, sync)
    k_times = time_brackets(kern, steps, reps, sync)
    l_times = time_brackets(lora, max(2, steps // 2), 3, sync)
    y = step()
    pin = [x.cpu().pin_memory(), idx.cpu().pin_memory()]
    y_host = torch.empty(T, n, dtype=torch.float16).pin_memory()

    def one():
        xd, idd = (t.to(dev, non_blocking=True) for t in pin)
        y_host.copy_(ops.sbmm_4bit_2_4_native(qs, xd, metas, ss, idd), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    one()
    t0 = time.perf_counter()
    for _ in range(3):
        one()
    t_e2e = (time.perf_counter() - t0) * 1e3 / 3
    ids = idx.cpu().numpy()
    rows = sorted(int(s * (T // SEG) + o) for s in range(SEG) for o in (3, 257, 511))    # three rows of every segment
    err = check_rows(y_host, lambda r, b0, nb: oracle_ops.sbmm_rows(qs, x, metas, ss, ids, r, b0, nb), rows, 17, 2)
    t_step, t_kern = statistics.median(times), statistics.median(k_times)
    flops = 2.0 * T * k * n
    _, dense, peak_src = peaks()
    ach = flops / (t_kern * 1e-3) / 1e12
    return {"metric": METRIC, "value": T / (t_step * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": steps,
            "ms_per_step": t_step, "timing": spread(times), "higher_is_better": True, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"sbmm-prefill-32x{k}x{n}-g128-8192tok-16seg",
                       "sgmv_rank64_ms": statistics.median(l_times),
                       "l2": "inputs larger than L2 (442 MB of packed deltas touched, 84-226 MB of activations)"},
            "e2e": {"value": T / (t_e2e * 1e-3), "unit": UNIT, "ms_per_step": t_e2e,
                    "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in pin)),
                    "d2h_bytes_per_step": int(y_host.numel() * 2), "steps_in_flight": 1,
                    "e2e_checked": bool(err <= TOL), "max_row_rel_err": err,
                    "note": "bound by the host link (x in, y out)"},
            "roofline": {"bound": "tensor", "achieved": ach, "peak": 2 * dense, "unit": "TFLOP/s", "frac": ach / (2 * dense),
                         "peak_source": "2 x dense bf16 burst, " + peak_src + " (no sparse entry there)",
                         "frac_of_dense_peak": ach / dense, "kernel": "delta_gemm_tcsp_kernel", "kernel_ms": t_kern,
                         "algorithmic_flops": flops, "traffic": None}}


# --------------------------------------------------------------------------- stack leg (any N, strong scaling)
def run_stack(args, world, rank, dev, barrier, dist, layers):
    """L layers of the Llama-2-7B linears (q/k/v and gate/up fused into one packed matrix each, as the
    reference's converter stores them: four linears per layer), 128 deltas sharded by id over the ranks, 512 tokens in all
    (512 / N per rank), delta id ~ Zipf(1.5); one dispatch and one combine per pass.  Strong scaling: the
    same batch and the same deltas at every N."""
    from triteia_b200 import stack

    D, T_total, L, group = 128, 512, layers, 128
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
    exchange = stack.FixedStackExchange(T, (4096, 11008), 4096, dev)
    step = lambda: exchange(xs, idx, local)

    def step_e2e():
        xd = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
        idd = idx_host.to(dev, non_blocking=True)
        y, cs = exchange(xd, idd, local)
        y_host.copy_(y, non_blocking=True)
        cs_host.copy_(cs, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        step()
    step_e2e()
    steps = max(2, min(args.steps, 10))
    times = time_brackets(step, steps, 5, barrier)
    barrier()
    tw = time.perf_counter()
    for _ in range(steps):
        step_e2e()
    t_e2e = (time.perf_counter() - tw) * 1e3 / steps
    barrier()
    mine = set(range(rank, D, world))
    touched_local = len({int(i) for i in ids_all if int(i) in mine})
    per_layer = sum(k * n // 4 + k * n // 8 + (k // group) * n * 2 for _, k, n in stack.LLAMA_7B_FUSED_LINEARS)
    t = torch.tensor(times + [t_e2e, float(touched_local)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    tl = t.tolist()
    times, t_e2e, touched_max = tl[:-2], tl[-2], tl[-1]
    t_step = statistics.median(times)
    del shard, local
    if rank != 0:
        return None
    peak, _, peak_src = peaks()
    alg = touched_max * per_layer * L          # the busiest rank's delta bytes: what bounds the pass
    ach = alg / (t_step * 1e-3) / 1e9
    return {"metric": "stack_tokens_per_s", "value": T_total / (t_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": steps, "ms_per_step": t_step, "timing": spread(times), "higher_is_better": True,
            "scaling": "strong", "dtype": "f16", "data": "synthetic",
            # own kernels per pass: pack, router, one gather per input width, per linear the 256-token-tile launch,
            # the 8-token-tile launch and the checksum, and the combine
            "gpu_launches": steps * (5 + 3 * len(stack.LLAMA_7B_FUSED_LINEARS) * L),
            "config": {"workload": f"stack-llama7b-linears-{L}layers-128deltas-512tok-zipf1.5-g128", "layers": L,
                       "tokens_total": T_total, "linears_per_pass": len(stack.LLAMA_7B_FUSED_LINEARS) * L, "linears": "qkv and gate_up fused as the reference's converter stores them", "ms_per_layer": t_step / L,
                       "distinct_deltas_touched": len(set(int(i) for i in ids_all)),
                       "touched_on_busiest_rank": int(touched_max), "build_s": t_build,
                       "l2": "inputs larger than L2 (every linear streams its touched deltas: 6-17 MB each, all distinct)",
                       "parallelism": "single GPU" if world == 1 else
                       f"deltas sharded by id over {world} GPUs; one equal-split all-to-all of [x4096|x11008] rows + ids "
                       "and one of last outputs + checksums per pass (fixed-capacity buffers, no host synchronisation)"},
            "e2e": {"value": T_total / (t_e2e * 1e-3), "unit": UNIT, "ms_per_step": t_e2e,
                    "h2d_bytes_per_step": int(T * (4096 + 11008) * 2 + T * 4), "d2h_bytes_per_step": int(T * 4096 * 2 + T * 4)},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "peak_source": peak_src, "kernel": "whole pass on the busiest rank",
                         "algorithmic_bytes": alg, "traffic": None}}


# --------------------------------------------------------------------------- phases of one sharded step (N > 1)
def run_shard_phases(args, world, rank, dev, barrier, dist):
    """Where one step of the sharded headline workload spends its time: growing prefixes of the step
    (pack kernel, + barrier, + router / gather / grouped kernel, + barrier) and two parts alone, each as
    a CUDA graph replayed 50 times between barriers; per-step microseconds, max over ranks."""
    import triteia_b200.ops as ops
    from triteia_b200 import _lib, sharded
    from triteia_b200._lib import lib, ptr, stream_of, dev_of

    qs, metas, ss = ops.random_packed_deltas(D_PER_GPU, K, N_OUT, groupsize=GROUP, device=dev, seed=1000 + rank)
    idx_np = make_indices(rank, TOKENS, D_PER_GPU * world)
    idx = torch.from_numpy(idx_np).to(dev)
    x = torch.randn(TOKENS, K, device=dev).half()
    ex = sharded.FixedCapacityExchange(TOKENS, K, N_OUT, dev, backend="p2p", qweights=qs, metas=metas, scales=ss)

    def pack():
        _lib.check(lib.trb_shard_dispatch(ptr(x), ptr(idx), TOKENS, K, world, None, ex.h_recv.buffer_ptrs_dev, rank,
                                          ptr(ex.y_out), N_OUT, ptr(ex.slot_of), ptr(ex.plan), dev_of(x), stream_of(x)), "pack")

    def compute():
        _lib.check(lib.trb_shard_compute(ptr(ex.recv), ptr(qs), ptr(metas), ptr(ss), None, world, TOKENS, N_OUT, K,
                                         D_PER_GPU, GROUP, ex.h_out.buffer_ptrs_dev, rank, ptr(ex.scratch),
                                         ex.scratch.numel(), dev_of(x), stream_of(x)), "compute")
    b1, b2 = (lambda: ex.h_recv.barrier(channel=0)), (lambda: ex.h_out.barrier(channel=0))
    variants = [("pack kernel", lambda: pack()), ("pack + barrier", lambda: (pack(), b1())),
                ("pack + barrier + router, gather, grouped kernel", lambda: (pack(), b1(), compute())),
                ("full step (+ barrier)", lambda: (pack(), b1(), compute(), b2())),
                ("router, gather, grouped kernel alone", lambda: compute()), ("one barrier alone", lambda: b1())]
    for _ in range(3):
        ex(x, idx)
    barrier()
    out = {}
    for name, fn in variants:
        graph, _ = graph_of(fn, barrier)
        for _ in range(5):
            graph.replay()
        ts = []
        for _ in range(7):
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(50):
                graph.replay()
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b) * 1e3 / 50)
        t = torch.tensor([statistics.median(ts)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = float(t.item())
    if rank != 0:
        return None
    rows = int((idx_np >= 0).sum())
    full = out["full step (+ barrier)"]
    return {"metric": METRIC, "value": TOKENS * world / (full * 1e-6), "unit": UNIT, "n_gpus": world, "steps": 50,
            "ms_per_step": full * 1e-3, "higher_is_better": True, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD + "-sharded-step-phases", "us_per_step": out,
                       "nvlink_bytes_per_rank_and_step": {"rows_out": int(rows * (world - 1) / world * K * 2),
                                                          "results_back": int(rows * (world - 1) / world * N_OUT * 2)}}}


# --------------------------------------------------------------------------- GPU arm
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
    from triteia_b200 import _lib

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def free():
        gc.collect()
        torch.cuda.empty_cache()

    legs = ([args.workload] if args.workload != "all" else
            ["decode", "stack"] + (["ldmm", "prefill_up", "prefill_down"] if world == 1 else []))
    if args.no_legs:
        legs = ["decode"]
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_wall0 = time.perf_counter()
    results = {}
    for leg in legs:
        if leg == "decode":
            results[leg] = run_decode(args, world, rank, dev, barrier, dist)
        elif leg == "stack":
            if world == 1 and not dist.is_initialized():
                dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % (29700 + os.getpid() % 200), rank=0,
                                        world_size=1, device_id=dev)
            results[leg] = run_stack(args, world, rank, dev, barrier, dist, args.layers)
        elif leg == "ldmm" and world == 1:
            results[leg] = run_ldmm(args, dev)
        elif leg in ("prefill_up", "prefill_down") and world == 1:
            results[leg] = run_prefill(args, dev, leg.split("_")[1])
        elif leg == "shard_phases":
            if world < 2:
                raise SystemExit("bench.py: --workload shard_phases needs --gpus 2 or more (torchrun)")
            results[leg] = run_shard_phases(args, world, rank, dev, barrier, dist)
        free()
        barrier()
    clocks = sampler.stop() if rank == 0 else None
    status = _lib.device_status(local_rank)
    if rank == 0:
        first = legs[0]
        line = results[first]
        line.setdefault("n_gpus", world)
        line.setdefault("warmup", max(3, args.warmup))
        line.setdefault("scaling", "weak")
        line.setdefault("vs_baseline", None)
        others = {k: v for k, v in results.items() if k != first and v is not None}
        if others:
            line["legs"] = others
        line["clocks"] = clocks
        line["device_status"] = status
        line["wall_s"] = time.perf_counter() - t_wall0
        if "gpu_launches" not in line:
            line["gpu_launches"] = None
        if first == "decode" and world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line))
    if dist.is_initialized():
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--brackets", type=int, default=25, help="how many times the K-step bracket is repeated (median reported)")
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (profiling runs)")
    ap.add_argument("--no-legs", action="store_true", help="headline leg only (profiling runs)")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of CUDA-graph replays")
    ap.add_argument("--workload", default="all", choices=["all", "decode", "prefill_up", "prefill_down", "ldmm", "stack", "shard_phases"],
                    help="all = the headline sbmm configuration with the other configurations as `legs` (default); "
                         "one name = that leg alone")
    ap.add_argument("--layers", type=int, default=2, help="stack: number of layers (2: 19 GB of deltas in all; 8 fits one GPU)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
