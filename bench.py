#!/usr/bin/env python
"""Benchmark of the W4A16 quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (N = 1): the decode GEMV sweep of the benchmark configuration "batched decode GEMV over every
linear of a Qwen2.5-7B-shaped layer" at M = 1 -- one STEP is one pass over the seven int4 group-128 linears
of a layer (q, k, v, o, gate, up, down) through the library's GEMV and its C ABI, as FOUR launches: q|k|v and
gate|up are row-concatenated matrices (rows of Wq / S are independent, so this is the same arithmetic in fewer
launches; `--seven-launches` runs them separately).  Weights rotate through eight distinct layer copies (961 MB)
so every step streams from HBM, not from the 126 MB L2.
Metric: algorithmic bytes moved per second (packed weights + scales + X + bf16 Y, the reference's byte model,
bench/bench_w4a16.cu:239).

With N > 1 ranks (one per GPU) every matrix is sharded by output rows over the ranks (tensor parallel) and
the outputs are all-gathered at the four layer boundaries (after q/k/v, o, gate/up, down) -- inside the GEMVs
(peer stores + arrival counters) or, with --tp-collective, by NCCL; the value is the whole-layer bytes over the
slowest rank's time, so scaling is "strong".  Rank 0 also holds one layer unsharded and checks the gathered
outputs of the sharded pass against it (`tp_check`).

One JSON line is printed by rank 0.  `value` is measured with inputs resident in HBM; `e2e` is the same
pass through the public Python/C-ABI call path with the step's activations copied from pinned host memory and
all outputs copied back inside the timed region; `roofline` times the dominant kernel (the 18944 x 3584 GEMV)
alone; `cpu_baseline` times the CPU oracle (a port of the reference's host dequant-then-matmul check,
bench/bench_w4a16.cu:156-173) on a bounded sample.  `--impl reference` times that CPU path alone with all host
threads.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from nanoserve_b200 import synth  # noqa: E402

METRIC = "W4A16 GEMV HBM GB/s at M=1 (Qwen2.5-7B-shaped layer, int4 g128)"
METRIC_70B = "W4A16 GEMV HBM GB/s at M=1 (70B-class layer: hidden 8192, intermediate 28672, int4 g128)"
DTYPE = ("int4 weights x bf16 activations; X as block fixed point per (token, 128-chunk) -- 32-bit for one token, 15-bit + "
         "sign above -- on 8-bit integer mma, s32 accumulation per chunk, fp32 across chunks, bf16 output")
UNIT = "GB/s"
G = 128
M_DECODE = 1
LAYER = synth.QWEN25_7B_LAYER
ORDER = ["q", "k", "v", "o", "gate", "up", "down"]
N_COPIES = 8
L2_BYTES = 126 * 2**20


def layer_bytes(M):
    return sum(synth.gemv_bytes(M, n, k, G) for n, k in (LAYER[x] for x in ORDER))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ---------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

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
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, val in zip(names, r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------- CPU legs (oracle)
def cpu_layer_pass(threads, n_passes, seed=100):
    """Times `n_passes` passes over the layer's seven linears at M = 1 on the host with the CPU oracle.
    Returns (seconds per pass, threads used)."""
    import oracle  # test infrastructure: used here only as the timed CPU baseline
    mats = {}
    for name in ORDER:
        n, k = LAYER[name]
        mats[name] = synth.synth_weight(n, k, G, seed)
    xs = {k: synth.synth_x(M_DECODE, k, seed) for k in {LAYER[x][1] for x in ORDER}}
    t0 = time.perf_counter()
    for _ in range(n_passes):
        for name in ORDER:
            Wq, S = mats[name]
            oracle.w4_linear_f32(xs[LAYER[name][1]], Wq, S, G, threads=threads)
    dt = (time.perf_counter() - t0) / n_passes
    return dt, (threads if threads > 1 else 1)


def run_reference_arm(args):
    """The reference's CPU implementation of the path (its host dequant-then-FP32/double check), all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    threads = oracle.max_threads()
    for _ in range(max(0, min(args.warmup, 2))):
        cpu_layer_pass(threads, 1)
    steps = max(1, args.steps)
    per_step_budget = 120.0 / steps  # keep the whole run within a few minutes
    one, _ = cpu_layer_pass(threads, 1)
    passes_per_step = 1
    if one > per_step_budget:
        passes_per_step = 1  # a step is never less than one pass; the cap below bounds the total instead
    steps_run = steps if one * steps <= 240.0 else max(1, int(240.0 / one))
    dt, used = cpu_layer_pass(threads, steps_run * passes_per_step)
    value = layer_bytes(M_DECODE) / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int4 weights x bf16 activations, fp64 accumulate (host)",
        "data": "synthetic",
        "config": {"workload": "decode GEMV pass over the 7 linears of a Qwen2.5-7B-shaped layer, M=1, int4 g128",
                   "steps_timed": steps_run},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": used, "kind": "port",
                         "sample": f"{steps_run} full layer passes (7 linears, 233M weights each pass)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------- sweep over the other configurations
def run_sweep(k, dev, stream, flags):
    """Decode GEMV at M in {1,2,4,8,16} over every 7B-shaped linear and the 70B-class gate/up and down, and the
    prefill GEMM at M in {512,2048,8192} (4096 for the 70B-class shape), on one GPU.  Weights are random nibbles with
    the benchmark's scale distribution, generated on the device; enough distinct copies are used in rotation that every
    launch streams from HBM.  Each entry: microseconds per launch (CUDA events around a replayed CUDA graph), GB/s of
    algorithmic bytes or TFLOP/s, and the fraction of the measured peak."""
    import torch
    peaks, which = measured_peaks()
    gen = torch.Generator(device=dev).manual_seed(7)

    def rand_w4(N, K):
        Wq = torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, device=dev, generator=gen)
        S = (0.005 + (torch.randn(N, K // G, device=dev, generator=gen) * 0.01).abs()).to(torch.bfloat16)
        return Wq, S

    def time_graph(fns, reps):
        with torch.cuda.stream(stream):
            for f in fns[:2]:
                f()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for f in fns:
                    f()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record(stream)
            for _ in range(reps):
                g.replay()
            ev1.record(stream)
            torch.cuda.synchronize()
        return ev0.elapsed_time(ev1) * 1e-3 / (reps * len(fns))

    out = {"peak_source": which, "hbm_gbs_peak": peaks["hbm_gbs"], "bf16_tflops_peak": peaks["bf16_tflops"],
           "gemv": [], "gemm": []}
    gemv_shapes = [("q/o", 3584, 3584), ("k/v", 512, 3584), ("gate/up", 18944, 3584), ("down", 3584, 18944),
                   ("70b gate/up", 28672, 8192), ("70b down", 8192, 28672)]
    for name, N, K in gemv_shapes:
        copies = max(4, min(32, (512 << 20) // (N * K // 2) + 1))
        ws = [rand_w4(N, K) for _ in range(copies)]
        for M in (1, 2, 4, 8, 16):
            x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
            y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            t = time_graph([(lambda w=w: k.w4_linear(x, w[0], w[1], G, flags=flags, out=y)) for w in ws], 10)
            nb = synth.gemv_bytes(M, N, K, G)
            out["gemv"].append({"shape": name, "N": N, "K": K, "M": M, "plan": k.gemv_describe(M, N, K, G, flags),
                                "us": round(t * 1e6, 2),
                                "gbs": round(nb / t / 1e9, 1), "frac": round(nb / t / 1e9 / peaks["hbm_gbs"], 3)})
        del ws
        torch.cuda.empty_cache()
    gemm_shapes = [("gate/up", 18944, 3584, (512, 2048, 8192)), ("down", 3584, 18944, (512, 2048, 8192)),
                   ("70b gate/up", 28672, 8192, (4096,))]
    for name, N, K, Ms in gemm_shapes:
        ws = [rand_w4(N, K) for _ in range(2)]
        for M in Ms:
            x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
            y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            t = time_graph([(lambda w=w: k.w4_linear(x, w[0], w[1], G, out=y)) for w in ws], 5)
            fl = 2.0 * M * N * K
            out["gemm"].append({"shape": name, "N": N, "K": K, "M": M, "us": round(t * 1e6, 1),
                                "tflops": round(fl / t / 1e12, 1),
                                "frac": round(fl / t / 1e12 / peaks["bf16_tflops"], 3)})
            del x, y
        del ws
        torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------- 70B-class prefill GEMM over the ranks
def run_prefill_tp(k, dev, stream, rank, world, M=4096, N=28672, K=8192, reps=6):
    """Prefill GEMM of the 70B-class gate/up shape with the output features sharded over the ranks (rank r holds rows
    [r N/P, (r+1) N/P) of the weight) and the outputs all-gathered by NCCL: once as GEMM then gather, once with M cut
    into chunks so the gather of one chunk runs on a second stream under the GEMM of the next.  Times are CUDA events
    on the compute stream between barriers, max over ranks; TFLOP/s is 2 M N K over that time (the whole job)."""
    import torch
    import torch.distributed as dist
    gen = torch.Generator(device=dev).manual_seed(21 + rank)
    nl = N // world
    ws = []
    for _ in range(2):
        Wq = torch.randint(-2**31, 2**31 - 1, (nl, K // 8), dtype=torch.int32, device=dev, generator=gen)
        S = (0.005 + (torch.randn(nl, K // G, device=dev, generator=gen) * 0.01).abs()).to(torch.bfloat16)
        ws.append((Wq, S))
    x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
    comm = torch.cuda.Stream(device=dev)

    def make(chunks, gather):
        mc = M // chunks
        ys = [torch.empty(mc, nl, dtype=torch.bfloat16, device=dev) for _ in range(chunks)]
        gs = [torch.empty(world, mc, nl, dtype=torch.bfloat16, device=dev) for _ in range(chunks)]
        evs = [torch.cuda.Event() for _ in range(chunks)]

        def step(w):
            for c in range(chunks):
                k.w4_linear(x[c * mc:(c + 1) * mc], w[0], w[1], G, out=ys[c])
                if gather and world > 1:
                    if chunks == 1:
                        dist.all_gather_into_tensor(gs[c], ys[c])
                    else:
                        evs[c].record(stream)
                        with torch.cuda.stream(comm):
                            comm.wait_event(evs[c])
                            dist.all_gather_into_tensor(gs[c], ys[c])
            if gather and world > 1 and chunks > 1:
                stream.wait_stream(comm)
        return step

    def timed(step):
        with torch.cuda.stream(stream):
            for i in range(3):
                step(ws[i % 2])
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record(stream)
            for i in range(reps):
                step(ws[i % 2])
            ev1.record(stream)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        t = torch.tensor([ev0.elapsed_time(ev1) * 1e-3 / reps], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    peaks, which = measured_peaks()
    fl = 2.0 * M * N * K
    out = {"M": M, "N": N, "K": K, "rows_per_rank": nl, "gathered_bytes_per_rank": M * N * 2,
           "peak_source": which, "bf16_tflops_peak_per_gpu": peaks["bf16_tflops"]}
    legs = [("gemm_only", 1, False)]
    if world > 1:
        legs += [("gemm_then_all_gather", 1, True), ("overlapped_2_chunks", 2, True), ("overlapped_4_chunks", 4, True)]
    for name, chunks, gather in legs:
        t = timed(make(chunks, gather))
        out[name] = {"ms": round(t * 1e3, 4), "tflops_aggregate": round(fl / t / 1e12, 1),
                     "frac_of_peak_x_gpus": round(fl / t / 1e12 / (peaks["bf16_tflops"] * world), 3)}
    return out


# ---------------------------------------------------------------------------- reference GPU kernels, copy ceiling
def ref_gpu_numbers(dev, stream):
    """The reference's own kernels (its C-ABI library built unchanged for sm_100a by oracle/Makefile, when present) on
    the same B200: the M = 1 GEMV of the dominant shape and the M = 2048 GEMM, CUDA events around a replayed graph
    over rotating weight copies.  Outside every timed region of this library's arm."""
    import torch
    path = os.path.join(ROOT, "oracle", "_ref", "libnanoserve_ref.so")  # the reference's library, not the oracle
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libnanoserve_ref.so not built"}
    lib = ctypes.CDLL(path)
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    lib.ns_w4_linear.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, vp]
    lib.ns_w4_linear.restype = i32
    gen = torch.Generator(device=dev).manual_seed(17)
    out = {}
    for key, M, N, K, copies, reps in (("gemv_m1_18944x3584", 1, 18944, 3584, 16, 10),
                                       ("gemm_m2048_18944x3584", 2048, 18944, 3584, 4, 3)):
        ws = []
        for _ in range(copies):
            Wq = torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, device=dev, generator=gen)
            S = (0.005 + (torch.randn(N, K // G, device=dev, generator=gen) * 0.01).abs()).to(torch.bfloat16)
            ws.append((Wq, S))
        x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

        def call(w):
            rc = lib.ns_w4_linear(x.data_ptr(), w[0].data_ptr(), w[1].data_ptr(), y.data_ptr(), M, N, K, G,
                                  ctypes.c_void_p(stream.cuda_stream))
            if rc != 0:
                raise RuntimeError(f"reference ns_w4_linear returned {rc}")
        try:
            with torch.cuda.stream(stream):
                for w in ws[:2]:
                    call(w)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    for w in ws:
                        call(w)
                g.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(reps):
                    g.replay()
                e1.record(stream)
                torch.cuda.synchronize()
            out[key + "_us"] = round(e0.elapsed_time(e1) * 1e3 / (reps * copies), 2)
        except Exception as e:  # noqa: BLE001 - a failure of the comparison leg must not lose the line
            out[key + "_us"] = f"{type(e).__name__}: {e}"
        del ws
        torch.cuda.empty_cache()
    return out


def copy_ceiling_gbs(dev, stream):
    """The reference's notion of the bandwidth ceiling (kernels/fused/vec.cuh:43-47, used at
    bench/bench_w4a16.cu:122-136): a device-to-device copy of 512 MiB with 16-byte accesses, read + write bytes over
    the time.  Restated with the device copy of the tensor library (the same access pattern)."""
    import torch
    n = (512 << 20) // 2
    a = torch.ones(n, dtype=torch.bfloat16, device=dev)
    b = torch.empty_like(a)
    best = 1e9
    with torch.cuda.stream(stream):
        for _ in range(3):
            b.copy_(a)
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            b.copy_(a)
            e1.record(stream)
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1e-3)
    return 2.0 * n * 2 / best / 1e9


# ---------------------------------------------------------------------------- GPU arm
class LayerBench:
    """Resident layer copies (sharded over the ranks), one CUDA graph per copy, replayed in rotation."""

    def __init__(self, k, shapes, n_copies, M, rank, world, dev, flags, fused_gather, seven, seed0=1000):
        import torch
        from nanoserve_b200.tp import PeerBuffers, ShardedLayer
        self.k, self.shapes, self.M, self.world, self.rank, self.dev = k, shapes, M, world, rank, dev
        self.seven, self.n_copies, self.seed0, self.flags = seven, n_copies, seed0, flags
        self.layers = [ShardedLayer.synthetic(k, shapes, ORDER, G, seed=seed0 + c, rank=rank, world=world, device=dev,
                                              flags=flags) for c in range(n_copies)]
        self.peer = None
        if fused_gather:
            if seven:
                rows = {name: M * shapes[name][0] for name in ORDER}
                ncnt = len(ShardedLayer.BOUNDARIES)
            else:
                rows = {f: M * sum(shapes[n][0] for n in names) for f, names in ShardedLayer.FUSED}
                ncnt = len(ShardedLayer.FUSED)
            self.peer = PeerBuffers(rows, ncnt, dev)
        for l in self.layers:
            if self.peer is not None:
                if seven:
                    l.attach_peer_buffers(self.peer, M)
                else:
                    l.peer, l.M = self.peer, M
            if not seven:
                l.fuse()
        hidden, inter = shapes["q"][1], shapes["down"][1]
        self.x_h = torch.from_numpy(synth.synth_x(M, hidden, 1).view(np.int16)).view(torch.bfloat16).pin_memory()
        self.a_h = torch.from_numpy(synth.synth_x(M, inter, 2).view(np.int16)).view(torch.bfloat16).pin_memory()
        self.x_d, self.a_d = self.x_h.to(dev), self.a_h.to(dev)
        self.stream = torch.cuda.Stream(device=dev)
        self.graphs = []

    def one_pass(self, l, x, a):
        return l.decode_pass(x, a) if self.seven else l.decode_pass_fused4(x, a)

    def capture(self):
        import torch
        with torch.cuda.stream(self.stream):
            # every kernel variant is loaded by a plain launch first and the ranks meet: a tensor-parallel launch
            # waits at most half a second for its peers, less than a first-use module load on a loaded host can take
            l0 = self.layers[0]
            for name in ORDER:
                Wq, S = l0.shards[name]
                self.k.w4_linear(self.a_d if name == "down" else self.x_d, Wq, S, G)
            if not self.seven:
                for fname, (Wq, S) in l0.fused.items():
                    self.k.w4_linear(self.a_d if fname == "down" else self.x_d, Wq, S, G)
            self.barrier()
            for l in self.layers:
                self.one_pass(l, self.x_d, self.a_d)  # warm-up passes before capture
            torch.cuda.synchronize()
            for l in self.layers:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream):
                    self.one_pass(l, self.x_d, self.a_d)
                self.graphs.append(g)

    def barrier(self):
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_replays(self, n):
        import torch
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        with torch.cuda.stream(self.stream):
            ev0.record(self.stream)
            for i in range(n):
                self.graphs[i % self.n_copies].replay()
            ev1.record(self.stream)
        self.barrier()
        return ev0.elapsed_time(ev1) * 1e-3

    def resident_bytes(self):
        return sum(l.resident_bytes() for l in self.layers)

    def launches_per_step(self):
        from nanoserve_b200.tp import ShardedLayer
        if self.seven:
            return len(ORDER) + (len(ShardedLayer.BOUNDARIES) if self.peer is not None else 0)
        # (a launch whose K is cut into slices across CTAs is followed by the kernel that adds the slices)
        sums = 0
        if self.peer is None:
            for _, names in ShardedLayer.FUSED:
                N = sum(self.shapes[n][0] for n in names)
                plan = self.k.gemv_describe(self.M, N, self.shapes[names[0]][1], G, self.flags)
                if "(sum kernel)" in plan:
                    sums += 1
        return len(ShardedLayer.FUSED) + sums + (1 if self.peer is not None else 0)


def tp_check(lb, k, dev):
    """Tensor parallel == single GPU.  The reference has no multi-GPU code, so the checker for the sharded path is
    this library's own unsharded result: rank 0 uploads layer copy 0 whole, runs the plain ns_w4_linear on it and
    compares with the gathered outputs of the sharded pass (every rank holds them).  Bound: one bf16 rounding of the
    value plus 1e-5 of the largest output (the sharded and the whole matrix may split K differently)."""
    import torch
    import torch.distributed as dist
    from nanoserve_b200.tp import ShardedLayer, _to_torch_bits
    with torch.cuda.stream(lb.stream):
        outs = [o.clone() for o in lb.one_pass(lb.layers[0], lb.x_d, lb.a_d)]
    lb.barrier()
    res = {"max_rel": 0.0, "ok": True, "matrices": 0}
    if lb.rank == 0:
        groups = [(n,) for n in ORDER] if lb.seven else [names for _, names in ShardedLayer.FUSED]
        for names, got in zip(groups, outs):
            full = []
            for n in names:
                N, K = lb.shapes[n]
                Wq, S = synth.synth_weight(N, K, G, lb.seed0)
                y = k.w4_linear(lb.a_d if n == "down" else lb.x_d, _to_torch_bits(Wq, torch.int32, dev),
                                _to_torch_bits(S, torch.bfloat16, dev), G)
                full.append(y)
            want = torch.cat(full, dim=1).float()
            g = got.float()
            scale = want.abs().max()
            excess = ((g - want).abs() - torch.maximum(g.abs(), want.abs()) * 2.0**-7).clamp(min=0) / scale
            res["max_rel"] = max(res["max_rel"], float(excess.max()))
            res["matrices"] += len(names)
        res["ok"] = res["max_rel"] <= 1e-5
    torch.cuda.synchronize()
    if lb.world > 1:
        dist.barrier()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=M_DECODE, help="tokens per step (1..16); the headline is 1")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the Qwen2.5-7B-shaped greedy-decode tokens/s leg")
    ap.add_argument("--flags", type=int, default=0, help="library flags for every launch (see include/nanoserve_b200.h)")
    ap.add_argument("--layer", default="7b", choices=["7b", "70b"],
                    help="shapes of the headline layer pass: the Qwen2.5-7B-shaped layer of the headline metric, or the "
                         "70B-class layer (hidden 8192, intermediate 28672) of the multi-GPU configuration")
    ap.add_argument("--tp-collective", action="store_true",
                    help="N > 1: all-gather the outputs with NCCL at the layer boundaries instead of fusing the gather "
                         "into the GEMVs (peer stores + arrival counters); implies --seven-launches")
    ap.add_argument("--seven-launches", action="store_true",
                    help="run q, k, v and gate, up as separate launches (seven per pass) instead of row-concatenated")
    ap.add_argument("--no-sweep", action="store_true",
                    help="skip the single-GPU sweep over the other benchmark configurations (decode GEMV at M = 1..16 over "
                         "every 7B-shaped and 70B-class linear, prefill GEMM at M = 512..8192), the 70B-class layer pass and "
                         "the 70B-class prefill GEMM sharded over the ranks")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    # stdout carries the one JSON line and nothing else: whatever a library prints there (NCCL announces its version
    # when the communicator is created) goes to stderr
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist
    from nanoserve_b200 import build as b2build
    from nanoserve_b200.ops import Kernels

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import datetime
        # a short collective time-out: a rank that falls out of step fails the run in a minute instead of hanging it
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    if not os.path.exists(b2build.LIB_PATH):
        if rank == 0:
            b2build.build()
        if world > 1:
            dist.barrier()
    k = Kernels(b2build.LIB_PATH)
    k.init()
    M = args.m
    warm = max(3, args.warmup)
    seven = args.seven_launches or args.tp_collective
    fused_gather = world > 1 and not args.tp_collective
    shapes = synth.QWEN25_7B_LAYER if args.layer == "7b" else synth.CLASS_70B_LAYER
    n_copies = N_COPIES if args.layer == "7b" else 4
    nbytes = sum(synth.gemv_bytes(M, n, kk, G) for n, kk in (shapes[x] for x in ORDER))

    # ---- device-resident timing: one CUDA graph per layer copy, replayed in rotation
    lb = LayerBench(k, shapes, n_copies, M, rank, world, dev, args.flags, fused_gather, seven)
    lb.capture()
    resident = lb.resident_bytes()
    lb.timed_replays(warm)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_first = lb.timed_replays(args.steps)
    # the K steps are timed again until at least 50 ms have been timed in all (a 56 us step would otherwise be measured
    # over a millisecond); every rank runs the same number of blocks (the count comes from rank 0: the replays hold
    # collectives or peer waits), and the per-step time is the mean over all of them
    blocks = [max(1, min(400, int(np.ceil(0.05 / max(t_first, 1e-6)))))]
    if world > 1:
        dist.broadcast_object_list(blocks, src=0)
    t_blocks = [lb.timed_replays(args.steps) for _ in range(blocks[0])]
    t_dev = float(np.mean(t_blocks))
    # keep the GPUs under the same load a little longer so the 100 ms clock sampler sees it
    n_extra = [max(1, int(0.6 / max(t_dev / args.steps, 1e-6) / 200))]
    if world > 1:
        dist.broadcast_object_list(n_extra, src=0)
    for _ in range(min(n_extra[0], 200)):
        lb.timed_replays(200)
    clocks = sampler.stop() if rank == 0 else None

    leg_status = {"layer_pass": k.device_status()}

    # ---- end to end: public API, host buffers, copies inside the timed region.  One pinned buffer holds the step's
    # two inputs (one host-to-device copy); on one GPU the four outputs are views of one device buffer (one copy back)
    stream = lb.stream
    hidden, inter = shapes["q"][1], shapes["down"][1]
    in_h = torch.cat([lb.x_h.reshape(-1), lb.a_h.reshape(-1)]).pin_memory()
    widths = None if seven else [sum(shapes[n][0] for n in names) for _, names in lb.layers[0].FUSED]
    out_d = out_h = out_views = None
    if world == 1 and not seven:
        out_d = torch.empty(M * sum(widths), dtype=torch.bfloat16, device=dev)
        out_h = torch.empty(M * sum(widths), dtype=torch.bfloat16).pin_memory()
        out_views, off = [], 0
        for w in widths:
            out_views.append(out_d[off:off + M * w].view(M, w))
            off += M * w
    outs_h = None

    def e2e_step(l):
        nonlocal outs_h
        in_d = in_h.to(dev, non_blocking=True)
        xd, ad = in_d[:M * hidden].view(M, hidden), in_d[M * hidden:].view(M, inter)
        if out_views is not None:
            l.decode_pass_fused4(xd, ad, outs=out_views)
            out_h.copy_(out_d, non_blocking=True)
        else:
            outs = lb.one_pass(l, xd, ad)
            if outs_h is None:
                outs_h = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
            for oh, o in zip(outs_h, outs):
                oh.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    with torch.cuda.stream(stream):
        for i in range(warm):
            e2e_step(lb.layers[i % n_copies])
        lb.barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            e2e_step(lb.layers[i % n_copies])
        lb.barrier()
        t_e2e_eager = time.perf_counter() - t0
    # the same step as a serving loop would issue it: ShardedLayer.host_step, one CUDA graph per step with the two
    # copies inside (one graph launch + one stream synchronisation per step)
    t_e2e_wall, e2e_path = t_e2e_eager, "Kernels.w4_linear per launch (ctypes -> C ABI), pinned host X in, all outputs out"
    if not seven:
        host_steps = [l.host_step(M, stream, zero_copy_out=(world == 1)) for l in lb.layers]
        for hs in host_steps:
            hs.x_host.copy_(lb.x_h)
            hs.act_host.copy_(lb.a_h)
        with torch.cuda.stream(stream):
            for i in range(warm):
                host_steps[i % n_copies]()
            lb.barrier()
            t0 = time.perf_counter()
            for i in range(args.steps):
                host_steps[i % n_copies]()
            lb.barrier()
            t_e2e_wall = time.perf_counter() - t0
        e2e_path = ("ShardedLayer.host_step: one CUDA graph per step (pinned host X in, 4 GEMV launches through the C "
                    "ABI, all outputs out to pinned host memory" +
                    (": the kernels store them there themselves" if world == 1 else "") +
                    "), graph launch + stream synchronise per step")
        if world == 1:
            last = (args.steps - 1) % n_copies  # the layer copy both paths ran last
            assert torch.equal(host_steps[last].out_host, out_h), "host_step and the per-launch path disagree"
        del host_steps
    h2d = in_h.numel() * 2
    d2h = out_h.numel() * 2 if out_h is not None else sum(o.numel() * 2 for o in outs_h)
    leg_status["e2e"] = k.device_status()

    # ---- tensor parallel == single GPU, on the real GPUs
    check = tp_check(lb, k, dev) if world > 1 else None
    leg_status["tp_check"] = k.device_status()

    # ---- the dominant kernel alone: the 18944 x 3584 GEMV over 16 distinct matrices (gate and up of 8 copies)
    roof = None
    peaks, which = measured_peaks()
    if world == 1 and args.layer == "7b":
        big = [l.shards["gate"] for l in lb.layers] + [l.shards["up"] for l in lb.layers]
        y_big = torch.empty(M, 18944, dtype=torch.bfloat16, device=dev)
        with torch.cuda.stream(stream):
            gk = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gk, stream=stream):
                for (Wq, S) in big:
                    k.w4_linear(lb.x_d, Wq, S, G, flags=args.flags, out=y_big)
            for _ in range(3):
                gk.replay()
            torch.cuda.synchronize()
            reps = 200  # 16 launches x 200 replays x ~8 us: 25 ms timed
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record(stream)
            for _ in range(reps):
                gk.replay()
            ev1.record(stream)
            torch.cuda.synchronize()
            t_k = ev0.elapsed_time(ev1) * 1e-3 / (reps * len(big))
        kb = synth.gemv_bytes(M, 18944, 3584, G)
        ach = kb / t_k / 1e9
        ceiling = copy_ceiling_gbs(dev, stream)
        roof = {"bound": "hbm", "kernel": "w4_gemv_stream_kernel (N=18944, K=3584, M=%d)" % M, "achieved": ach,
                "peak": peaks["hbm_gbs"], "peak_source": which + " copy bandwidth (MEASURED_PEAKS.json)"
                if which == "measured" else "fallback 6650 GB/s",
                "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "us_per_launch": t_k * 1e6,
                "bytes_per_launch": kb, "traffic": None,
                "frac_of_copy_ceiling": ach / ceiling, "copy_ceiling_gbs": ceiling,
                "copy_ceiling_def": "512 MiB device copy, 16-byte accesses, read + write bytes (reference: kernels/fused/"
                                    "vec.cuh:43-47, bench/bench_w4a16.cu:122-136), measured in this run",
                "frac_of_nominal_8tbs": ach / 8000.0}
        traffic_file = os.path.join(ROOT, "profiles", "gemv_traffic.json")
        if os.path.exists(traffic_file):
            with open(traffic_file) as f:
                roof["traffic"] = json.load(f).get("dram_bytes_per_launch_m%d" % M)
        del big, y_big

    # ---- the reference's own GPU kernels on the same box (the kernels to beat), outside the timed regions
    ref_gpu = ref_gpu_numbers(dev, stream) if world == 1 and not args.no_sweep else None
    if ref_gpu is not None and roof is not None and isinstance(ref_gpu.get("gemv_m1_18944x3584_us"), float):
        ref_gpu["gemv_speedup"] = round(ref_gpu["gemv_m1_18944x3584_us"] / roof["us_per_launch"], 2)

    # ---- free the headline layer copies before the wider legs
    del lb.graphs[:], lb.layers[:]
    torch.cuda.empty_cache()

    # ---- the other benchmark configurations on one GPU: every decode shape at M = 1..16, the prefill GEMMs
    sweep = None
    if world == 1 and not args.no_sweep and args.layer == "7b":
        sweep = run_sweep(k, dev, stream, args.flags)
        if ref_gpu is not None and isinstance(ref_gpu.get("gemm_m2048_18944x3584_us"), float):
            ours = [e for e in sweep["gemm"] if e["N"] == 18944 and e["M"] == 2048]
            if ours:
                ref_gpu["gemm_speedup"] = round(ref_gpu["gemm_m2048_18944x3584_us"] / ours[0]["us"], 2)

    # ---- configuration 5: the 70B-class layer pass (same code, other shapes) and its sharded prefill GEMM, at every N
    layer70 = None
    prefill = None
    if not args.no_sweep:
        if args.layer == "7b":
            try:
                lb70 = LayerBench(k, synth.CLASS_70B_LAYER, 4, M, rank, world, dev, args.flags, fused_gather, seven, seed0=2000)
                lb70.capture()
                lb70.timed_replays(warm)
                t70 = float(np.mean([lb70.timed_replays(40) for _ in range(3)])) / 40
                tt = torch.tensor([t70], dtype=torch.float64, device=dev)
                if world > 1:
                    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                t70 = float(tt.item())
                nb70 = sum(synth.gemv_bytes(M, n, kk, G) for n, kk in (synth.CLASS_70B_LAYER[x] for x in ORDER))
                layer70 = {"us_per_pass": round(t70 * 1e6, 2), "gbs": round(nb70 / t70 / 1e9, 1), "bytes_per_pass": nb70,
                           "frac_of_hbm_peak_x_gpus": round(nb70 / t70 / 1e9 / (peaks["hbm_gbs"] * world), 3),
                           "launches_per_pass": lb70.launches_per_step()}
                if world > 1:
                    layer70["tp_check"] = tp_check(lb70, k, dev)
                del lb70.graphs[:], lb70.layers[:]
                del lb70
                torch.cuda.empty_cache()
            except Exception as e:  # noqa: BLE001 - the headline must not be lost to a failure of the wider leg
                layer70 = {"error": f"{type(e).__name__}: {e}"}
        leg_status["layer_70b"] = k.device_status()
        if world > 1 or args.layer == "70b":
            prefill = run_prefill_tp(k, dev, stream, rank, world)
        leg_status["prefill_tp"] = k.device_status()

    # ---- second half of the headline metric: W4 greedy decode tokens/s of a Qwen2.5-7B-shaped model (512-token prompt,
    # 256 new tokens, batch 1, tensor parallel over the ranks)
    decode = None
    if not args.no_decode and args.layer == "7b":
        try:
            from nanoserve_b200.qwen import decode_rate
            d = decode_rate(k, dev, rank=rank, world=world, fused_gather=not args.tp_collective)
            t = torch.tensor([d["ms_per_token"]], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            d["ms_per_token"] = float(t.item())
            d["tok_s"] = 1e3 / d["ms_per_token"]
            d["hbm_frac_of_" + which] = d["weight_bytes_per_token_per_rank"] / (d["ms_per_token"] * 1e-3) / 1e9 / peaks["hbm_gbs"]
            decode = d
        except Exception as e:  # the GEMV line must not be lost to a failure of the wider leg
            decode = {"error": f"{type(e).__name__}: {e}"}

    # ---- max over ranks
    times = torch.tensor([t_dev, t_e2e_wall, t_e2e_eager], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    t_dev, t_e2e_wall, t_e2e_eager = times.tolist()
    status = k.device_status()
    if status != 0:
        raise SystemExit(f"rank {rank}: device status {status}: a kernel reported a time-out; numbers are invalid "
                         f"(status after each leg: {leg_status})")

    if rank == 0:
        metric = METRIC if args.layer == "7b" else METRIC_70B
        layer_name = "Qwen2.5-7B-shaped" if args.layer == "7b" else "70B-class (hidden 8192, intermediate 28672)"
        # which kernel and launch shape the library picks for each launch of the pass (this rank's shard)
        from nanoserve_b200.tp import ShardedLayer as _SL
        groups = [(n, (n,)) for n in ORDER] if seven else list(_SL.FUSED)
        plans = {f: k.gemv_describe(M, sum(shapes[n][0] for n in names) // world, shapes[names[0]][1], G, args.flags)
                 for f, names in groups}
        line = {
            "metric": metric if M == 1 else metric.replace("M=1", f"M={M}"), "value": nbytes * args.steps / t_dev / 1e9,
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": t_dev / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {
                "workload": f"decode GEMV pass over the 7 linears of a {layer_name} layer, M={M}, int4 g128",
                "launches": ("7 GEMV launches per pass" if seven else
                             "4 GEMV launches per pass: q|k|v and gate|up as row-concatenated matrices (same arithmetic)"
                             "; a GEMV whose K is cut into slices across CTAs is followed by the kernel that adds them "
                             "(counted in gpu_launches, see plans)"),
                "parallelism": (f"tp{world}, all-gather " + ("fused into the GEMVs (peer stores + arrival counters; each "
                                                             "launch waits for the previous gathered row in-kernel)"
                                                             if fused_gather else "by NCCL at the 4 layer boundaries"))
                if world > 1 else "single GPU",
                "l2": f"weights rotate through {n_copies} layer copies ({resident * world / 1e6:.0f} MB) > 126 MB L2",
                "bytes_per_step": nbytes, "launch": "one CUDA graph per layer copy, replayed in rotation",
                "timed": f"{blocks[0]} blocks of {args.steps} steps ({t_dev * blocks[0] * 1e3:.1f} ms in all), mean per step",
                "seeds": "X 1/2, layer copy c: 1000+c", "flags": args.flags,
                "plans": plans,
            },
            "e2e": {"value": nbytes * args.steps / t_e2e_wall / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": t_e2e_wall / args.steps * 1e3, "path": e2e_path,
                    "per_launch_api": {"value": nbytes * args.steps / t_e2e_eager / 1e9,
                                       "ms_per_step": t_e2e_eager / args.steps * 1e3,
                                       "path": "Kernels.w4_linear per launch (ctypes -> C ABI), same copies, no graph"}},
            "gpu_launches": lb.launches_per_step() * args.steps * (blocks[0] + 1),
            "clocks": clocks,
        }
        if roof is not None:
            line["roofline"] = roof
        if check is not None:
            line["tp_check"] = check
        if ref_gpu is not None:
            line["ref_gpu"] = ref_gpu
        if sweep is not None:
            line["sweep"] = sweep
        if layer70 is not None:
            line["layer_70b"] = layer70
        if decode is not None:
            line["decode"] = decode
        if prefill is not None:
            line["prefill_tp"] = prefill
        if world == 1 and not args.no_cpu_baseline:
            one, _ = cpu_layer_pass(1, 1)
            n = max(1, min(8, int(15.0 / max(one, 1e-3))))
            dt, used = cpu_layer_pass(1, n)
            line["cpu_baseline"] = {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": used, "kind": "port",
                                    "sample": f"{n} full layer passes at M=1 on one host thread (as the reference "
                                              f"runs its check), {dt:.2f} s per pass"}
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        # Captured graphs hold peer waits or NCCL work; tearing the communicator down under them can block.  Everything
        # is measured and printed: synchronise, meet once more, and leave without running the destructors.
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
