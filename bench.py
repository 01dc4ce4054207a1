#!/usr/bin/env python
"""Benchmark of the quantized-weight matmul path on B200.

Headline workload (the decode half of the Qwen3-4B-shaped config): a stack of 4-bit
group-64 linears (36 layers x {q 2560->4096, k, v 2560->1024, o 4096->2560, gate, up
2560->9728, down 9728->2560}), random-init, one token (M=1) per step.  Metric: HBM GB/s on
the algorithmic bytes of a token (packed codes + bf16 scales/biases + activations in/out).
Every linear is one call of the C ABI (`lisa_cuda_quantized_matmul_ex`), 252 launches per
token, replayed from a CUDA graph.  The weights of a token (2.04 GB) are far larger than
L2, so no flush is needed between steps.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--mode decode|prefill]

`--mode prefill` makes the second half of the same config the headline: the same stack at
M=2048 through the tcgen05 GEMM, metric bf16 TFLOP/s against the measured dense bf16 peak.  The
default (decode) line carries a short prefill measurement as well, under "qmm".

One JSON line on stdout (rank 0).  With N > 1 (torchrun) each rank decodes its own token
stream through its own replica ("replicas only": this config has no exchange step), value is
the aggregate.  `--impl reference` times the CPU restatement of the reference's Rust dequant
+ scalar matmul (oracle/) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, Q_OUT, KV_OUT, INTER, LAYERS = 2560, 4096, 1024, 9728, 36
GROUP, BITS = 64, 4
# (name, K, N, which input buffer)
LINEARS = [("q", HIDDEN, Q_OUT, "h"), ("k", HIDDEN, KV_OUT, "h"), ("v", HIDDEN, KV_OUT, "h"),
           ("o", Q_OUT, HIDDEN, "a"), ("gate", HIDDEN, INTER, "h"), ("up", HIDDEN, INTER, "h"),
           ("down", INTER, HIDDEN, "i")]
# linears of a layer that read the same activations: one launch each group in the sibling form
SIBLINGS = [(0, 1, 2), (3,), (4, 5), (6,)]


def linear_bytes(k: int, n: int, m: int = 1) -> int:
    """Algorithmic bytes of one linear: codes + bf16 scale and bias + x in + y out."""
    return n * k * BITS // 8 + 2 * n * (k // GROUP) * 2 + m * k * 2 + m * n * 2


def token_bytes(layers: int = LAYERS) -> int:
    return layers * sum(linear_bytes(k, n) for _, k, n, _ in LINEARS)


def token_weights(layers: int = LAYERS) -> int:
    return layers * sum(k * n for _, k, n, _ in LINEARS)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def tensor_peak():
    """Dense bf16 TFLOP/s for a kernel timed inside a long step (the sustained figure)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops_sustained)"
    return 1400.0, "fallback (1.4 PFLOP/s sustained, earlier measurement on this pool)"


def tensor_peaks():
    """(sustained, burst) dense bf16 TFLOP/s and where they come from."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["bf16_tflops_sustained"]), float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json)"
    return 1400.0, 1590.0, "fallback (1.4 / 1.59 PFLOP/s, earlier measurement on this pool)"


def leg_summary(line):
    """{workload, ms, value, unit, roofline} of a leg from its full result line."""
    unit = line["unit"]
    n = max(int(line.get("n_gpus", 1)), 1)
    per_gpu = line["value"] / n
    if unit == "TFLOP/s":
        sus, burst, src = tensor_peaks()
        roof = {"bound": "tensor", "frac": per_gpu / sus, "frac_of_burst": per_gpu / burst, "peak": sus, "peak_burst": burst,
                "peak_source": src + ", per GPU"}
    else:
        peak, src = peaks()
        roof = {"bound": "hbm", "frac": per_gpu / peak, "peak": peak, "peak_source": src + ", per GPU"}
    return {"workload": line["config"]["workload"], "parallelism": line["config"].get("parallelism"), "ms": line["ms_per_step"],
            "value": line["value"], "unit": unit, "n_gpus": n, "scaling": line.get("scaling"), "steps": line.get("steps"),
            "gpu_launches": line.get("gpu_launches"), "roofline": roof}


# dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the same launches, from the
# ncu captures (qmv_tc_kernel on 4 layers of the decode stack; qmm_affine_kernel
# on 2 layers of the prefill stack).  Traffic grows in proportion to the units processed, so the ratio
# carries over to a full launch.
DRAM_TRAFFIC_RATIO = {"decode": 1.005, "prefill": 0.578}
PREFILL_M = 2048


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for name, val in zip(names, r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_sample_layers() -> int:
    return 4


_CPU_MATS = {}


def cpu_sample(seed: int, layers: int):
    """Host copies of `layers` layers of the stack (same shapes and distributions, seed `seed`)."""
    import numpy as np
    from tests import util

    key = (seed, layers)
    if key not in _CPU_MATS:
        rng = np.random.default_rng(seed)
        mats = []
        for _ in range(layers):
            for _, k, n, _ in LINEARS:
                mats.append((util.affine_weights(rng, n, k, BITS, GROUP), util.activations(rng, 1, k)))
        _CPU_MATS[key] = mats
    return _CPU_MATS[key]


def run_cpu_baseline(seed: int, layers: int):
    """Times the oracle (port of the reference's Rust dequant + scalar f32 matmul, output rows
    split over all host cores) on `layers` layers of the stack.  Returns (GB/s, seconds, cores)."""
    from oracle import oracle as O

    cores = os.cpu_count() or 1
    mats = cpu_sample(seed, layers)
    t0 = time.perf_counter()
    for (w, s, b), x in mats:
        O.affine_matmul(x, w, s, b, GROUP, BITS, round_weight_bf16=True, threads=cores)
    dt = time.perf_counter() - t0
    return token_bytes(layers) / dt / 1e9, dt, cores


def reference_arm(args, rank: int):
    if rank != 0:
        return
    layers = cpu_sample_layers()
    times = []
    for _ in range(args.warmup):
        run_cpu_baseline(0, layers)
    cores = os.cpu_count() or 1
    for _ in range(args.steps):
        gbs, dt, cores = run_cpu_baseline(0, layers)
        times.append(dt)
    dt = statistics.mean(times)
    value = token_bytes(layers) / dt / 1e9
    sample = f"{layers} of {LAYERS} layers of the stack (7 linears each), M=1, seed 0; weights generated on the host"
    line = {
        "impl": "reference", "metric": "4-bit qmv HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 * LAYERS / layers,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's Rust dequant + scalar f32 matmul (the Rust crate cannot be "
                "built here: no Rust toolchain); ms_per_step is the sample scaled to a full token",
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int, launches_per_token: int = 0):
    if not launches_per_token:  # the default call pattern of this bench (also what the reference arm names)
        launches_per_token = LAYERS * (len(SIBLINGS) if os.environ.get("LISA_BENCH_SIBLINGS", "1") == "1" else 7)
    return {"workload": "configs[1] decode: Qwen3-4B-shaped 4-bit gs64 linear stack, 36 layers x 7 linears, M=1",
            "calls": ("q|k|v and gate|up through lisa_cuda_quantized_matmul_siblings (linears that read the same x: one "
                      "launch), o and down through lisa_cuda_quantized_matmul"
                      if launches_per_token < LAYERS * 7 else "one lisa_cuda_quantized_matmul call per linear"),
            "bytes_per_token": token_bytes(), "weights_per_token": token_weights(), "launches_per_token": launches_per_token,
            "l2": "inputs larger than L2 (2.04 GB of weights per step)",
            "parallelism": "replicas only" if n_gpus > 1 else "single GPU"}


class DecodeStack:
    """Device-resident synthetic weights and the per-token launch sequence."""

    def __init__(self, dev, seed: int, layers: int = LAYERS):
        import torch
        from lisa_b200 import _cabi

        self.torch = torch
        self.dev = dev
        self.layers = layers
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        self.weights = []
        for _ in range(layers):
            per = []
            for _, k, n, src in LINEARS:
                w = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k * BITS // 32), dtype=torch.int32, device=dev, generator=g)
                s = (torch.randn((n, k // GROUP), device=dev, generator=g) * 0.02).abs().to(torch.bfloat16)
                b = (torch.randn((n, k // GROUP), device=dev, generator=g) * 0.01).to(torch.bfloat16)
                y = torch.empty((1, n), dtype=torch.bfloat16, device=dev)
                per.append((w, s, b, y, k, n, src))
            self.weights.append(per)
        self.inputs = {"h": torch.randn((1, HIDDEN), device=dev, generator=g).to(torch.bfloat16),
                       "a": torch.randn((1, Q_OUT), device=dev, generator=g).to(torch.bfloat16),
                       "i": torch.randn((1, INTER), device=dev, generator=g).to(torch.bfloat16)}
        self.flags = _cabi.FLAG_PDL if os.environ.get("LISA_BENCH_PDL", "1") != "0" else 0
        if os.environ.get("LISA_BENCH_SIMPLE", "0") == "1":
            self.flags |= _cabi.FLAG_FORCE_QMV_SIMPLE
        if os.environ.get("LISA_BENCH_TC", "1") == "0":  # the mma.sync kernel instead of the tensor-memory one
            self.flags |= _cabi.FLAG_FORCE_QMV
        self.graph = None
        self.siblings = os.environ.get("LISA_BENCH_SIBLINGS", "1") == "1"
        self.calls = []  # sibling form: one argument pack per launch
        import ctypes as C
        for per in self.weights:
            for group in SIBLINGS:
                c = len(group)
                wp, sp, bp, yp, ns = (C.c_void_p * c)(), (C.c_void_p * c)(), (C.c_void_p * c)(), (C.c_void_p * c)(), (C.c_int64 * c)()
                for j, i in enumerate(group):
                    w, s, b, y, k, n, src = per[i]
                    wp[j], sp[j], bp[j], yp[j], ns[j] = w.data_ptr(), s.data_ptr(), b.data_ptr(), y.data_ptr(), n
                self.calls.append((self.inputs[src].data_ptr(), k, c, wp, sp, bp, ns, yp))

    def launches_per_token(self) -> int:
        return len(self.calls) if self.siblings else self.layers * len(LINEARS)

    def token(self):
        from lisa_b200 import _cabi

        lib = _cabi.lib()
        stream = self.torch.cuda.current_stream().cuda_stream
        if self.siblings:
            for x, k, c, wp, sp, bp, ns, yp in self.calls:
                _cabi.check(lib.lisa_cuda_quantized_matmul_siblings(stream, x, 1, k, c, wp, sp, bp, ns, 1, GROUP, BITS, 0, yp,
                                                                    self.flags))
            return
        for per in self.weights:
            for w, s, b, y, k, n, src in per:
                rc = lib.lisa_cuda_quantized_matmul_ex(stream, self.inputs[src].data_ptr(), 1, k, w.data_ptr(),
                                                       s.data_ptr(), b.data_ptr(), n, 1, GROUP, BITS, 0, y.data_ptr(),
                                                       self.flags)
                _cabi.check(rc)

    def capture(self):
        torch = self.torch
        self.token()  # sets kernel attributes outside capture
        torch.cuda.synchronize()
        if os.environ.get("LISA_BENCH_GRAPH", "1") == "0":
            return
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                self.token()
        torch.cuda.current_stream().wait_stream(side)
        self.graph = graph

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.token()

    def time_other_form(self, steps: int):
        """ms per token of the other call pattern (one call per linear when the sibling form is the timed
        one, and the reverse), graph-captured the same way."""
        torch = self.torch
        keep = (self.siblings, self.graph)
        self.siblings, self.graph = (not self.siblings), None
        try:
            self.capture()
            for _ in range(3):
                self.step()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                self.step()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / steps, self.launches_per_token()
        finally:
            self.siblings, self.graph = keep

    # ---- prefill: the same weights at M = PREFILL_M through the tensor-core GEMM
    def prefill_setup(self, m: int = PREFILL_M):
        torch = self.torch
        g = torch.Generator(device=self.dev)
        g.manual_seed(1234)
        self.pm = m
        from lisa_b200 import _cabi
        self.pflags = _cabi.FLAG_PDL if os.environ.get("LISA_BENCH_PREFILL_PDL", "1") != "0" else 0
        self.pin = {"h": torch.randn((m, HIDDEN), device=self.dev, generator=g).to(torch.bfloat16),
                    "a": torch.randn((m, Q_OUT), device=self.dev, generator=g).to(torch.bfloat16),
                    "i": torch.randn((m, INTER), device=self.dev, generator=g).to(torch.bfloat16)}
        self.pout = {n: torch.empty((m, n), dtype=torch.bfloat16, device=self.dev) for n in (Q_OUT, KV_OUT, HIDDEN, INTER)}
        # sibling form: every linear of a launch needs its own output
        import ctypes as C
        self.pouts = [torch.empty((m, n), dtype=torch.bfloat16, device=self.dev) for _, _, n, _ in LINEARS]
        self.pcalls = []
        for per in self.weights:
            for group in SIBLINGS:
                c = len(group)
                wp, sp, bp, yp, ns = (C.c_void_p * c)(), (C.c_void_p * c)(), (C.c_void_p * c)(), (C.c_void_p * c)(), (C.c_int64 * c)()
                for j, i in enumerate(group):
                    w, s, b, _, k, n, src = per[i]
                    wp[j], sp[j], bp[j], yp[j], ns[j] = w.data_ptr(), s.data_ptr(), b.data_ptr(), self.pouts[i].data_ptr(), n
                self.pcalls.append((self.pin[src].data_ptr(), k, c, wp, sp, bp, ns, yp))

    def prefill(self):
        from lisa_b200 import _cabi

        lib = _cabi.lib()
        stream = self.torch.cuda.current_stream().cuda_stream
        if self.siblings:
            for x, k, c, wp, sp, bp, ns, yp in self.pcalls:
                _cabi.check(lib.lisa_cuda_quantized_matmul_siblings(stream, x, self.pm, k, c, wp, sp, bp, ns, 1, GROUP, BITS, 0, yp,
                                                                    self.pflags))
            return
        for per in self.weights:
            for w, s, b, _, k, n, src in per:
                rc = lib.lisa_cuda_quantized_matmul_ex(stream, self.pin[src].data_ptr(), self.pm, k, w.data_ptr(),
                                                       s.data_ptr(), b.data_ptr(), n, 1, GROUP, BITS, 0,
                                                       self.pout[n].data_ptr(), self.pflags)
                _cabi.check(rc)

    def prefill_flops(self) -> float:
        return 2.0 * self.pm * token_weights(self.layers)

    def prefill_bytes(self) -> int:
        return self.layers * sum(linear_bytes(k, n, self.pm) for _, k, n, _ in LINEARS)


def time_prefill(torch, stack, steps: int, warmup: int):
    """ms per prefill pass of the stack (CUDA events on the launching stream)."""
    for _ in range(warmup):
        stack.prefill()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        stack.prefill()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS, help="fewer layers for profiler captures only")
    ap.add_argument("--skip-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--skip-legs", action="store_true", help="headline only: skip the legs of the other workloads")
    ap.add_argument("--mode", default="decode", choices=["decode", "prefill", "shard", "moe", "gguf"],
                    help="decode: M=1 GEMV stack, HBM GB/s (headline); prefill: M=2048 GEMM stack, bf16 TFLOP/s; "
                         "shard: configs[2] 2-bit MLP stack, N-sharded over the ranks with an all-gather; "
                         "moe: configs[3] routed experts, expert-parallel over the ranks with all-to-all; "
                         "gguf: configs[4] Q2_K / Q4_K matvec (M=1) and tensor-core matmul (M=512), one GPU")
    ap.add_argument("--rows", dest="m", type=int, default=1, help="rows of x for --mode shard (1, 8 or 512)")
    ap.add_argument("--tokens", type=int, default=4096, help="tokens per rank for --mode moe (1, 64 or 4096)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU arm)")
    if rank == 0:
        entry.build()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
    from lisa_b200 import ops

    warmup = max(args.warmup, 3)
    if args.mode in ("shard", "moe"):
        sharded_main(args, torch, dist, dev, rank, world, warmup)
        return
    if args.mode == "gguf":
        gguf_main(args, torch, dev, rank, warmup)
        return
    stack = DecodeStack(dev, seed=rank, layers=args.layers)
    if args.mode == "prefill":
        prefill_main(args, torch, dist, stack, rank, local_rank, world, warmup)
        return
    before = ops.launch_count()
    stack.capture()
    launches_per_token = (ops.launch_count() - before) // (2 if stack.graph is not None else 1)
    bytes_token = token_bytes(args.layers)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        stack.step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- device-resident timing: inputs already in HBM
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for i in range(args.steps):
        stack.step()
        ev[i + 1].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    step_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    # ---- end to end: host buffers in, host result out, every step
    pinned_in = {k: v.cpu().pin_memory() for k, v in stack.inputs.items()}
    last_y = stack.weights[-1][-1][3]
    pinned_out = torch.empty_like(last_y, device="cpu").pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in pinned_in.values())
    d2h = pinned_out.numel() * pinned_out.element_size()
    for _ in range(2):
        for k, v in pinned_in.items():
            stack.inputs[k].copy_(v, non_blocking=True)
        stack.step()
        pinned_out.copy_(last_y, non_blocking=True)
        torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        for k, v in pinned_in.items():
            stack.inputs[k].copy_(v, non_blocking=True)
        stack.step()
        pinned_out.copy_(last_y, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result before the next token
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    # ---- the same step for about a second more (the contract's K steps last tens of milliseconds: too short for
    # a power cap to show), while the clock sampler keeps running
    long_steps = 1000 if args.layers == LAYERS else 50
    l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0.record()
    for _ in range(long_steps):
        stack.step()
    l1.record()
    barrier()
    long_ms = l0.elapsed_time(l1)
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = float(t[0]), float(t[1])
    status = ops.device_status()

    legs = {}
    if rank == 0:
        value = world * bytes_token * args.steps / (total_ms * 1e-3) / 1e9
        e2e_value = world * bytes_token * args.steps / (e2e_ms * 1e-3) / 1e9
        peak, peak_src = peaks()
        per_gpu = bytes_token * args.steps / (total_ms * 1e-3) / 1e9
        line = {
            "metric": "4-bit qmv HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8*s8->s32, f32 epilogue", "data": "synthetic",
            "config": workload_config(world, launches_per_token),
            "pct_of_8TBps": 100.0 * per_gpu / 8000.0,
            "tokens_per_s": world * args.steps / (total_ms * 1e-3),
            "ms_per_step_median": statistics.median(step_ms),
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                         "traffic": (DRAM_TRAFFIC_RATIO["decode"] * bytes_token / max(launches_per_token, 1)
                                     if DRAM_TRAFFIC_RATIO["decode"] else None),
                         "kernel": "qmv_tc_kernel<4>", "peak_source": peak_src,
                         "bytes_per_launch_avg": bytes_token / max(launches_per_token, 1),
                         "us_per_launch_avg": 1e3 * total_ms / args.steps / max(launches_per_token, 1)},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches_per_token * args.steps,
            "clocks": clocks, "device_status": status,
            "launch": {"graph": stack.graph is not None, "pdl": bool(stack.flags & 8), "layers": args.layers},
            "long_run": {"steps": long_steps, "ms_per_step": long_ms / long_steps,
                         "value": bytes_token * long_steps / (long_ms * 1e-3) / 1e9, "unit": "GB/s per GPU (rank 0)"},
        }
        if args.layers == LAYERS:
            oms, olaunch = stack.time_other_form(min(args.steps, 20))
            line["other_call_pattern"] = {"calls": workload_config(world, olaunch)["calls"], "launches_per_token": olaunch,
                                          "ms_per_step": oms, "value": bytes_token / (oms * 1e-3) / 1e9, "unit": "GB/s"}
        # the prefill half of the same config (full stack, M = 2048), 20 passes
        stack.prefill_setup()
        psteps = 20 if args.layers == LAYERS else 3
        pms = time_prefill(torch, stack, steps=psteps, warmup=3)
        sus, burst, tsrc = tensor_peaks()
        tf = stack.prefill_flops() / (pms * 1e-3) / 1e12
        line["qmm"] = {"metric": "qmm bf16 TFLOP/s", "value": tf, "m": PREFILL_M, "ms_per_pass": pms, "passes": psteps,
                       "frac_of_bf16_peak": tf / sus, "peak": sus, "frac_of_burst_peak": tf / burst, "peak_burst": burst,
                       "peak_source": tsrc,
                       "launches_per_pass": args.layers * (len(SIBLINGS) if stack.siblings else 7), "kernel": "qmm_affine_kernel<4>"}
        legs["configs[1] prefill M=2048"] = {
            "workload": f"configs[1] prefill: the same stack, {args.layers} layers x 7 linears, M={PREFILL_M}", "ms": pms,
            "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": psteps,
            "roofline": {"bound": "tensor", "frac": tf / sus, "frac_of_burst": tf / burst, "peak": sus, "peak_burst": burst,
                         "peak_source": tsrc}}
        del stack.pin, stack.pout, stack.pouts
        if args.layers == LAYERS and not args.skip_legs:
            # configs[4]: GGUF Q2_K / Q4_K, both shapes, M in {1, 512}
            for r in gguf_legs(torch, dev, steps=20, warmup=3):
                key = f"configs[4] {r['format']} K={r['k']} N={r['n']} M={r['m']}"
                if "experts" in r:
                    key = f"GGUF expert form {r['format']} K={r['k']} N={r['n']}, one token, top-{r['top_k']} of {r['experts']}"
                if r["m"] == 1:
                    hp, hsrc = peaks()
                    legs[key] = {"workload": key, "ms": r["us"] * 1e-3, "value": r["GB/s"], "unit": "GB/s", "n_gpus": 1, "steps": 20,
                                 "roofline": {"bound": "hbm", "frac": r["GB/s"] / hp, "peak": hp, "peak_source": hsrc}}
                else:
                    legs[key] = {"workload": key, "ms": r["us"] * 1e-3, "value": r["TFLOP/s"], "unit": "TFLOP/s", "n_gpus": 1, "steps": 20,
                                 "roofline": {"bound": "tensor", "frac": r["TFLOP/s"] / sus, "frac_of_burst": r["TFLOP/s"] / burst,
                                              "peak": sus, "peak_burst": burst, "peak_source": tsrc}}
        if not args.skip_cpu:
            layers = cpu_sample_layers()
            gbs, dt, cores = run_cpu_baseline(0, layers)
            line["cpu_baseline"] = {
                "value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                "sample": f"{layers} of {LAYERS} layers (7 linears each), M=1, seed 0, {dt:.2f} s; "
                          "restatement of the reference's Rust dequant + scalar f32 matmul"}
    # ---- the other workloads, every rank: the 2-bit stack N-sharded over the ranks (all-gather fused into the
    # kernels' epilogues, peer barrier) and the routed experts expert-parallel (all-to-all); with one rank the same
    # code runs unsharded, which is the baseline of the scaling curve
    if args.layers == LAYERS and not args.skip_legs:
        del stack
        torch.cuda.empty_cache()
        if world > 1:
            dist.barrier()
        for m in (1, 8, 512):
            res = sharded_leg(LegArgs("shard", m=m, steps=10), torch, dist, dev, rank, world, 3)
            if rank == 0:
                legs[f"configs[2] M={m}"] = leg_summary(res)
            torch.cuda.empty_cache()
        for tokens in (1, 64, 4096):
            res = sharded_leg(LegArgs("moe", tokens=tokens, steps=10), torch, dist, dev, rank, world, 3)
            if rank == 0:
                legs[f"configs[3] T={tokens}"] = leg_summary(res)
            torch.cuda.empty_cache()
    if rank == 0:
        line["configs"] = legs
        line["device_status"] = ops.device_status()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def prefill_main(args, torch, dist, stack, rank, local_rank, world, warmup):
    """Headline = the prefill half of the config: M=2048 through qmm_affine_kernel, TFLOP/s."""
    from lisa_b200 import ops

    stack.prefill_setup()
    before = ops.launch_count()
    stack.prefill()
    launches = ops.launch_count() - before
    for _ in range(warmup - 1):
        stack.prefill()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = time_prefill(torch, stack, steps=args.steps, warmup=0)
    # end to end: activations from pinned host memory in, last output back, every pass
    pinned_in = {k: v.cpu().pin_memory() for k, v in stack.pin.items()}
    out = stack.pouts[-1] if stack.siblings else stack.pout[HIDDEN]
    pinned_out = torch.empty_like(out, device="cpu").pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in pinned_in.values())
    d2h = pinned_out.numel() * pinned_out.element_size()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        for k, v in pinned_in.items():
            stack.pin[k].copy_(v, non_blocking=True)
        stack.prefill()
        pinned_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=torch.device("cuda", local_rank))
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    if rank == 0:
        flops = stack.prefill_flops()
        per_gpu = flops / (ms * 1e-3) / 1e12
        peak, src = tensor_peak()
        ratio = DRAM_TRAFFIC_RATIO["prefill"]
        cfg = workload_config(world)
        cfg["workload"] = ("configs[1] prefill: Qwen3-4B-shaped 4-bit gs64 linear stack, "
                           f"{args.layers} layers x 7 linears, M={PREFILL_M}")
        cfg["launches_per_pass"] = launches
        cfg["l2"] = "inputs larger than L2 (2.04 GB of weights per pass)"
        line = {
            "metric": "qmm bf16 TFLOP/s", "value": world * per_gpu, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                         "frac": per_gpu / peak,
                         "traffic": ratio * stack.prefill_bytes() / launches if ratio else None,
                         "kernel": "qmm_affine_kernel<4>", "peak_source": src},
            "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
            "gpu_launches": launches * args.steps, "clocks": clocks, "device_status": ops.device_status(),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def gguf_legs(torch, dev, steps, warmup):
    """configs[4]: GGUF Q2_K / Q4_K, K=7168 N=18432 and K=18432 N=7168, M=1 (matvec, HBM GB/s on the block
    bytes) and M=512 (tensor-core matmul with a workspace, TFLOP/s).  Uniform random code and scale bytes,
    d, dmin ~ |N(0, 0.01)| as f16, activations ~ N(0, 1).  One result per (format, shape, M)."""
    from lisa_b200 import _cabi, ops

    g = torch.Generator(device=dev)
    g.manual_seed(0)
    results = []
    for fmt, block, code, d_at in (("Q4K", 144, _cabi.GGUF_Q4_K, 0), ("Q2K", 84, _cabi.GGUF_Q2_K, 80)):
        for k, n in ((7168, 18432), (18432, 7168)):
            nb = k // 256
            w = torch.randint(0, 256, (n, nb, block), dtype=torch.uint8, device=dev, generator=g)
            dd = (torch.randn((n, nb, 2), device=dev, generator=g) * 0.01).abs().to(torch.float16).view(torch.uint8)
            w[:, :, d_at:d_at + 4] = dd.reshape(n, nb, 4)
            w = w.reshape(n, nb * block).contiguous()
            for m in (1, 512):
                x = torch.randn((m, k), device=dev, generator=g)
                ws = torch.empty(_cabi.lib().lisa_cuda_gguf_packed_matmul_workspace_bytes(m, nb * block, code),
                                 dtype=torch.uint8, device=dev)
                fn = (lambda: ops.packed_matmul(fmt, w, x, workspace=ws)) if m > 1 else (lambda: ops.packed_matvec(fmt, w, x))
                for _ in range(warmup):
                    fn()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(steps):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) / steps * 1e3
                results.append({"format": fmt, "k": k, "n": n, "m": m, "us": us,
                                "GB/s": w.numel() / us / 1e3 if m == 1 else None,
                                "TFLOP/s": 2.0 * m * n * k / us / 1e6 if m > 1 else None})
            del w
        # the expert form at decode size: one token, top-8 of 64 experts, the GGUF checkpoints' routed down projection
        # (2048 -> 4096); bytes = the eight experts' rows
        e, k, n, top_k = 64, 2048, 4096, 8
        nb = k // 256
        w = torch.randint(0, 256, (e, n, nb, block), dtype=torch.uint8, device=dev, generator=g)
        dd = (torch.randn((e, n, nb, 2), device=dev, generator=g) * 0.01).abs().to(torch.float16).view(torch.uint8)
        w[:, :, :, d_at:d_at + 4] = dd.reshape(e, n, nb, 4)
        w = w.reshape(e, n, nb * block).contiguous()
        x = torch.randn((1, top_k, k), device=dev, generator=g)
        perms = [torch.randperm(e, device=dev, generator=g)[:top_k].to(torch.int32).reshape(1, top_k) for _ in range(8)]
        for i in range(warmup):
            ops.expert_matvec(fmt, w, x, perms[i % 8])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            ops.expert_matvec(fmt, w, x, perms[i % 8])
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / steps * 1e3
        results.append({"format": fmt, "k": k, "n": n, "m": 1, "experts": e, "top_k": top_k, "us": us,
                        "GB/s": top_k * n * nb * block / us / 1e3, "TFLOP/s": None})
        del w
    return results


def gguf_main(args, torch, dev, rank, warmup):
    if rank != 0:
        return
    from lisa_b200 import ops

    results = gguf_legs(torch, dev, args.steps, warmup)
    best = max(r["TFLOP/s"] for r in results if r["TFLOP/s"])
    print(json.dumps({"metric": "GGUF K-quant matmul TFLOP/s (M=512, best of the four)", "value": best, "unit": "TFLOP/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": warmup, "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "configs[4]: GGUF Q2_K/Q4_K, K=7168 N=18432 and K=18432 N=7168, M in {1, 512}"},
                      "results": results, "device_status": ops.device_status()}), flush=True)


def sharded_main(args, torch, dist, dev, rank, world, warmup):
    line = sharded_leg(args, torch, dist, dev, rank, world, warmup)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


class LegArgs:
    """The arguments sharded_leg reads, for the legs of the default line."""

    def __init__(self, mode, m=1, tokens=4096, steps=10, layers=LAYERS):
        self.mode, self.m, self.tokens, self.steps, self.layers = mode, m, tokens, steps, layers


def sharded_leg(args, torch, dist, dev, rank, world, warmup):
    """configs[2] (N-sharded 2-bit MLP stack + all-gather) and configs[3] (expert-parallel routed experts +
    all-to-all).  With one rank the same code runs unsharded and no collective is issued.  Returns the result
    line on rank 0 (None elsewhere); every rank must call it."""
    from lisa_b200 import ops, parallel
    from lisa_b200.quant import QuantizedLinear, SwitchGlu

    g = torch.Generator(device=dev)
    g.manual_seed(0)
    closers = []

    def affine(lead, n, k, bits):
        w = torch.randint(-2 ** 31, 2 ** 31 - 1, lead + (n, k * bits // 32), dtype=torch.int32, device=dev, generator=g)
        s = (torch.randn(lead + (n, k // GROUP), device=dev, generator=g) * 0.02).abs().to(torch.bfloat16)
        b = (torch.randn(lead + (n, k // GROUP), device=dev, generator=g) * 0.01).to(torch.bfloat16)
        return w, s, b

    if args.mode == "shard":
        hidden, inter, bits, m = 5120, 17408, 2, args.m
        layers = args.layers if args.layers != LAYERS else 64
        shapes = [(hidden, inter), (hidden, inter), (inter, hidden)]  # gate, up, down (K, N)
        lins = []
        for _ in range(layers):
            per = []
            for k, n in shapes:
                n0, n1 = parallel.shard_rows(n, world, rank)
                w, s, b = affine((), n1 - n0, k, bits)  # this rank's rows only: full matrices never exist
                per.append(parallel.ShardedQuantizedLinear(w, s, b, n, n0, n1, GROUP, bits))
            lins.append(per)
        xs = {hidden: torch.randn((m, hidden), device=dev, generator=g).to(torch.bfloat16),
              inter: torch.randn((m, inter), device=dev, generator=g).to(torch.bfloat16)}

        # the GEMV (m <= 8) or GEMM whose epilogue stores into every rank's buffer + peer barrier (no NCCL on
        # the data path); LISA_BENCH_FUSED=0: local kernel + NCCL all-gather
        fused = world > 1 and os.environ.get("LISA_BENCH_FUSED", "1") != "0"
        fused_sib = fused and m <= 8 and os.environ.get("LISA_BENCH_SIBLINGS", "1") == "1"
        if fused_sib:  # gate|up: one launch and one barrier for both
            lins = [[parallel.FusedShardedSiblings(per[:2], max_rows=m), parallel.FusedShardedLinear(per[2], max_rows=m)]
                    for per in lins]
        elif fused:
            lins = [[parallel.FusedShardedLinear(lin, max_rows=m) for lin in per] for per in lins]
        if fused:
            closers.extend(obj for per in lins for obj in per)

        # one GPU, few rows: gate and up read the same x, so they go out as one sibling launch
        siblings = world == 1 and m <= 8 and os.environ.get("LISA_BENCH_SIBLINGS", "1") == "1"

        def step():
            for per in lins:
                if fused_sib:
                    per[0].forward(xs[hidden])
                    per[1].forward(xs[inter])
                    continue
                if siblings:
                    ops.quantized_matmul_siblings(xs[hidden], [(l.weight, l.scales, l.biases) for l in per[:2]], True, GROUP, bits)
                    ops.quantized_matmul(xs[inter], per[2].weight, per[2].scales, per[2].biases, True, GROUP, bits)
                    continue
                for lin, (k, n) in zip(per, shapes):
                    if world > 1:
                        lin.forward(xs[k])
                    else:
                        ops.quantized_matmul(xs[k], lin.weight, lin.scales, lin.biases, True, GROUP, bits)

        weights = layers * sum(k * n for k, n in shapes)
        work_bytes = layers * sum(n * k * bits // 8 + 2 * n * (k // GROUP) * 2 + m * k * 2 + m * n * 2 for k, n in shapes)
        flops = 2.0 * m * weights
        name = f"configs[2]: 27B-class 2-bit gs64 MLP stack, {layers} layers x (gate, up, down), M={m}"
        par = (("single GPU, gate|up as one sibling launch" if siblings else "single GPU") if world == 1 else
               f"N-sharded over {world} ranks, all-gather fused into the {'GEMV' if m <= 8 else 'GEMM'} epilogue (peer stores) + peer barrier{', gate|up as one sibling launch' if fused_sib else ''}" if fused
               else f"N-sharded over {world} ranks, NCCL all-gather of every output")
        scaling = "strong"
    else:
        experts, top_k, hidden, inter, tokens = 128, 8, 2048, 768, args.tokens
        e0, e1 = parallel.expert_range(experts, world, rank)
        mk = lambda n, k: QuantizedLinear(*affine((e1 - e0,), n, k, 4), GROUP, 4)
        block = SwitchGlu(mk(inter, hidden), mk(inter, hidden), mk(hidden, inter), top_k)
        x = torch.randn((tokens, hidden), device=dev, generator=g).to(torch.bfloat16)
        lg = torch.Generator(device=dev)
        lg.manual_seed(100 + rank)
        logits = torch.randn((tokens, experts), device=dev, generator=lg)

        def local_experts(rows, local_ids):
            order = torch.sort(local_ids, stable=True).indices
            xr, ids = rows[order].contiguous(), local_ids[order].contiguous()
            r = rows.shape[0]
            gg = ops.gather_qmm(xr.reshape(r, 1, hidden), block.gate.weight, block.gate.scales, block.gate.biases, None,
                                ids, True, GROUP, 4, True).reshape(r, inter)
            uu = ops.gather_qmm(xr.reshape(r, 1, hidden), block.up.weight, block.up.scales, block.up.biases, None, ids,
                                True, GROUP, 4, True).reshape(r, inter)
            dd = ops.gather_qmm(ops.swiglu(gg, uu).reshape(r, 1, inter), block.down.weight, block.down.scales,
                                block.down.biases, None, ids, True, GROUP, 4, True).reshape(r, hidden)
            res = torch.empty_like(dd)
            res[order] = dd
            return res

        ep = None
        if world > 1 and os.environ.get("LISA_BENCH_EP", "peer") == "peer":
            ep = parallel.ExpertParallelMoe(block, experts, tokens, hidden)
            closers.append(ep)

        def step():
            if ep is not None:
                ep.forward(x, logits)
            elif world > 1:
                idx, wts = ops.moe_route(logits, top_k)
                parallel.ep_moe_forward(x, idx, wts, experts, local_experts)
            else:
                block.forward(x, logits)

        flops = 2.0 * tokens * top_k * 3 * inter * hidden  # per rank: its own tokens
        # bytes of the distinct experts this rank's tokens touch (packed codes + scales and biases of gate, up, down)
        distinct = int(torch.unique(ops.moe_route(logits, top_k)[0]).numel())
        work_bytes = distinct * 3 * (inter * hidden // 2 + 2 * inter * (hidden // GROUP) * 2)
        name = f"configs[3]: routed experts 128 x top-8, hidden 2048, intermediate 768, 4-bit gs64, {tokens} tokens per rank"
        par = ("single GPU" if world == 1 else
               f"expert-parallel, {(e1 - e0)} experts per rank, dispatch and return by peer stores (library kernels) + peer barriers"
               if ep is not None else f"expert-parallel, {(e1 - e0)} experts per rank, NCCL all-to-all dispatch and combine")
        scaling = "weak"

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    graphed = False
    fused_mode = args.mode == "shard" and world > 1 and os.environ.get("LISA_BENCH_FUSED", "1") != "0"
    # the peer-store expert-parallel block without its host read (small receive capacity) is graph-capturable too
    if args.mode == "moe" and world > 1 and ep is not None and world * tokens * top_k <= ep.DEVICE_COUNT_ROWS:
        fused_mode = os.environ.get("LISA_BENCH_EP_GRAPH", "1") != "0"
    if (world == 1 or fused_mode) and os.environ.get("LISA_BENCH_GRAPH", "1") != "0":
        # no collective library inside the step (one GPU, or the fused GEMV + peer barrier form), so it
        # replays from a CUDA graph like the decode stack (eager launches through the Python mirror are
        # host-bound at small sizes)
        if world > 1:
            dist.barrier()
        eager = step
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                eager()
        torch.cuda.current_stream().wait_stream(side)
        step = graph.replay
        graphed = True
        for _ in range(2):
            step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    e0_, e1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = ops.launch_count()
    e0_.record()
    for _ in range(args.steps):
        step()
    e1_.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches = ops.launch_count() - before
    if graphed:  # replays do not pass through the library's launch counter
        before = ops.launch_count()
        eager()
        torch.cuda.synchronize()
        launches = (ops.launch_count() - before) * args.steps
    ms = e0_.elapsed_time(e1_) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    line = None
    for obj in closers:  # peer buffers are explicit allocations: give them back
        obj.close()
    if rank == 0:
        total_flops = flops * (world if args.mode == "moe" else 1)
        tensor_bound = (args.mode == "moe" and args.tokens > 64) or (args.mode == "shard" and args.m > 8)
        line = {"metric": "qmm bf16 TFLOP/s" if tensor_bound else ("2-bit qmv HBM GB/s" if args.mode == "shard" else "4-bit gather_qmm HBM GB/s"),
                "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": name, "parallelism": par, "graph": graphed}, "gpu_launches": launches,
                "clocks": clocks,
                "device_status": ops.device_status()}
        if tensor_bound:
            line.update(value=total_flops / (ms * 1e-3) / 1e12, unit="TFLOP/s")
        else:
            # whole job: all ranks' weight bytes (moe: the distinct experts of rank 0's tokens, times the ranks)
            line.update(value=work_bytes * (world if args.mode == "moe" else 1) / (ms * 1e-3) / 1e9, unit="GB/s")
    return line


if __name__ == "__main__":
    main()
