#!/usr/bin/env python
"""Benchmark of the hot path on B200: one "step" = one pass of a configuration's serialized
graph through Executable.execute() on device-resident synthetic inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c1_nchw|c2|c3|c4|c5]
    python bench.py --impl reference ...     # the CPU restatement of the reference, timed

Prints ONE JSON line. `value` is whole-job throughput in the workload's unit with inputs
already in HBM: K CUDA-graph replays of Executable.execute() back to back, rotating over
buffer replicas larger than twice the L2 (cold data every step, no flush kernel in the
timed region), one CUDA-event pair around the K steps, max over ranks; `e2e` is the same
metric with, every step, pinned-host -> device copies of every input and the device ->
host read of every output inside the timed region (upload, kernels and download of
consecutive steps overlap on three streams); `roofline` is measured per kernel with CUDA
events in a separate pass over the same plan; `cpu_baseline` times the CPU oracle (a port
of the reference's algorithm: the reference binary needs LLVM/MLIR 22.1.8, absent here)
on a bounded sample of the same workload, single-threaded like the reference; the
`--impl reference` arm runs one such sample per host thread side by side.

Multi-GPU (torchrun, one rank per GPU): every rank runs the full per-GPU configuration on
its own data (the path has no exchange step), so scaling is "weak"; --gather adds the NCCL
all-gather of the outputs to the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"], "bf16_tflops_sustained": data["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML reads every 2 ms from a
    thread (read-only queries), or nvidia-smi every 100 ms when the NVML binding is missing."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.index = index
        self.samples = []  # (sm_mhz, max_mhz, [4 flags])
        self.process = None
        self.thread = None
        self.running = False
        self.source = None

    def start(self):
        self.running = True
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = self.index
            if visible:
                entries = [e.strip() for e in visible.split(",") if e.strip()]
                if self.index < len(entries) and entries[self.index].isdigit():
                    physical = int(entries[self.index])
            handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            maximum = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            masks = [pynvml.nvmlClocksEventReasonHwSlowdown, pynvml.nvmlClocksEventReasonHwThermalSlowdown,
                     pynvml.nvmlClocksEventReasonSwThermalSlowdown, pynvml.nvmlClocksEventReasonSwPowerCap]

            def poll():
                while self.running:
                    try:
                        mhz = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                        reasons = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                        self.samples.append((int(mhz), int(maximum), [bool(reasons & m) for m in masks]))
                    except Exception:
                        pass
                    time.sleep(0.002)

            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            self.source = "nvml"
            return
        except Exception:
            pass
        try:
            self.process = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                            stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.source = "nvidia-smi"
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6 and parts[0].isdigit():
                self.samples.append((int(parts[0]), int(parts[1]), [p.lower().startswith("active") for p in parts[2:6]]))

    def stop(self) -> dict:
        self.running = False
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        elif self.thread is not None:
            self.thread.join(timeout=1)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(s[0] for s in self.samples)
        reasons = [name for i, name in enumerate(self.NAMES) if any(s[2][i] for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.samples[0][1], "reasons": reasons, "samples": len(sm), "source": self.source}


# ---- CPU baseline: the oracle on the workload, or on a bounded sample of it -------------------------

def cpu_sample(name: str, fraction: float = 1.0, threads: int = 1):
    """Returns (sample description, callable running one pass, units of the metric it covers, whether the sample
    is the whole configuration). The convolutions, the matmul and the SDPA (batch, head) pairs run as slabs on
    `threads` host threads inside the oracle (1 = the reference's own single-threaded execution); `fraction` < 1
    shrinks the sample (fewer images / matrix rows / (batch, head) pairs / sequences)."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import df_oracle_binding as oracle
    import graph_oracle
    from deepforge_b200 import workloads
    oracle.use_native()  # -O3 -march=native build, compiled on this host
    fraction = min(1.0, max(fraction, 1e-4))
    if name in ("c1", "c1_nchw"):
        wl = workloads.BUILDERS[name]()
        x, w = wl.inputs[1](), wl.inputs[2]()
        if name == "c1" and threads == 1:
            run = lambda: oracle.conv_mvp(x, w, 1, 56, 56, 64, 64, 3, 3, (1, 1, 1, 1), vector_width=16)
            return "full workload, the single-node path's 16-lane channel-vector schedule (vf16)", run, wl.flops / 1e12, True
        ins = {1: x, 2: w}
        return "full workload, generic strided path", (lambda: graph_oracle.run(wl.document, ins, threads=threads)), wl.flops / 1e12, True
    if name == "c2":
        images = max(1, int(round(32 * fraction)))
        wl = workloads.c2(n=images)
        ins = {uid: graph_oracle.widen(make(), wl.tensor(uid)["data_type"]) for uid, make in wl.inputs.items()}
        what = "full workload (N = 32)" if images == 32 else f"{images} of the 32 images at full geometry"
        return (f"{what}: all three convolutions and the pointwise nodes, all-FLOAT twin of the DAG, static loop nests",
                (lambda: graph_oracle.run(wl.document, ins, threads=threads)), wl.flops / 1e12, images == 32)
    if name == "c3":
        rows = max(32, int(round(4096 * fraction)) // 32 * 32)
        wl = workloads.c3(m=rows, k=4096, n=rows)
        ins = {uid: graph_oracle.widen(make(), "BFLOAT16") for uid, make in wl.inputs.items()}
        storage = {uid: make() for uid, make in wl.inputs.items()}
        what = "full workload" if rows == 4096 else f"{rows} rows of A x {rows} columns of B over the full K=4096"
        return (f"{what} (quantize, dequantize, matmul)",
                (lambda: graph_oracle.run(wl.document, ins, storage_inputs=storage, threads=threads)), wl.flops / 1e12, rows == 4096)
    if name == "fp8":
        rows = max(32, int(round(4096 * fraction)) // 32 * 32)
        wl = workloads.matmul_fp8(m=rows, k=4096, n=rows)
        ins = {uid: graph_oracle.widen(make(), wl.tensor(uid)["data_type"]) for uid, make in wl.inputs.items()}
        return (f"{rows} rows of A x {rows} columns of B over the full K=4096", (lambda: graph_oracle.run(wl.document, ins)), wl.flops / 1e12, rows == 4096)
    if name == "c4":
        pairs = max(1, int(round(256 * fraction)))
        heads = min(pairs, 32)
        batch = max(1, pairs // 32)
        wl = workloads.c4(b=batch, h=heads, s=2048)
        ins = {uid: graph_oracle.widen(make(), "BFLOAT16") for uid, make in wl.inputs.items()}
        what = "full workload" if batch * heads == 256 else f"{batch * heads} of the 256 (batch, head) pairs, every query row, S=2048"
        return what, (lambda: graph_oracle.run(wl.document, ins, threads=threads)), wl.flops / 1e12, batch * heads == 256
    if name == "c5":
        sequences = max(1, int(round(64 * fraction)))
        wl = workloads.c5(batch=sequences, pages=min(16384, max(256, 256 * sequences)))
        ins = {uid: graph_oracle.widen(make(), wl.tensor(uid)["data_type"]) for uid, make in wl.inputs.items()}
        what = f"{sequences} of the 64 sequences (all 32 query heads, lengths U[512, 8192], a pool of {wl.tensor(2)['dim'][0]} pages)"
        return what, (lambda: graph_oracle.run(wl.document, ins, threads=threads)), wl.bytes / 1e9, False
    raise KeyError(name)


# Fraction of each configuration one single-threaded pass of the oracle covers in roughly 10-30 s on one host core.
CPU_BASELINE_FRACTION = {"c1": 1.0, "c1_nchw": 1.0, "c2": 1.0, "c3": 1.0 / 16, "fp8": 1.0 / 16, "c4": 8.0 / 256, "c5": 4.0 / 64}


def time_cpu(name: str, budget_s: float = 20.0, max_runs: int = 3):
    description, run, units, whole = cpu_sample(name, CPU_BASELINE_FRACTION[name], threads=1)
    run()  # warm caches and page in
    times = []
    start = time.perf_counter()
    while len(times) < max_runs and (not times or time.perf_counter() - start < budget_s):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    best = min(times)
    return description, units / best, best, len(times), whole


def reference_arm(args) -> None:
    """The reference's CPU implementation of the path (its restatement: the binary cannot be built here), on all
    the host cores this process may use: the oracle's loops cut into slabs of output pixels / rows / (batch, head)
    pairs, one slab per thread. The reference itself is single-threaded. A step is one pass over the configuration,
    or over the largest part of it that keeps the whole run within a few minutes (stated in the line)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from deepforge_b200 import workloads
    wl = workloads.BUILDERS[args.workload]()
    try:
        threads = len(os.sched_getaffinity(0))
    except AttributeError:
        threads = os.cpu_count() or 1
    threads = max(1, min(threads, args.ref_threads if args.ref_threads > 0 else threads))
    # size the per-step sample: try a small part, then scale to about 150 s for warm-up + steps
    fraction = min(1.0, CPU_BASELINE_FRACTION[args.workload] * 0.5)
    description, run, units, whole = cpu_sample(args.workload, fraction, threads)
    t0 = time.perf_counter()
    run()
    one = time.perf_counter() - t0
    passes = max(args.warmup, 1) + args.steps
    wanted = min(1.0, fraction * (150.0 / passes) / max(one, 1e-3))
    if args.workload in ("c1", "c1_nchw"):
        wanted = 1.0
    if abs(wanted - fraction) > 1e-9:
        description, run, units, whole = cpu_sample(args.workload, wanted, threads)
    for _ in range(max(args.warmup, 1)):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    elapsed = time.perf_counter() - t0
    value = units * args.steps / elapsed
    line = {
        "impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {**wl.description, "sample_per_step": description, "whole_configuration_per_step": bool(whole)},
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": threads, "kind": "port", "sample": description,
                         "note": "restatement of the reference algorithm as static loop nests (same per-element arithmetic and order), slabs on all host threads; the reference is single-threaded and its binary needs LLVM/MLIR 22.1.8"},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- GPU arm -----------------------------------------------------------------------------------

L2_BYTES = 126 << 20
TIMED_BLOCKS = 32  # the K timed steps are cut into this many event-stamped blocks (median and min are reported beside the total)


def measure_peaks_here(torch, device, seconds: float = 2.0) -> dict:
    """Dense tensor-core peaks of the FP8 and TF32 kinds on this GPU, measured the way the bf16 figure in
    MEASURED_PEAKS.json was (a library GEMM, 8192^3, best of 10 and back to back for `seconds`): the denominators of
    the FP8 / MXFP8 and f32 contraction fractions. Each entry is null when the library refuses the call."""
    n = 8192
    flops = 2.0 * n ** 3
    out = {"how": f"torch._scaled_mm (E4M3 x E4M3 -> bf16, unit scales) and torch.matmul with TF32 allowed, {n}^3, best of 10 (burst) and back to back for {seconds:.0f} s (sustained)"}

    def run(call):
        for _ in range(3):
            call()
        torch.cuda.synchronize(device)
        best = float("inf")
        for _ in range(10):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            call()
            end.record()
            torch.cuda.synchronize(device)
            best = min(best, begin.elapsed_time(end))
        count = max(10, int(seconds * 1e3 / best))
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(count):
            call()
        end.record()
        torch.cuda.synchronize(device)
        return flops / (best * 1e-3) / 1e12, flops * count / (begin.elapsed_time(end) * 1e-3) / 1e12

    try:
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()  # column-major B, as the FP8 GEMM wants it
        one = torch.ones((), device=device, dtype=torch.float32)
        burst, sustained = run(lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
        out["fp8_tflops"], out["fp8_tflops_sustained"] = burst, sustained
        del a, b
    except Exception as error:  # noqa: BLE001
        out["fp8_tflops"] = out["fp8_tflops_sustained"] = None
        out["fp8_error"] = str(error)[:160]
    try:
        previous = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        a = torch.randn(n, n, device=device)
        b = torch.randn(n, n, device=device)
        burst, sustained = run(lambda: torch.matmul(a, b))
        torch.backends.cuda.matmul.allow_tf32 = previous
        out["tf32_tflops"], out["tf32_tflops_sustained"] = burst, sustained
        del a, b
    except Exception as error:  # noqa: BLE001
        out["tf32_tflops"] = out["tf32_tflops_sustained"] = None
        out["tf32_error"] = str(error)[:160]
    torch.cuda.empty_cache()
    return out


def checked_pass(name: str, wl, session) -> dict:
    """One compared run before anything is timed (as the reference's benchmark tool does): the outputs the session
    just produced against the CPU oracle on a bounded sample of the workload, with the parity gates of the tests."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import df_oracle_binding as oracle
    import graph_oracle
    from deepforge_b200 import workloads
    threads = oracle.host_threads()
    bf16_gate = lambda got, ref: bool(np.all(np.abs(got - ref) <= 1e-2 + 2e-2 * np.abs(ref)))
    storage_view = {"BFLOAT16": np.uint16, "HALF": np.float16, "FLOAT": np.float32, "INT32": np.int32}
    raw = {uid: session.raw(uid) for uid in list(wl.inputs)}
    widened = {uid: graph_oracle.widen(raw[uid], wl.tensor(uid)["data_type"]) for uid in raw}
    try:
        if name in ("c1", "c1_nchw"):
            ref = graph_oracle.run(wl.document, widened, threads=threads)[3]
            got = session.output(3)
            ok = float(np.max(np.abs(got - ref))) <= 1e-4 * float(np.max(np.abs(ref)))
            return {"ok": bool(ok), "sample": "every output", "gate": "max|d| <= 1e-4 max|ref|"}
        if name == "c2":
            n, c, h, w = wl.tensor(1)["dim"]
            sub = workloads.c2(n=1, h=h, w=w, c_in=c, c_mid=wl.tensor(2)["dim"][0])
            ins = dict(widened)
            ins[1] = widened[1][: c * h * w]
            ref = graph_oracle.run(sub.document, ins, threads=threads)[7]
            return {"ok": bf16_gate(session.output(7)[: ref.size], ref), "sample": f"every output of the first image ({ref.size} values), all-FLOAT twin of the DAG",
                    "gate": "|d| <= 1e-2 + 2e-2 |ref|"}
        if name == "c3":
            m, k = wl.tensor(1)["dim"]
            n = wl.tensor(2)["dim"][1]
            rows, depth = min(m, 64), min(k, 64)
            a_doc, b_doc = workloads.c3(m=rows, k=k, n=n).document, workloads.c3(m=m, k=depth, n=n).document
            ref_a = graph_oracle.run({**a_doc, "nodes": [a_doc["nodes"][0]]}, {}, storage_inputs={1: raw[1].view(np.uint16)[: rows * k]})
            ref_b = graph_oracle.run({**b_doc, "nodes": [b_doc["nodes"][1]]}, {}, storage_inputs={2: raw[2].view(np.uint16)[: depth * n]})
            aq, sfa, bq, sfb = (session.output(uid) for uid in (3, 4, 5, 6))
            exact = (np.array_equal(aq[: rows * k], ref_a[3]) and np.array_equal(sfa[: rows * k // 32], ref_a[4])
                     and np.array_equal(bq[: depth * n], ref_b[5]) and np.array_equal(sfb[: depth // 32 * n], ref_b[6]))
            # C rows 0..7 from the device's own codes: the oracle's dequantize and f32 matmul
            T, dq = oracle.tensor, oracle.block_scale_dequantize
            from deepforge_b200 import dfgpu
            af, bf, c_ref = np.zeros(8 * k, np.float32), np.zeros(k * n, np.float32), np.zeros(8 * n, np.float32)
            dq(T(dfgpu.E4M3, [8, k]), aq[: 8 * k], T(dfgpu.E8M0, [8, k // 32]), sfa[: 8 * k // 32], T(dfgpu.F32, [8, k]), af, [1, 32])
            dq(T(dfgpu.E4M3, [k, n]), bq, T(dfgpu.E8M0, [k // 32, n]), sfb, T(dfgpu.F32, [k, n]), bf, [32, 1])
            oracle.matmul(T(dfgpu.F32, [8, k]), af, T(dfgpu.F32, [k, n]), bf, T(dfgpu.F32, [8, n]), c_ref, threads=threads)
            close = bf16_gate(session.output(9)[: 8 * n], c_ref)
            return {"ok": bool(exact and close), "sample": f"codes and scales of {rows} rows of A and {depth} K-rows of B bit for bit; 8 rows of C", "gate": "bit-exact; |d| <= 1e-2 + 2e-2 |ref|"}
        if name == "fp8":
            return {"ok": None, "sample": "not sampled here (tests/test_gpu_matmul_fp8.py compares whole matrices)", "gate": None}
        if name == "c4":
            b, h, sq, d = wl.tensor(1)["dim"]
            pair = b * h - 1
            ref = graph_oracle.run(wl.document, widened, sdpa_bh=(pair, pair + 1), sdpa_q_step=8)
            got = session.output(4).reshape(b * h, sq, d)[pair, ::8]
            want = ref[4].reshape(b * h, sq, d)[pair, ::8]
            return {"ok": bf16_gate(got, want), "sample": f"every 8th query row of the last (batch, head) pair ({want.shape[0]} rows)", "gate": "|d| <= 1e-2 + 2e-2 |ref|"}
        if name == "c5":
            batch, hq, _, d = wl.tensor(1)["dim"]
            store = {uid: session.raw(uid).view(np.uint16) for uid in wl.device_inputs}
            for uid, make in wl.inputs.items():
                if uid in (2, 3):
                    store[uid] = raw[uid].view(np.uint16)
                    widened.pop(uid, None)
            ref = graph_oracle.run(wl.document, widened, sdpa_bh=(0, hq), storage_inputs=store)
            got = session.output(4).reshape(batch, hq, d)[0]
            return {"ok": bf16_gate(got, ref[4].reshape(batch, hq, d)[0]), "sample": f"all {hq} heads of the first sequence", "gate": "|d| <= 1e-2 + 2e-2 |ref|"}
    except Exception as error:  # noqa: BLE001 - the benchmark reports a failed check, it does not die of it
        return {"ok": False, "error": str(error)[:200]}
    return {"ok": None, "sample": "none"}


def measure(name: str, steps: int, warmup: int, torch, device, distributed: bool, gather: bool, sampler=None, pin: bool = True,
            sharded: bool = False, check: bool = False, options: int = 0) -> dict:
    """Timed region: `steps` passes back to back on the launching stream, each pass a CUDA-graph replay of
    Executable.execute() on the next of R replicas of all buffers; R is chosen so that the replicas
    together exceed twice the L2, i.e. every pass reads and writes cold data without an explicit flush.
    With `sharded` (torchrun) the rank runs its share of the configuration and, with `gather`, every step ends
    with the NCCL all-gather of each output inside the timed region."""
    from deepforge_b200 import harness, workloads
    rank, world = 0, 1
    if distributed:
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
    wl = workloads.shard(name, rank, world) if sharded else workloads.BUILDERS[name]()
    session = harness.Session(wl, device, pin=pin, options=options)
    checked = None
    if check:
        session.run()
        torch.cuda.synchronize(device)
        checked = checked_pass(name, wl, session)
    footprint = session.footprint_bytes()
    replicas = max(1, min(8, -(-2 * L2_BYTES // max(footprint, 1))))
    if wl.bytes > 2 * L2_BYTES:
        replicas = 1  # one pass already streams more than twice the L2
    session.make_replicas(replicas)
    graphs = session.capture()
    stream = torch.cuda.current_stream(device)
    gathered = None
    gather_bytes = 0
    if gather and distributed:
        # only what the shards split: an output every rank computes in full (the quantized B operand) is not exchanged
        gathered = {uid: torch.empty(world * session.dev[uid].numel(), dtype=torch.uint8, device=device) for uid in wl.outputs if uid in workloads.GATHER_AXIS.get(name, {})}
        gather_bytes = sum(t.numel() for t in gathered.values())

    # The all-gather of step i runs on a side stream while the kernels of step i + 1 run on the launching stream (the
    # steps rotate over the buffer replicas; a replica's outputs are not overwritten before their gather has finished).
    side = torch.cuda.Stream(device) if gathered is not None else None
    computed = [torch.cuda.Event() for _ in range(replicas)]
    gather_done = [torch.cuda.Event() for _ in range(replicas)]
    pending = [False] * replicas

    def step(i):
        r = i % replicas
        if pending[r]:
            stream.wait_event(gather_done[r])
        graphs[r].replay()
        if gathered is not None:
            import torch.distributed as dist
            tensors = session.replica_tensors(r)
            computed[r].record(stream)
            with torch.cuda.stream(side):
                side.wait_event(computed[r])
                for uid in gathered:
                    dist.all_gather_into_tensor(gathered[uid], tensors[uid])
                gather_done[r].record(side)
            pending[r] = True

    def join_gathers():
        """The launching stream waits for every gather in flight (so that an event recorded on it covers them)."""
        for r in range(replicas):
            if pending[r]:
                stream.wait_event(gather_done[r])

    def barrier():
        if distributed:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize(device)

    for i in range(max(warmup, 3)):
        step(i)
    join_gathers()
    if sampler is not None:
        sampler.start()  # before the barrier: what one rank does between the barrier and its first event, the others wait for inside their timed region
    barrier()
    # exactly `steps` steps between the first and the last event; the events in between cut them into blocks
    blocks = max(1, min(TIMED_BLOCKS, steps))
    edges = [steps * j // blocks for j in range(blocks + 1)]
    events = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
    events[0].record(stream)
    for j in range(blocks):
        for i in range(edges[j], edges[j + 1]):
            step(i)
        if j + 1 == blocks:
            join_gathers()  # the timed region ends when the last gather has
        events[j + 1].record(stream)
    barrier()
    device_ms = events[0].elapsed_time(events[-1])
    block_ms = sorted(events[j].elapsed_time(events[j + 1]) / (edges[j + 1] - edges[j]) for j in range(blocks) if edges[j + 1] > edges[j])
    clocks = sampler.stop() if sampler is not None else None

    # the all-gather on its own (same buffers), for the record
    gather_ms = None
    if gathered is not None:
        import torch.distributed as dist
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        begin.record(stream)
        for i in range(20):
            for uid in gathered:
                dist.all_gather_into_tensor(gathered[uid], session.replica_tensors(i % replicas)[uid])
        end.record(stream)
        barrier()
        gather_ms = begin.elapsed_time(end) / 20

    # end to end: pinned host -> device for every input, execute, device -> host for every output, every step;
    # upload, kernels and download of consecutive steps overlap on three streams over the replicas
    if replicas < 3 and footprint < (8 << 30):
        session.make_replicas(3)
        graphs = session.capture()
    pipeline_depth = len(session.replicas)
    host_out = [{uid: torch.empty(session.dev[uid].numel(), dtype=torch.uint8).pin_memory() for uid in wl.outputs} for _ in range(pipeline_depth)]
    h2d = sum(t.numel() for t in session.host.values())
    d2h = sum(t.numel() for t in host_out[0].values())
    session.run_pipelined(max(3, pipeline_depth), graphs, host_out)
    barrier()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record(stream)
    session.run_pipelined(steps, graphs, host_out)
    end.record(stream)
    barrier()
    e2e_ms = begin.elapsed_time(end)

    # per-kernel pass: each launch group of the plan over all replicas in turn as ONE graph (a stream of launches of
    # that kernel, each on buffers the one before did not touch), replayed back to back
    plan = session.exe.steps()
    per_step = []
    count = len(session.replicas)
    repeats = max(3, -(-max(10, min(steps, 50)) // count))
    for index in range(len(plan)):
        round_graph = session.capture_round(index, index + 1)
        for i in range(2):
            round_graph.replay()
        torch.cuda.synchronize(device)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        for i in range(repeats):
            round_graph.replay()
        end.record(stream)
        torch.cuda.synchronize(device)
        per_step.append(begin.elapsed_time(end) / (repeats * count))
    from deepforge_b200 import dfgpu
    status = dfgpu.device_status()
    return {"workload": wl, "session": session, "device_ms": device_ms, "e2e_ms": e2e_ms, "h2d": h2d, "d2h": d2h, "clocks": clocks,
            "plan": plan, "per_step_ms": per_step, "device_status": status, "replicas": replicas, "footprint": footprint,
            "block_ms": block_ms, "gather_ms": gather_ms, "gather_bytes": gather_bytes, "checked": checked}


# dram__bytes_read.sum + dram__bytes_write.sum per launch of each configuration's dominant kernel, from the ncu
# captures summarised under profiles/ (keyed by configuration number and launch label).
NCU_TRAFFIC_BYTES = {
    (1, "conv_fprop"): 1.01e6,         # profiles/umma_conv_f32_kernel_c1_f32_conv.md (the output stays in L2 inside the capture)
    (2, "conv2+bias2+relu2>conv3+residual"): 91.3e6,  # profiles/umma_conv_pair_kernel_c2_bottleneck.md
    (3, "dequantize_b+dequantize_a+matmul"): 35.6e6,  # profiles/umma_mxf8_and_bsq_kernels_c3_quantize_matmul.md
    (4, "sdpa"): 511.2e6,              # profiles/sdpa_umma_pair_kernel_c4_sdpa.md
    (5, "paged_decode"): 1313.1e6,     # profiles/sdpa_decode_umma_kernel_c5_paged_decode.md
}


def roofline_for(result: dict, peaks: dict, here: dict | None = None) -> dict:
    wl, plan, per_step = result["workload"], result["plan"], result["per_step_ms"]
    dominant = int(np.argmax(per_step))
    info = plan[dominant]
    duration_s = per_step[dominant] / 1e3
    # algorithmic bytes of the dominant launch: every tensor bound to it once; the paged decode
    # touches only the valid tokens of the pool, so it uses the workload's figure
    nbytes = wl.bytes if info["op"] == 5 and wl.config == 5 else float(info["bound_bytes"])
    kernels = []
    for p, t in zip(plan, per_step):
        entry = {"label": p["label"], "kernel": p["kernel"], "ms": round(t, 5)}
        if p["op"] in (0, 1, 2) or wl.bound == "hbm":  # bandwidth-bound launches carry their own HBM fraction
            launch_bytes = wl.bytes if p["op"] == 5 and wl.config == 5 else float(p["bound_bytes"])
            entry.update({"algorithmic_bytes": launch_bytes, "gbs": launch_bytes / 1e9 / (t / 1e3), "frac_of_hbm": launch_bytes / 1e9 / (t / 1e3) / peaks["hbm_gbs"]})
        kernels.append(entry)
    # the whole step against the fused roofline: the workload's algorithmic bytes (inputs once, outputs once, virtual
    # intermediates free) or FLOPs over the step time of the timed region
    step_s = result["device_ms"] / 1e3 / max(1, result.get("steps", 1))
    step = {"ms": step_s * 1e3, "algorithmic_bytes": wl.bytes, "gbs": wl.bytes / 1e9 / step_s, "frac_of_hbm": wl.bytes / 1e9 / step_s / peaks["hbm_gbs"]}
    if wl.bound == "tensor" and info["op"] in (4, 5, 6):
        tflops = wl.flops / 1e12 / duration_s
        peak, note = peaks["bf16_tflops"], " (bf16 burst)"
        if (info["op"] == 4 and info["kernel"] == 3) or (info["op"] == 6 and info["kernel"] == 2):
            if here and here.get("fp8_tflops"):
                peak, note = here["fp8_tflops"], " (FP8 dense burst measured in this run, see peaks_measured_here)"
            else:
                peak, note = 2.0 * peak, " (2 x bf16 burst ASSUMED: no FP8 figure could be measured in this run)"
        return {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak, "traffic": NCU_TRAFFIC_BYTES.get((wl.config, info["label"])),
                "kernel": info["label"], "peak_source": peaks["source"] + note, "kernels": kernels, "step": step}
    gbs = nbytes / 1e9 / duration_s
    return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES.get((wl.config, info["label"])),
            "kernel": info["label"], "algorithmic_bytes": nbytes, "peak_source": peaks["source"], "kernels": kernels, "step": step}


def cores_near_gpu(index: int) -> list[int]:
    """Host cores NVML reports as local to GPU `index` of this process (its NUMA node); empty when that cannot be read."""
    try:
        import pynvml
        import torch
        pynvml.nvmlInit()
        uuid = torch.cuda.get_device_properties(index).uuid
        handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        return [64 * w + bit for w, word in enumerate(words) for bit in range(64) if (int(word) >> bit) & 1]
    except Exception:
        return []


def spread_over_cores(local_rank: int, local_world: int) -> str:
    """Gives each rank of a multi-GPU run its own share of the host cores this process may use, taken from the cores
    local to its GPU's NUMA node where NVML tells (the copy threads, pinned buffers and the Python driver of eight
    ranks otherwise crowd onto the same cores, or sit across the socket from their GPU). Returns what was done."""
    try:
        allowed = sorted(os.sched_getaffinity(0))
        if local_world <= 1 or len(allowed) < 2 * local_world:
            return "unchanged"
        near = [sorted(set(cores_near_gpu(r)) & set(allowed)) for r in range(local_world)]
        mine = near[local_rank]
        sharing = [r for r in range(local_world) if near[r] == mine]  # ranks whose GPUs hang off the same node
        if len(mine) >= 2 * len(sharing):
            share = len(mine) // len(sharing)
            position = sharing.index(local_rank)
            chosen = mine[position * share:(position + 1) * share]
            os.sched_setaffinity(0, chosen)
            return f"cores {chosen[0]}-{chosen[-1]}: this GPU's NUMA node ({len(mine)} cores, {len(sharing)} ranks on it)"
        share = len(allowed) // local_world
        chosen = allowed[local_rank * share:(local_rank + 1) * share]
        os.sched_setaffinity(0, chosen)
        return f"cores {chosen[0]}-{chosen[-1]} of {len(allowed)} allowed (GPU locality unknown)"
    except (AttributeError, OSError, ValueError):
        return "unchanged"


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=500)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--workload", default="c2", choices=["c1", "c1_nchw", "c2", "c3", "c4", "c5", "fp8"])
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--replicas", action="store_true", help="multi-GPU: every rank runs the full configuration (weak scaling, no exchange) instead of its shard")
    parser.add_argument("--no-gather", action="store_true", help="multi-GPU, sharded: leave the NCCL all-gather of the outputs out of the timed region")
    parser.add_argument("--bf16-intermediates", action="store_true", help="compile with the lossy bf16 storage of virtual tensors (off by default)")
    parser.add_argument("--no-also", action="store_true", help="skip the short runs of the other configurations")
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    parser.add_argument("--no-peaks", action="store_true", help="skip the FP8 / TF32 peak measurement")
    parser.add_argument("--no-check", action="store_true", help="skip the compared pass before timing")
    parser.add_argument("--no-modes", action="store_true", help="multi-GPU default run: skip the short measurements of the two other modes (shards without the gather, replicas)")
    parser.add_argument("--ref-threads", type=int, default=0, help="host threads of the reference arm (0 = all this process may use)")
    args = parser.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    from deepforge_b200 import build, runtime
    build.build_all()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the kernels")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    cores = spread_over_cores(local_rank, int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))) if distributed else "unchanged"
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    peaks = load_peaks()
    here = None
    if rank == 0 and not args.no_peaks and args.workload in ("c3", "fp8", "c1", "c1_nchw", "c2"):
        here = measure_peaks_here(torch, device)
    if distributed:
        import torch.distributed as dist
        dist.barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    shards = distributed and not args.replicas and args.workload not in ("c1", "c1_nchw", "fp8")
    gather = shards and not args.no_gather
    options = runtime.BF16_INTERMEDIATES if args.bf16_intermediates else 0
    result = measure(args.workload, args.steps, args.warmup, torch, device, distributed, gather, sampler, sharded=shards,
                     check=not args.no_check and rank == 0, options=options)
    result["steps"] = args.steps
    wl = result["workload"]
    device_ms, e2e_ms = result["device_ms"], result["e2e_ms"]
    if distributed:
        import torch.distributed as dist
        times = torch.tensor([device_ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        device_ms, e2e_ms = times.tolist()
    # whole-job units per step: N shards make one full configuration; N replicas are N configurations
    units = wl.units_per_second(1.0)
    if distributed:
        import torch.distributed as dist
        total = torch.tensor([units], device=device, dtype=torch.float64)
        dist.all_reduce(total, op=dist.ReduceOp.SUM)
        units = float(total.item())
    if rank == 0:
        per_step_s = device_ms / args.steps / 1e3
        value = units / per_step_s
        e2e_value = units / (e2e_ms / args.steps / 1e3)
        blocks = result["block_ms"]
        if shards:
            per_gpu = f"rank r of {world} runs its shard (workloads.shard: images / rows of A and C / batch entries / sequences r*1/{world} .. (r+1)*1/{world}); whole-job value = the full configuration over the slowest rank's time"
        elif distributed:
            per_gpu = "every rank runs the full configuration on its own buffers (replicas, no exchange)"
        else:
            per_gpu = "one GPU runs the full configuration"
        plan_kind = "virtual FLOAT tensors between tcgen05 convolutions stored as (hi, lo) bf16 pairs (f32-grade, the default)" if not args.bf16_intermediates else "virtual FLOAT tensors stored as bf16 (lossy option)"
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": device_ms / args.steps, "higher_is_better": True, "scaling": "strong" if shards else "weak", "vs_baseline": None,
            "dtype": "f32" if wl.config == 1 else ("u8+bf16" if wl.config == 3 else "bf16"), "data": "synthetic",
            "config": {**wl.description,
                       "l2": (f"steps rotate over {result['replicas']} replicas of all buffers ({result['replicas'] * result['footprint'] >> 20} MiB in total, L2 is 126 MiB); each step is one CUDA-graph replay of Executable.execute()"
                              if result["replicas"] > 1 else "one step streams more than twice the L2 (126 MiB); each step is one CUDA-graph replay of Executable.execute()"),
                       "per_gpu": per_gpu,
                       "gather_outputs": bool(gather),
                       "plan": plan_kind,
                       "host_cores": cores},
            "timing": {"blocks": len(blocks), "ms_per_step_median": blocks[len(blocks) // 2], "ms_per_step_min": blocks[0], "ms_per_step_max": blocks[-1],
                       "note": "the timed steps, cut into event-stamped blocks on the launching stream; rank 0's blocks"},
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": result["h2d"], "d2h_bytes_per_step": result["d2h"], "ms_per_step": e2e_ms / args.steps,
                    "note": "per rank and step: pinned host -> device of the rank's inputs, execute, device -> pinned host of its outputs (sharded runs deliver the shards to the host; the device-side all-gather is part of `value` only)"},
            "gpu_launches": result["session"].exe.launch_count * args.steps,
            "clocks": result["clocks"],
            "roofline": roofline_for(result, peaks, here),
            "checked_before_timing": result["checked"],
            "device_status": result["device_status"],
            "plan": result["session"].exe.plan_text().strip().split("\n"),
        }
        if gather:
            line["all_gather"] = {"bytes_received_per_rank_and_step": result["gather_bytes"], "ms_alone": result["gather_ms"],
                                  "collective": "ncclAllGather of every output tensor (torch.distributed.all_gather_into_tensor) after the kernels of each step, inside the timed region, on a side stream: the gather of step i overlaps the kernels of step i + 1, and the region ends when the last gather has"}
        if here is not None:
            line["peaks_measured_here"] = here
        del result
        torch.cuda.empty_cache()
        if world == 1 and not args.no_also:
            also = {}
            for other in ("c1", "c2", "c3", "c4", "c5", "fp8"):
                if other == args.workload:
                    continue
                try:
                    r = measure(other, 64, 3, torch, device, False, False, None, pin=False, check=not args.no_check)
                    r["steps"] = 64
                    w = r["workload"]
                    if here is None and other in ("c3", "fp8") and not args.no_peaks:
                        here = measure_peaks_here(torch, device)
                        line["peaks_measured_here"] = here
                    also[other] = {"metric": w.metric, "value": w.units_per_second(r["device_ms"] / 64 / 1e3), "unit": w.unit, "ms_per_step": r["device_ms"] / 64,
                                   "ms_per_step_median": r["block_ms"][len(r["block_ms"]) // 2], "ms_per_step_min": r["block_ms"][0],
                                   "checked_before_timing": r["checked"],
                                   "roofline": {k: v for k, v in roofline_for(r, peaks, here).items() if k != "traffic"}}
                    del r
                    torch.cuda.empty_cache()
                except Exception as error:  # noqa: BLE001 - report, do not hide, a failing side workload
                    also[other] = {"error": str(error)[:200]}
            line["also"] = also
        if world == 1 and not args.no_cpu:
            description, cpu_value, seconds, runs, whole = time_cpu(args.workload)
            line["cpu_baseline"] = {"value": cpu_value, "unit": wl.unit, "cores": 1, "kind": "port", "sample": description,
                                    "seconds_per_sample": seconds, "runs": runs, "whole_configuration": bool(whole),
                                    "note": "CPU restatement of the reference algorithm, single-threaded like the reference; its binary needs LLVM/MLIR 22.1.8 (absent)"}
    # the same configuration in the other two multi-GPU modes, measured briefly by all ranks and carried in the same line:
    # the shards without the exchange, and one full configuration per GPU (weak scaling, no exchange)
    if distributed and shards and gather and not args.no_modes:
        import torch.distributed as dist
        if rank != 0:
            del result
        torch.cuda.empty_cache()
        modes = {}
        for mode, mode_sharded in (("sharded_without_gather", True), ("replicas", False)):
            steps = min(args.steps, 100)
            r = measure(args.workload, steps, args.warmup, torch, device, True, False, None, sharded=mode_sharded, check=False, options=options, pin=False)
            times = torch.tensor([r["device_ms"]], device=device, dtype=torch.float64)
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
            total = torch.tensor([r["workload"].units_per_second(1.0)], device=device, dtype=torch.float64)
            dist.all_reduce(total, op=dist.ReduceOp.SUM)
            ms = float(times.item()) / steps
            modes[mode] = {"value": float(total.item()) / (ms / 1e3), "unit": r["workload"].unit, "ms_per_step": ms, "steps": steps,
                           "scaling": "strong" if mode_sharded else "weak",
                           "per_gpu": "its shard of the full configuration, outputs left where they are" if mode_sharded else "the full configuration (N configurations per step in all)"}
            del r
            torch.cuda.empty_cache()
        if rank == 0:
            line["other_modes"] = modes
    if rank == 0:
        print(json.dumps(line))
    if distributed:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
