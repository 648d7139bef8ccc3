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


# ---- CPU baseline: the oracle on a bounded sample of the workload ----------------------------

def cpu_sample(name: str, fraction: float = 1.0):
    """Returns (sample description, callable running one pass, units of the metric it covers). `fraction` < 1
    shrinks the sample (fewer strip rows / matrix rows / query rows / tokens) for runs with many steps."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import df_oracle_binding as oracle
    import graph_oracle
    from deepforge_b200 import workloads
    oracle.use_native()  # -O3 -march=native build, compiled on this host
    fraction = min(1.0, max(fraction, 1e-3))
    if name in ("c1", "c1_nchw"):
        wl = workloads.BUILDERS[name]()
        x, w = wl.inputs[1](), wl.inputs[2]()
        if name == "c1":
            run = lambda: oracle.conv_mvp(x, w, 1, 56, 56, 64, 64, 3, 3, (1, 1, 1, 1), vector_width=16)
            return "full workload, the single-node path's 16-lane channel-vector schedule (vf16)", run, wl.flops / 1e12
        ins = {1: x, 2: w}
        return "full workload, generic strided path", (lambda: graph_oracle.run(wl.document, ins)), wl.flops / 1e12
    if name == "c2":
        rows = max(1, int(round(14 * fraction)))
        wl = workloads.c2(n=1, h=rows, w=56)
        ins = {uid: graph_oracle.widen(make(), wl.tensor(uid)["data_type"]) for uid, make in wl.inputs.items()}
        return (f"a {rows}x56 strip of one image, 1/{32 * 56 // rows} of the batch (all three convolutions and the pointwise nodes), f32 twin of the DAG",
                (lambda: graph_oracle.run(wl.document, ins)), wl.flops / 1e12)
    if name == "c3":
        rows = max(32, int(round(256 * fraction)) // 32 * 32)
        wl = workloads.c3(m=rows, k=4096, n=rows)
        ins = {uid: graph_oracle.widen(make(), "BFLOAT16") for uid, make in wl.inputs.items()}
        storage = {uid: make() for uid, make in wl.inputs.items()}
        return (f"{rows} rows of A x {rows} columns of B over the full K=4096 (quantize, dequantize, matmul)",
                (lambda: graph_oracle.run(wl.document, ins, storage_inputs=storage)), wl.flops / 1e12)
    if name == "fp8":
        rows = max(32, int(round(256 * fraction)) // 32 * 32)
        wl = workloads.matmul_fp8(m=rows, k=4096, n=rows)
        ins = {uid: graph_oracle.widen(make(), wl.tensor(uid)["data_type"]) for uid, make in wl.inputs.items()}
        return (f"{rows} rows of A x {rows} columns of B over the full K=4096", (lambda: graph_oracle.run(wl.document, ins)), wl.flops / 1e12)
    if name == "c4":
        wl = workloads.c4(b=1, h=1, s=2048)
        ins = {uid: graph_oracle.widen(make(), "BFLOAT16") for uid, make in wl.inputs.items()}
        step = min(2048, max(32, int(round(32 / fraction))))
        rows = len(range(0, 2048, step))
        flops = sum(4.0 * 128 * (q + 1) for q in range(0, 2048, step))
        return (f"{rows} query rows (every {step}th) of one (batch, head) pair at S=2048",
                (lambda: graph_oracle.run(wl.document, ins, sdpa_q_step=step)), flops / 1e12)
    if name == "c5":
        longest = max(512, int(round(8192 * fraction)) // 64 * 64)
        wl = workloads.c5(batch=2, hq=4, hkv=1, pages=256, max_len=longest, min_len=max(256, longest // 2))
        ins = {uid: graph_oracle.widen(make(), wl.tensor(uid)["data_type"]) for uid, make in wl.inputs.items()}
        return (f"2 sequences x 1 KV head (4 query heads) with lengths in [{max(256, longest // 2)}, {longest}]",
                (lambda: graph_oracle.run(wl.document, ins)), wl.bytes / 1e9)
    raise KeyError(name)


def time_cpu(name: str, budget_s: float = 12.0, max_runs: int = 5):
    description, run, units = cpu_sample(name)
    run()  # warm caches and page in
    times = []
    start = time.perf_counter()
    while len(times) < max_runs and (not times or time.perf_counter() - start < budget_s):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    best = min(times)
    return description, units / best, best, len(times)


def reference_arm(args) -> None:
    """The reference's CPU implementation of the path (its restatement: the binary cannot be built here), on all
    the host cores this process may use. The reference itself is single-threaded; the sample is one independent
    piece of the workload (an image strip, a block of rows, a few (batch, head) pairs), so T threads run T such
    pieces side by side (the C library is called with the GIL released) and a step is one piece per thread."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from concurrent.futures import ThreadPoolExecutor
    from deepforge_b200 import workloads
    wl = workloads.BUILDERS[args.workload]()
    description, run, units = cpu_sample(args.workload)
    # keep the whole run (warm-up + steps) within about two and a half minutes: shrink the per-step sample when the
    # caller asks for many steps (throughput, the reported value, does not depend on the sample size)
    t0 = time.perf_counter()
    run()
    one = time.perf_counter() - t0
    wanted = 150.0 / (max(args.warmup, 1) + args.steps)
    if one * 1.5 > wanted:
        description, run, units = cpu_sample(args.workload, fraction=wanted / (one * 1.5))
    try:
        threads = len(os.sched_getaffinity(0))
    except AttributeError:
        threads = os.cpu_count() or 1
    threads = max(1, min(threads, args.ref_threads if args.ref_threads > 0 else threads))
    pool = ThreadPoolExecutor(max_workers=threads)

    def step():
        for future in [pool.submit(run) for _ in range(threads)]:
            future.result()

    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    elapsed = time.perf_counter() - t0
    value = units * threads * args.steps / elapsed
    line = {
        "impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {**wl.description, "sample_per_step": f"{threads} x ({description}), one per host thread"},
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": threads, "kind": "port", "sample": f"{threads} x ({description})",
                         "note": "restatement of the reference algorithm; the reference is single-threaded and its binary needs LLVM/MLIR 22.1.8"},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- GPU arm -----------------------------------------------------------------------------------

L2_BYTES = 126 << 20


def measure(name: str, steps: int, warmup: int, torch, device, distributed: bool, gather: bool, sampler=None, pin: bool = True) -> dict:
    """Timed region: `steps` passes back to back on the launching stream, each pass a CUDA-graph replay of
    Executable.execute() on the next of R replicas of all buffers; R is chosen so that the replicas
    together exceed twice the L2, i.e. every pass reads and writes cold data without an explicit flush."""
    from deepforge_b200 import harness, workloads
    wl = workloads.BUILDERS[name]()
    session = harness.Session(wl, device, pin=pin)
    footprint = session.footprint_bytes()
    replicas = max(1, min(8, -(-2 * L2_BYTES // max(footprint, 1))))
    if wl.bytes > 2 * L2_BYTES:
        replicas = 1  # one pass already streams more than twice the L2
    session.make_replicas(replicas)
    graphs = session.capture()
    stream = torch.cuda.current_stream(device)
    gathered = None
    if gather and distributed:
        import torch.distributed as dist
        world = dist.get_world_size()
        gathered = {uid: torch.empty(world * session.dev[uid].numel(), dtype=torch.uint8, device=device) for uid in wl.outputs}

    def step(i):
        graphs[i % replicas].replay()
        if gathered is not None:
            import torch.distributed as dist
            for uid in wl.outputs:
                dist.all_gather_into_tensor(gathered[uid], session.dev[uid])

    def barrier():
        if distributed:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize(device)

    for i in range(max(warmup, 3)):
        step(i)
    barrier()
    if sampler is not None:
        sampler.start()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record(stream)
    for i in range(steps):
        step(i)
    end.record(stream)
    barrier()
    device_ms = begin.elapsed_time(end)
    clocks = sampler.stop() if sampler is not None else None

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

    # per-kernel pass: each launch group of the plan as its own graph, replayed back to back over the replicas
    plan = session.exe.steps()
    per_step = []
    repeats = max(10, min(steps, 50))
    for index in range(len(plan)):
        step_graphs = session.capture(index, index + 1)
        for i in range(3):
            step_graphs[i % replicas].replay()
        torch.cuda.synchronize(device)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        for i in range(repeats):
            step_graphs[i % replicas].replay()
        end.record(stream)
        torch.cuda.synchronize(device)
        per_step.append(begin.elapsed_time(end) / repeats)
    from deepforge_b200 import dfgpu
    status = dfgpu.device_status()
    return {"workload": wl, "session": session, "device_ms": device_ms, "e2e_ms": e2e_ms, "h2d": h2d, "d2h": d2h, "clocks": clocks,
            "plan": plan, "per_step_ms": per_step, "device_status": status, "replicas": replicas, "footprint": footprint}


# dram__bytes_read.sum + dram__bytes_write.sum per launch of each configuration's dominant kernel, from the ncu
# captures summarised under profiles/ (full-size workloads; keyed by configuration number and launch label).
NCU_TRAFFIC_BYTES = {
    (2, "conv3+residual"): 73.0e6,     # profiles/umma_conv_persistent_kernel_c2_bottleneck.md
    (3, "dequantize_b+dequantize_a+matmul"): 34.8e6,  # profiles/umma_mxf8_and_bsq_kernels_c3_quantize_matmul.md
    (4, "sdpa"): 511.2e6,              # profiles/sdpa_umma_pair_kernel_c4_sdpa.md
    (5, "paged_decode"): 1313.1e6,     # profiles/sdpa_decode_umma_kernel_c5_paged_decode.md
}


def roofline_for(result: dict, peaks: dict) -> dict:
    wl, plan, per_step = result["workload"], result["plan"], result["per_step_ms"]
    dominant = int(np.argmax(per_step))
    info = plan[dominant]
    duration_s = per_step[dominant] / 1e3
    # algorithmic bytes of the dominant launch: every tensor bound to it once; the paged decode
    # touches only the valid tokens of the pool, so it uses the workload's figure
    nbytes = wl.bytes if info["op"] == 5 and wl.config == 5 else float(info["bound_bytes"])
    kernels = [{"label": p["label"], "kernel": p["kernel"], "ms": round(t, 5)} for p, t in zip(plan, per_step)]
    if wl.bound == "tensor" and info["op"] in (4, 5, 6):
        tflops = wl.flops / 1e12 / duration_s
        peak, note = peaks["bf16_tflops"], " (bf16 burst)"
        if (info["op"] == 4 and info["kernel"] == 3) or (info["op"] == 6 and info["kernel"] == 2):
            # The block-scaled MXFP8 tensor-core kind issues twice the bf16 rate (dense nominal 4.5 vs 2.25 PFLOP/s);
            # the measured peaks hold no fp8 figure, so the denominator is twice the measured bf16 burst.
            peak, note = 2.0 * peak, " (2 x bf16 burst: MXFP8 kind, no measured fp8 peak)"
        return {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak, "traffic": NCU_TRAFFIC_BYTES.get((wl.config, info["label"])),
                "kernel": info["label"], "peak_source": peaks["source"] + note, "kernels": kernels}
    gbs = nbytes / 1e9 / duration_s
    return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES.get((wl.config, info["label"])),
            "kernel": info["label"], "algorithmic_bytes": nbytes, "peak_source": peaks["source"], "kernels": kernels}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=500)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--workload", default="c2", choices=["c1", "c1_nchw", "c2", "c3", "c4", "c5", "fp8"])
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--gather", action="store_true", help="all-gather the outputs over NCCL inside the timed region")
    parser.add_argument("--no-also", action="store_true", help="skip the short runs of the other configurations")
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    parser.add_argument("--ref-threads", type=int, default=0, help="host threads of the reference arm (0 = all this process may use)")
    args = parser.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    from deepforge_b200 import build
    build.build_all()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the kernels")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    peaks = load_peaks()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    result = measure(args.workload, args.steps, args.warmup, torch, device, distributed, args.gather, sampler)
    wl = result["workload"]
    device_ms, e2e_ms = result["device_ms"], result["e2e_ms"]
    if distributed:
        import torch.distributed as dist
        times = torch.tensor([device_ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        device_ms, e2e_ms = times.tolist()
    if rank == 0:
        per_step_s = device_ms / args.steps / 1e3
        value = world * wl.units_per_second(per_step_s)
        e2e_value = world * wl.units_per_second(e2e_ms / args.steps / 1e3)
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": device_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32" if wl.config == 1 else ("u8+bf16" if wl.config == 3 else "bf16"), "data": "synthetic",
            "config": {**wl.description,
                       "l2": (f"steps rotate over {result['replicas']} replicas of all buffers ({result['replicas'] * result['footprint'] >> 20} MiB in total, L2 is 126 MiB); each step is one CUDA-graph replay of Executable.execute()"
                              if result["replicas"] > 1 else "one step streams more than twice the L2 (126 MiB); each step is one CUDA-graph replay of Executable.execute()"),
                       "per_gpu": "every rank runs the full configuration",
                       "gather_outputs": bool(args.gather and distributed)},
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": result["h2d"], "d2h_bytes_per_step": result["d2h"], "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": result["session"].exe.launch_count * args.steps,
            "clocks": result["clocks"],
            "roofline": roofline_for(result, peaks),
            "device_status": result["device_status"],
            "plan": result["session"].exe.plan_text().strip().split("\n"),
        }
        del result
        torch.cuda.empty_cache()
        if world == 1 and not args.no_also:
            also = {}
            for other in ("c1", "c2", "c3", "c4", "c5", "fp8"):
                if other == args.workload:
                    continue
                try:
                    r = measure(other, 10, 3, torch, device, False, False, None, pin=False)
                    w = r["workload"]
                    also[other] = {"metric": w.metric, "value": w.units_per_second(r["device_ms"] / 10 / 1e3), "unit": w.unit, "ms_per_step": r["device_ms"] / 10,
                                   "roofline": {k: v for k, v in roofline_for(r, peaks).items() if k != "traffic"}}
                    del r
                    torch.cuda.empty_cache()
                except Exception as error:  # noqa: BLE001 - report, do not hide, a failing side workload
                    also[other] = {"error": str(error)[:200]}
            line["also"] = also
        if world == 1 and not args.no_cpu:
            description, cpu_value, seconds, runs = time_cpu(args.workload)
            line["cpu_baseline"] = {"value": cpu_value, "unit": wl.unit, "cores": 1, "kind": "port", "sample": description,
                                    "seconds_per_sample": seconds, "runs": runs,
                                    "note": "CPU restatement of the reference algorithm, single-threaded like the reference; its binary needs LLVM/MLIR 22.1.8 (absent)"}
        print(json.dumps(line))
    if distributed:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
