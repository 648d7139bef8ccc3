"""Times the POINTWISE kernel per mode on packed tensors and reports the fraction of HBM bandwidth each reaches.

    python -m deepforge_b200.pointwise_bench [--modes ADD,RELU_FWD,...|all] [--dtype bf16|f32|both]
                                             [--elements N] [--steps K] [--warmup W] [--peak-gbs P]

One JSON line: per mode and storage type the CUDA-event time of one launch (mean over K launches that rotate over three
sets of buffers, so that no launch finds its operands in L2) and the algorithmic bytes (every input read once, the
output written once) over that time. The default size is the bottleneck block's output tensor, 32 x 56 x 56 x 256
values. The values go through `dfgpu_pointwise` (include/dfgpu.h), the entry point the Executable calls for a POINTWISE
node that no contraction absorbed (lib/Compiler/FoundationalGraph.cpp:2957-3004 is what it replaces).
"""
import argparse
import json

from . import dfgpu

DEFAULT_MODES = ("ADD", "RELU_FWD", "MUL", "DIV", "TANH_FWD", "SIGMOID_FWD", "SWISH_FWD", "GELU_FWD", "GELU_APPROX_TANH_FWD",
                 "GELU_APPROX_TANH_BWD", "ERF", "EXP", "POW", "CMP_GT", "MAX")


def measure(mode: str, storage: str, elements: int, steps: int, warmup: int, torch) -> dict:
    device = torch.device("cuda", torch.cuda.current_device())
    code, torch_type, width = {"bf16": (dfgpu.BF16, torch.bfloat16, 2), "f32": (dfgpu.F32, torch.float32, 4)}[storage]
    count = dfgpu.pointwise_input_count(mode)
    if count > 2 or mode == "GEN_INDEX":
        raise ValueError(f"{mode} does not run on the packed kernel")
    generator = torch.Generator(device=device).manual_seed(20261125)
    sets = []
    for _ in range(3):
        a = torch.randn(elements, device=device, generator=generator).to(torch_type)
        b = (torch.randn(elements, device=device, generator=generator) + 2.0).to(torch_type)
        sets.append((a, b, torch.empty(elements, device=device, dtype=torch_type)))
    params = dfgpu.PointwiseParams()
    described = dfgpu.tensor(code, [elements // 256, 256])
    params.in0, params.in1, params.out, params.mode = described, described, described, dfgpu.PW_MODES[mode]
    params.relu_upper = 3.4028234663852886e38
    stream = torch.cuda.current_stream().cuda_stream

    def launch(step: int) -> None:
        a, b, out = sets[step % 3]
        dfgpu.pointwise(params, a.data_ptr(), b.data_ptr() if count >= 2 else 0, out.data_ptr(), stream=stream)

    for step in range(warmup):
        launch(step)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for step in range(steps):
        launch(step)
    end.record()
    torch.cuda.synchronize()
    microseconds = begin.elapsed_time(end) / steps * 1e3
    algorithmic = elements * width * (count + 1)
    return {"us": round(microseconds, 2), "algorithmic_bytes": algorithmic, "gbs": round(algorithmic / microseconds / 1e3, 1)}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--modes", default=",".join(DEFAULT_MODES))
    parser.add_argument("--dtype", default="both", choices=["bf16", "f32", "both"])
    parser.add_argument("--elements", type=int, default=32 * 56 * 56 * 256)
    parser.add_argument("--steps", type=int, default=30)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--peak-gbs", type=float, default=None, help="HBM copy bandwidth to report fractions of")
    args = parser.parse_args()
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("pointwise_bench needs a CUDA device")
    if args.elements % 1024:
        raise SystemExit("--elements must be a multiple of 1024")
    names = [name for name in dfgpu.PW_MODE_NAMES if dfgpu.pointwise_input_count(name) <= 2 and name != "GEN_INDEX"] if args.modes == "all" \
        else args.modes.split(",")
    results = {}
    for storage in (("bf16", "f32") if args.dtype == "both" else (args.dtype,)):
        for name in names:
            entry = measure(name, storage, args.elements, args.steps, args.warmup, torch)
            if args.peak_gbs:
                entry["frac_of_hbm"] = round(entry["gbs"] / args.peak_gbs, 3)
            results[f"{name}/{storage}"] = entry
    print(json.dumps({"elements": args.elements, "steps": args.steps, "warmup": args.warmup, "device_status": dfgpu.device_status(),
                      "modes": results}))


if __name__ == "__main__":
    main()
