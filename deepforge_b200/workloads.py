"""The five benchmark configurations as runnable workloads: graph document, seeded
synthetic inputs with the shapes and value distributions the configuration names, and
the algorithmic FLOPs / bytes the roofline is computed from.

Inputs are synthetic stand-ins (there is no dataset in this benchmark): element i of the
tensor with UID u in configuration c is a pure function of (20261125 + c, u, i), see
synthetic.py. Tensors above 2^27 elements (the paged KV pool) are the same streams evaluated
on the device (synthetic.normal_on_device), because the host generator would take minutes.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Callable, Dict, List, Optional

import numpy as np

from . import graphs, synthetic

BASE_SEED = 20261125
NP_DTYPE = {"FLOAT": np.float32, "BFLOAT16": np.uint16, "HALF": np.float16, "FP8_E4M3": np.uint8, "FP8_E5M2": np.uint8, "FP8_E8M0": np.uint8, "INT32": np.int32, "UINT8": np.uint8}
DTYPE_BYTES = {"FLOAT": 4, "BFLOAT16": 2, "HALF": 2, "FP8_E4M3": 1, "FP8_E5M2": 1, "FP8_E8M0": 1, "INT32": 4, "UINT8": 1}


@dataclasses.dataclass
class Workload:
    name: str
    config: int
    document: dict
    description: Dict[str, object]
    metric: str
    unit: str               # "TFLOP/s" or "GB/s"
    flops: float            # algorithmic FLOPs of one pass
    bytes: float            # algorithmic bytes of one pass (inputs read once, outputs written once)
    bound: str              # "hbm" or "tensor"
    inputs: Dict[int, Callable[[], np.ndarray]]   # uid -> generator of the host array (storage dtype)
    device_inputs: Dict[int, Callable[[object], object]] = dataclasses.field(default_factory=dict)  # uid -> torch generator fn(device)
    outputs: List[int] = dataclasses.field(default_factory=list)
    notes: str = ""

    def tensor(self, uid: int) -> dict:
        return self.document["tensors"][str(uid)]

    def nbytes(self, uid: int) -> int:
        t = self.tensor(uid)
        span = sum((d - 1) * s for d, s in zip(t["dim"], t["stride"])) + 1
        if t["reordering_type"] != "NONE":
            span = int(np.prod(t["dim"]))
        return span * DTYPE_BYTES[t["data_type"]]

    def units_per_second(self, seconds: float) -> float:
        amount = self.flops / 1e12 if self.unit == "TFLOP/s" else self.bytes / 1e9
        return amount / seconds


def _store(values: np.ndarray, data_type: str) -> np.ndarray:
    if data_type == "BFLOAT16":
        return synthetic.to_bf16_bits(values)
    if data_type == "HALF":
        return values.astype(np.float16)
    return np.ascontiguousarray(values, dtype=np.float32)


def _normal(seed: int, uid: int, count: int, data_type: str, std: float = 1.0, first: int = 0) -> Callable[[], np.ndarray]:
    """Elements [first, first + count) of the tensor's N(0, std) stream (first must be even)."""
    def make():
        out = np.empty(count, dtype=NP_DTYPE[data_type])
        chunk = 1 << 23
        for start in range(0, count, chunk):
            n = min(chunk, count - start)
            # Box-Muller pairs are indexed from the chunk start (chunks are even-sized)
            u = synthetic.unit(seed, uid, n + (n & 1), first + start)
            u1 = np.maximum(u[0::2], 2.0 ** -53)
            radius = np.sqrt(-2.0 * np.log(u1))
            values = np.empty(n + (n & 1), dtype=np.float64)
            values[0::2] = radius * np.cos(2.0 * np.pi * u[1::2])
            values[1::2] = radius * np.sin(2.0 * np.pi * u[1::2])
            out[start:start + n] = _store((std * values[:n]).astype(np.float32), data_type)
        return out
    return make


def _uniform(seed: int, uid: int, count: int, data_type: str, low: float, high: float) -> Callable[[], np.ndarray]:
    return lambda: _store(synthetic.uniform(seed, uid, count, low, high), data_type)


def c1(layout: str = "nhwc", **shape) -> Workload:
    doc = graphs.c1_conv(layout, **shape)
    seed = BASE_SEED + 1
    x, w, y = (doc["tensors"][k] for k in ("1", "2", "3"))
    n, c, h, wd = x["dim"]
    k, _, r, s = w["dim"]
    p, q = y["dim"][2], y["dim"][3]
    flops = 2.0 * n * p * q * k * r * s * c
    nbytes = 4.0 * (np.prod(x["dim"]) + np.prod(w["dim"]) + np.prod(y["dim"]))
    return Workload(
        name=f"c1_conv_f32_{layout}", config=1, document=doc,
        description={"workload": f"CONV_FPROP f32 X[{n},{c},{h},{wd}] W[{k},{c},{r},{s}] pad {(r - 1) // 2} {layout}"},
        metric="conv_fprop_throughput", unit="TFLOP/s", flops=flops, bytes=nbytes, bound="hbm",
        inputs={1: _uniform(seed, 1, int(np.prod(x["dim"])), "FLOAT", -1.0, 1.0), 2: _uniform(seed, 2, int(np.prod(w["dim"])), "FLOAT", -1.0, 1.0)},
        outputs=[3], notes="231 MFLOP over 1.75 MB: latency-bound, neither roof binds")


def c2(n=32, h=56, w=56, c_in=256, c_mid=64, io="BFLOAT16", first_image=0) -> Workload:
    """first_image: index of this shard's first image inside the full batch (its X slice of the stream)."""
    doc = graphs.c2_bottleneck(n, h, w, c_in, c_mid, io)
    seed = BASE_SEED + 2
    pixels = n * h * w
    flops = 2.0 * pixels * (c_in * c_mid + 9 * c_mid * c_mid + c_mid * c_in)
    width = DTYPE_BYTES[io]
    nbytes = width * (2.0 * pixels * c_in + c_in * c_mid * 2 + 9 * c_mid * c_mid + 2 * c_mid)
    inputs = {
        1: _normal(seed, 1, pixels * c_in, io, first=first_image * h * w * c_in),
        2: _normal(seed, 2, c_mid * c_in, io, math.sqrt(2.0 / c_in)),
        3: _uniform(seed, 3, c_mid, io, -0.1, 0.1),
        4: _normal(seed, 4, c_mid * c_mid * 9, io, math.sqrt(2.0 / (9 * c_mid))),
        5: _uniform(seed, 5, c_mid, io, -0.1, 0.1),
        6: _normal(seed, 6, c_in * c_mid, io, math.sqrt(2.0 / c_mid)),
    }
    return Workload(
        name="c2_resnet50_bottleneck", config=2, document=doc,
        description={"workload": f"ResNet-50 bottleneck DAG {io} NHWC X[{n},{h},{w},{c_in}] 1x1({c_in}->{c_mid})+bias+ReLU, 3x3({c_mid}->{c_mid})+bias+ReLU, 1x1({c_mid}->{c_in})+X"},
        metric="conv_bottleneck_throughput", unit="TFLOP/s", flops=flops, bytes=nbytes, bound="hbm", inputs=inputs, outputs=[7],
        notes="fused end to end the DAG is HBM-bound (arithmetic intensity 136 < ridge ~212)")


def c3(m=4096, k=4096, n=4096, io="BFLOAT16", c_type="BFLOAT16", first_row=0) -> Workload:
    """first_row: index of this shard's first row of A (and of C) inside the full matrix."""
    doc = graphs.c3_quantize_matmul(m, k, n, io, c_type)
    seed = BASE_SEED + 3

    def operand(uid: int, count: int, first: int = 0):
        def make():
            values = _normal(seed, uid, count, "FLOAT", first=first)()
            mask = synthetic.raw_u64(seed, uid + 0x5151, count, first) % np.uint64(100) == 0
            values[mask] *= np.float32(64.0)
            return _store(values, io)
        return make

    width = DTYPE_BYTES[io]
    quant_bytes = (m * k + k * n) * (width + 1.0) + (m * k + k * n) / 32.0
    matmul_bytes = (m * k + k * n) * (1.0 + 1.0 / 32.0) + m * n * DTYPE_BYTES[c_type]
    return Workload(
        name="c3_mxfp8_quantize_matmul", config=3, document=doc,
        description={"workload": f"block-scale quantize (MXFP8 E4M3, 32-element blocks, E8M0 scales) -> MATMUL M={m} K={k} N={n} {io}"},
        metric="quantize_matmul_throughput", unit="TFLOP/s", flops=2.0 * m * n * k, bytes=quant_bytes + matmul_bytes, bound="tensor",
        inputs={1: operand(1, m * k, first_row * k), 2: operand(2, k * n)}, outputs=[3, 4, 5, 6, 9])


def matmul_fp8(m=4096, k=4096, n=4096, c_type="BFLOAT16", batch=(1,), b_k_major=False, a_batch=None, b_batch=None,
               scalars=(0.5, 0.25, 0.125), exact=True, a_type="FP8_E4M3", b_type="FP8_E4M3") -> Workload:
    """One MATMUL_FP8 node (the first row of the "next" list after the five configurations). Operands are E4M3 codes
    with exponent fields 6..8 (|value| in [0.5, 3.75], one in sixteen a zero): with `exact` every partial sum of up to
    2^10 products is exactly representable in f32, so the result does not depend on the order of the additions and
    the tensor-core kernel can be compared bit for bit; without it the exponent fields span 1..9."""
    doc = graphs.matmul_fp8(m, k, n, c_type, batch, b_k_major, a_batch, b_batch, a_type, b_type)
    seed = BASE_SEED + 8

    def codes(uid: int, count: int, data_type: str):
        def make():
            r = synthetic.raw_u64(seed, uid, count, 0)
            sign = ((r >> np.uint64(16)) & np.uint64(1)).astype(np.uint8)
            if data_type == "FP8_E5M2":  # two mantissa bits, bias 15: the same [0.5, 3.5] (or wider) value range
                mantissa = (r & np.uint64(3)).astype(np.uint8)
                span = 3 if exact else 9
                exponent = ((r >> np.uint64(3)) % np.uint64(span)).astype(np.uint8) + np.uint8(14 if exact else 9)
                out = (sign << 7) | (exponent << 2) | mantissa
            else:
                mantissa = (r & np.uint64(7)).astype(np.uint8)
                span = 3 if exact else 9
                exponent = ((r >> np.uint64(3)) % np.uint64(span)).astype(np.uint8) + np.uint8(6 if exact else 1)
                out = (sign << 7) | (exponent << 3) | mantissa
            out[((r >> np.uint64(20)) & np.uint64(15)) == 0] = 0
            return out.astype(np.uint8)
        return make

    def scalar(value: float):
        return lambda: np.array([value], dtype=np.float32)

    def count(uid: int) -> int:
        return int(np.prod(doc["tensors"][str(uid)]["dim"]))

    batches = int(np.prod(batch))
    return Workload(
        name="matmul_fp8", config=8, document=doc,
        description={"workload": f"MATMUL_FP8 {a_type[4:]} x {b_type[4:]} -> {c_type}, M={m} K={k} N={n} batch={list(batch)}, scalar descales, Amax_C"},
        metric="matmul_fp8_throughput", unit="TFLOP/s", flops=2.0 * batches * m * n * k,
        bytes=float(count(21) + count(22) + batches * m * n * DTYPE_BYTES[c_type]), bound="tensor",
        inputs={21: codes(21, count(21), a_type), 22: codes(22, count(22), b_type), 23: scalar(scalars[0]), 24: scalar(scalars[1]), 25: scalar(scalars[2])},
        outputs=[26, 27])


def c4(b=8, h=32, s=2048, d=128, io="BFLOAT16", causal=True, first_batch=0) -> Workload:
    doc = graphs.c4_sdpa(b, h, s, d, io, causal)
    seed = BASE_SEED + 4
    pairs = s * (s + 1) / 2 if causal else s * s
    count = b * h * s * d
    first = first_batch * h * s * d
    return Workload(
        name="c4_sdpa_forward", config=4, document=doc,
        description={"workload": f"SDPA forward {io} BHSD [{b},{h},{s},{d}] causal={causal} scale=1/sqrt({d}) with f32 Stats"},
        metric="sdpa_forward_throughput", unit="TFLOP/s", flops=4.0 * b * h * d * pairs, bytes=4.0 * count * DTYPE_BYTES[io] + 4.0 * b * h * s,
        bound="tensor", inputs={1: _normal(seed, 1, count, io, first=first), 2: _normal(seed, 2, count, io, first=first), 3: _normal(seed, 3, count, io, first=first)},
        outputs=[4, 5])


def c5(batch=64, hq=32, hkv=8, d=128, pages=16384, block=64, max_len=8192, min_len=512, io="BFLOAT16", first_sequence=0, compact=False) -> Workload:
    """first_sequence: index of this shard's first sequence inside the full batch (the KV pool is replicated).
    compact: page tables stored back to back with exactly the slots each sequence needs, plus their offsets."""
    doc = graphs.c5_paged_decode(batch, hq, hkv, d, pages, block, max_len, io, compact=compact)
    seed = BASE_SEED + 5
    table = max_len // block
    lengths = synthetic.integers(seed, 6, first_sequence + batch, min_len, max_len).astype(np.int32)[first_sequence:]
    total = int(lengths.sum())
    pool = pages * hkv * block * d

    def tables(stream: int):
        return lambda: np.stack([synthetic.permutation_prefix(seed, stream * 1000 + first_sequence + i, pages, table) for i in range(batch)]).astype(np.int32).reshape(-1)

    inputs = {1: _normal(seed, 1, batch * hq * d, io, first=first_sequence * hq * d), 5: lambda: np.ones(batch, dtype=np.int32), 6: lambda: lengths.copy(), 7: tables(7), 8: tables(8)}
    if compact:
        slots = (lengths.astype(np.int64) + block - 1) // block
        offsets = np.concatenate([[0], np.cumsum(slots)])

        def packed(stream: int):
            full = tables(stream)
            return lambda: np.concatenate([full().reshape(batch, table)[i, :slots[i]] for i in range(batch)]).astype(np.int32)

        inputs[7], inputs[8] = packed(7), packed(8)
        inputs[9] = lambda: offsets.astype(np.int64)
        inputs[10] = lambda: offsets.astype(np.int32)
    device_inputs = {}
    if pool <= (1 << 27):
        inputs[2] = _normal(seed, 2, pool, io)
        inputs[3] = _normal(seed, 3, pool, io)
    else:
        def device_pool(uid: int):
            # the tensor's documented stream (synthetic.py), evaluated on the device
            return lambda device: synthetic.normal_on_device(device, seed, uid, pool, bf16=io != "FLOAT")
        device_inputs = {2: device_pool(2), 3: device_pool(3)}
    width = DTYPE_BYTES[io]
    nbytes = total * hkv * d * width * 2.0 + 2.0 * batch * hq * d * width + 2.0 * batch * table * 4
    workload = Workload(
        name="c5_paged_decode", config=5, document=doc,
        description={"workload": f"paged-KV SDPA decode {io} batch {batch}, Hq {hq}/Hkv {hkv}, D {d}, {pages} pages x {block} tokens, lengths U[{min_len},{max_len}] (sum {total})"},
        metric="paged_decode_bandwidth", unit="GB/s", flops=4.0 * total * hq * d, bytes=nbytes, bound="hbm", inputs=inputs,
        device_inputs=device_inputs, outputs=[4])
    return workload


BUILDERS = {"c1": c1, "c1_nchw": lambda **kw: c1("nchw", **kw), "c2": c2, "c3": c3, "c4": c4, "c5": c5, "fp8": matmul_fp8}


# which axis of which output tensor the shards concatenate along when gathered
GATHER_AXIS = {"c2": {7: 0}, "c3": {3: 0, 4: 0, 9: 0}, "c4": {4: 0, 5: 0}, "c5": {4: 0}}


def shard(name: str, rank: int, world: int, **size) -> Workload:
    """The rank's share of a configuration that splits naturally: images for the bottleneck, rows of A
    and C for the quantize->matmul (B is quantized on every rank), batch entries for SDPA, sequences
    for paged decode (the KV pool is replicated). Each shard draws exactly its slice of the full
    problem's input streams, so gathering the shards' outputs along GATHER_AXIS reproduces the
    unsharded result. C1 has N = 1 and does not shard: every rank runs a replica."""
    if world == 1 or name in ("c1", "c1_nchw"):
        return BUILDERS[name](**size)
    if name == "c2":
        n = size.pop("n", 32)
        assert n % world == 0
        return c2(n=n // world, first_image=rank * (n // world), **size)
    if name == "c3":
        m = size.pop("m", 4096)
        assert m % world == 0
        return c3(m=m // world, first_row=rank * (m // world), **size)
    if name == "c4":
        b = size.pop("b", 8)
        assert b % world == 0
        return c4(b=b // world, first_batch=rank * (b // world), **size)
    if name == "c5":
        batch = size.pop("batch", 64)
        assert batch % world == 0
        return c5(batch=batch // world, first_sequence=rank * (batch // world), **size)
    if name == "fp8":  # every rank runs the full matrix product on its own stream of codes (Amax_C is a whole-matrix result)
        return matmul_fp8(**size)
    raise KeyError(name)
