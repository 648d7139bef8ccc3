"""ctypes face of the CPU oracle (df_oracle.c) -- TEST INFRASTRUCTURE ONLY.

Imported by the tests, by the smoke check and by the benchmark's CPU-baseline leg; never by
the product package. use_native() switches to the -O3 -march=native build used for timing (it
is built on the machine that runs it)."""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
_LIB = None

from deepforge_b200 import dfgpu  # noqa: E402  (struct layout shared with dfo_tensor)

Tensor = dfgpu.Tensor  # the oracle's dfo_tensor has the same field layout
tensor = dfgpu.tensor


class ConvAttrs(C.Structure):
    _fields_ = [("spatial_rank", C.c_int32), ("reverse_filter", C.c_int32), ("pre_pad", C.c_int64 * 3),
                ("post_pad", C.c_int64 * 3), ("stride", C.c_int64 * 3), ("dilation", C.c_int64 * 3)]


class SdpaParams(C.Structure):
    _fields_ = [("q", Tensor), ("k", Tensor), ("v", Tensor), ("o", Tensor), ("stats", Tensor), ("max", Tensor),
                ("sum_exp", Tensor), ("seq_q", Tensor), ("seq_kv", Tensor), ("page_table_k", Tensor),
                ("page_table_v", Tensor), ("attn_scale", C.c_float), ("padding_mask", C.c_int32),
                ("has_left_bound", C.c_int32), ("has_right_bound", C.c_int32), ("left_bound", C.c_int64),
                ("right_bound", C.c_int64), ("bottom_right", C.c_int32), ("reserved", C.c_int32), ("s_kv", C.c_int64),
                ("bias", Tensor), ("alibi_mask", C.c_int32), ("reserved2", C.c_int32), ("sink", Tensor), ("block_mask", Tensor),
                ("page_offsets_k", Tensor), ("page_offsets_v", Tensor),
                ("dropout_kind", C.c_int32), ("reserved3", C.c_int32), ("dropout_probability", C.c_double),
                ("dropout_mask", Tensor), ("rng_dump", Tensor)]


def _declare(l: C.CDLL) -> C.CDLL:
    l.dfo_decode_e4m3.restype = C.c_float
    l.dfo_decode_e4m3.argtypes = [C.c_uint8]
    l.dfo_decode_e8m0.restype = C.c_float
    l.dfo_decode_e8m0.argtypes = [C.c_uint8]
    l.dfo_encode_e4m3.restype = C.c_uint8
    l.dfo_encode_e4m3.argtypes = [C.c_float]
    l.dfo_encode_e8m0.restype = C.c_uint8
    l.dfo_encode_e8m0.argtypes = [C.c_float]
    l.dfo_decode_e5m2.restype = C.c_float
    l.dfo_decode_e5m2.argtypes = [C.c_uint8]
    l.dfo_encode_e5m2.restype = C.c_uint8
    l.dfo_encode_e5m2.argtypes = [C.c_float]
    l.dfo_block_scale_code.restype = C.c_uint8
    l.dfo_block_scale_code.argtypes = [C.c_float]
    l.dfo_f32_to_bf16.restype = C.c_uint16
    l.dfo_f32_to_bf16.argtypes = [C.c_float]
    l.dfo_f32_to_f16.restype = C.c_uint16
    l.dfo_f32_to_f16.argtypes = [C.c_float]
    l.dfo_f16_to_f32.restype = C.c_float
    l.dfo_f16_to_f32.argtypes = [C.c_uint16]
    l.dfo_f8_128x4_offset.restype = C.c_int64
    l.dfo_f8_128x4_offset.argtypes = [C.c_int64] * 5
    return l


def use_native() -> None:
    """Switch every wrapper in this module to the -O3 -march=native build (compiled on this
    machine by `make native`); used only for timing the CPU baseline."""
    global _LIB
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "-B", "native"], check=True, capture_output=True)
    _LIB = _declare(C.CDLL(str(ROOT / "oracle" / "_build" / "libdf_oracle_native.so")))


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = ROOT / "oracle" / "_build" / "libdf_oracle.so"
        source = ROOT / "oracle" / "df_oracle.c"
        if not path.exists() or path.stat().st_mtime < source.stat().st_mtime:
            subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
        _LIB = _declare(C.CDLL(str(path)))
    return _LIB


def ptr(array: np.ndarray) -> C.c_void_p:
    return C.c_void_p(array.ctypes.data)


def encode_e4m3_many(values: np.ndarray) -> np.ndarray:
    values = np.ascontiguousarray(values, dtype=np.float32)
    out = np.empty(values.size, dtype=np.uint8)
    lib().dfo_encode_e4m3_many(ptr(values), ptr(out), C.c_int64(values.size))
    return out.reshape(values.shape)


def block_scale_code_many(amax: np.ndarray) -> np.ndarray:
    amax = np.ascontiguousarray(amax, dtype=np.float32)
    out = np.empty(amax.size, dtype=np.uint8)
    lib().dfo_block_scale_code_many(ptr(amax), ptr(out), C.c_int64(amax.size))
    return out.reshape(amax.shape)


def block_scale_quantize(xd: Tensor, x: np.ndarray, yd: Tensor, y: np.ndarray, sd: Tensor, scale: np.ndarray,
                         block: int, axis: int) -> None:
    code = lib().dfo_block_scale_quantize(C.byref(xd), ptr(x), C.byref(yd), ptr(y), C.byref(sd), ptr(scale),
                                          C.c_int64(block), C.c_int32(axis))
    assert code == 0, code


def block_scale_dequantize(xd, x, sd, scale, yd, y, blocks) -> None:
    arr = (C.c_int64 * len(blocks))(*blocks)
    code = lib().dfo_block_scale_dequantize(C.byref(xd), ptr(x), C.byref(sd), ptr(scale), C.byref(yd), ptr(y), arr,
                                            C.c_int32(len(blocks)))
    assert code == 0, code


def pointwise(mode, ad, a, bd, b, od, out, lower=0.0, upper=3.4028234663852886e38, slope=0.0, threads: int = 1) -> None:
    count = 1
    for i in range(od.rank):
        count *= int(od.dim[i])
    fn = lib().dfo_pointwise_range
    _run_slabs(lambda lo, hi: fn(C.c_int32(mode), C.byref(ad), ptr(a), C.byref(bd) if bd is not None else None, ptr(b) if b is not None else None,
                                 C.byref(od), ptr(out), C.c_float(lower), C.c_float(upper), C.c_float(slope), C.c_int64(lo), C.c_int64(hi)),
               count, threads if count >= (1 << 16) else 1)


class PointwiseScalars(C.Structure):
    _fields_ = [("relu_lower", C.c_float), ("relu_upper", C.c_float), ("relu_slope", C.c_float), ("elu_alpha", C.c_float),
                ("softplus_beta", C.c_float), ("swish_beta", C.c_float), ("axis", C.c_int32)]


def pointwise_general(mode, ad, a, bd, b, cd, c, od, out, lower=0.0, upper=3.4028234663852886e38, slope=0.0, elu_alpha=1.0,
                      softplus_beta=1.0, swish_beta=1.0, axis=0, threads: int = 1) -> None:
    """Any POINTWISE mode; (cd, c) is IN_2 of BINARY_SELECT, None otherwise."""
    count = 1
    for i in range(od.rank):
        count *= int(od.dim[i])
    scalars = PointwiseScalars(lower, upper, slope, elu_alpha, softplus_beta, swish_beta, axis)
    fn = lib().dfo_pointwise_general_range
    fn.restype = C.c_int

    def slab(lo, hi):
        return fn(C.c_int32(mode), C.byref(ad), ptr(a), C.byref(bd) if bd is not None else None, ptr(b) if b is not None else None,
                  C.byref(cd) if cd is not None else None, ptr(c) if c is not None else None, C.byref(od), ptr(out),
                  C.byref(scalars), C.c_int64(lo), C.c_int64(hi))
    _run_slabs(slab, count, threads if count >= (1 << 16) else 1)


def conv_attrs(pre, post, stride, dilation, reverse=False) -> ConvAttrs:
    a = ConvAttrs()
    a.spatial_rank = len(pre)
    a.reverse_filter = int(reverse)
    for i in range(len(pre)):
        a.pre_pad[i], a.post_pad[i], a.stride[i], a.dilation[i] = pre[i], post[i], stride[i], dilation[i]
    return a


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def _slabs(total: int, threads: int):
    threads = max(1, min(threads, total))
    edges = [total * i // threads for i in range(threads + 1)]
    return [(lo, hi) for lo, hi in zip(edges[:-1], edges[1:]) if hi > lo]


def _run_slabs(call, total: int, threads: int) -> None:
    """call(lo, hi) -> status code, over slabs of [0, total) on `threads` host threads (ctypes drops the GIL)."""
    slabs = _slabs(total, threads)
    if len(slabs) == 1:
        codes = [call(*slabs[0])]
    else:
        with ThreadPoolExecutor(max_workers=len(slabs)) as pool:
            codes = list(pool.map(lambda slab: call(*slab), slabs))
    assert all(code == 0 for code in codes), codes


def conv_generic_flat(xd, x, wd, w, yd, y, attrs) -> None:
    """The literal flat loop over the logical output (any rank, groups, strides, storage types)."""
    code = lib().dfo_conv_generic(C.byref(xd), ptr(x), C.byref(wd), ptr(w), C.byref(yd), ptr(y), C.byref(attrs))
    assert code == 0, code


def conv_generic(xd, x, wd, w, yd, y, attrs, threads: int = 1) -> None:
    """Static-loop-nest form when the tensors allow it (bit-identical to the flat loop, see df_oracle.c), in pixel
    slabs on `threads` host threads; the flat loop otherwise."""
    pixels = int(yd.dim[0] * yd.dim[2] * yd.dim[3]) if yd.rank == 4 else 0
    fn = lib().dfo_conv_generic_nhwc
    probe = fn(C.byref(xd), ptr(x), C.byref(wd), ptr(w), C.byref(yd), ptr(y), C.byref(attrs), C.c_int64(0), C.c_int64(0)) if pixels else 20
    if probe != 0:
        return conv_generic_flat(xd, x, wd, w, yd, y, attrs)
    _run_slabs(lambda lo, hi: fn(C.byref(xd), ptr(x), C.byref(wd), ptr(w), C.byref(yd), ptr(y), C.byref(attrs), C.c_int64(lo), C.c_int64(hi)), pixels, threads)


def conv_mvp(x, w, n, h, wd, c, k, r, s, pads, vector_width=0) -> np.ndarray:
    top, left, bottom, right = pads
    oh, ow = h + top + bottom - r + 1, wd + left + right - s + 1
    y = np.empty((n, oh, ow, k), dtype=np.float32)
    args = [ptr(x), ptr(w), ptr(y)] + [C.c_int64(v) for v in (n, h, wd, c, k, r, s, top, left, bottom, right)]
    if vector_width:
        code = lib().dfo_conv_mvp_vector(*args, C.c_int32(vector_width))
    else:
        code = lib().dfo_conv_mvp_scalar(*args)
    assert code == 0, code
    return y


def matmul(ad, a, bd, b, cd, c, row_begin=0, row_end=-1, threads: int = 1) -> None:
    rows = int(cd.dim[cd.rank - 2])
    row_end = rows if row_end < 0 else min(row_end, rows)
    if row_end <= row_begin:
        return
    _run_slabs(lambda lo, hi: lib().dfo_matmul(C.byref(ad), ptr(a), C.byref(bd), ptr(b), C.byref(cd), ptr(c), C.c_int64(row_begin + lo), C.c_int64(row_begin + hi)),
               row_end - row_begin, threads)


def matmul_fp8(ad, a, bd, b, cd, c, descale_a: float, descale_b: float, scale_c: float) -> float:
    """C in place; returns Amax_C."""
    amax = C.c_float(0.0)
    code = lib().dfo_matmul_fp8(C.byref(ad), ptr(a), C.byref(bd), ptr(b), C.byref(cd), ptr(c), C.c_float(descale_a), C.c_float(descale_b),
                                C.c_float(scale_c), C.byref(amax))
    assert code == 0, code
    return amax.value


def validate_page_prefix(params: SdpaParams, arrays, which: int) -> int:
    """The reference's runtime rule for a compact page table's batch prefix: 0 valid, 17 invalid."""
    arrays = list(arrays) + [None] * (16 - len(arrays))
    pointers = (C.c_void_p * 16)(*[C.c_void_p(a.ctypes.data) if a is not None else C.c_void_p(None) for a in arrays])
    return int(lib().dfo_validate_page_prefix(C.byref(params), pointers, C.c_int(which)))


def bernoulli(seed: int, offset: int, linear: int, keep_probability: float) -> float:
    fn = lib().dfo_bernoulli
    fn.restype = C.c_float
    return float(fn(C.c_int64(seed), C.c_int64(offset), C.c_int64(linear), C.c_double(keep_probability)))


def sdpa_forward(params: SdpaParams, arrays, bh_begin=0, bh_end=1 << 62, q_step=1, threads: int = 1) -> None:
    # the twelfth is the bias, then the sink token, the block mask, the offsets of compact K and V page tables, Dropout_mask, Dropout_scale,
    # Seed, Offset, RNG_DUMP
    assert 11 <= len(arrays) <= 21
    arrays = list(arrays) + [None] * (21 - len(arrays))
    pointers = (C.c_void_p * 21)(*[C.c_void_p(a.ctypes.data) if a is not None else C.c_void_p(None) for a in arrays])
    bh_end = min(bh_end, int(params.q.dim[0] * params.q.dim[1]))
    if bh_end <= bh_begin:
        return
    # (batch, head) pairs write disjoint outputs: slabs of them run side by side
    _run_slabs(lambda lo, hi: lib().dfo_sdpa_forward(C.byref(params), pointers, C.c_int64(bh_begin + lo), C.c_int64(bh_begin + hi), C.c_int64(q_step)),
               bh_end - bh_begin, threads)
