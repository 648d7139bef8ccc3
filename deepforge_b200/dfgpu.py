"""ctypes view of the kernel library's C ABI (include/dfgpu.h).

Thin by design: structs mirror the header field for field, wrappers only turn a
non-zero return code into an exception carrying dfgpu_last_error(). Pointers are
raw device addresses (e.g. torch.Tensor.data_ptr()).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Iterable, Optional, Sequence

MAX_RANK = 8
MAX_EPILOGUE = 4

F32, F16, BF16, E4M3, E8M0, I32, E5M2, U8, BF16X2, I64, FP4, I4 = range(12)
REORDER_NONE, REORDER_F8_128x4 = 0, 1
DTYPE_BYTES = {F32: 4, F16: 2, BF16: 2, E4M3: 1, E8M0: 1, I32: 4, E5M2: 1, U8: 1, BF16X2: 4, I64: 8}  # (FP4 and I4: two elements per byte)

EPI_ADD, EPI_RELU = 1, 2
PW_ADD, PW_RELU_FWD, PW_IDENTITY, PW_MUL, PW_SUB = range(5)
# Every POINTWISE mode by the reference's name (lib/Import/Schema.cpp:301-316), numbered as DFGPU_PW_* in dfgpu.h.
PW_MODE_NAMES = (
    "ADD", "RELU_FWD", "IDENTITY", "MUL", "SUB", "DIV", "ADD_SQUARE", "MIN", "MAX", "MOD", "POW", "SQRT", "RSQRT", "EXP",
    "LOG", "NEG", "ABS", "CEIL", "FLOOR", "COS", "SIN", "TAN", "ERF", "RECIPROCAL", "GEN_INDEX", "LOGICAL_NOT",
    "LOGICAL_AND", "LOGICAL_OR", "BINARY_SELECT", "CMP_EQ", "CMP_NEQ", "CMP_GT", "CMP_GE", "CMP_LT", "CMP_LE", "RELU_BWD",
    "TANH_FWD", "TANH_BWD", "SIGMOID_FWD", "SIGMOID_BWD", "ELU_FWD", "ELU_BWD", "SOFTPLUS_FWD", "SOFTPLUS_BWD",
    "SWISH_FWD", "SWISH_BWD", "GELU_FWD", "GELU_BWD", "GELU_APPROX_TANH_FWD", "GELU_APPROX_TANH_BWD")
PW_MODES = {name: code for code, name in enumerate(PW_MODE_NAMES)}
_PW_BINARY = {"ADD", "MUL", "SUB", "DIV", "ADD_SQUARE", "MIN", "MAX", "MOD", "POW", "LOGICAL_AND", "LOGICAL_OR", "CMP_EQ",
              "CMP_NEQ", "CMP_GT", "CMP_GE", "CMP_LT", "CMP_LE"}


def pointwise_input_count(name: str) -> int:
    """Inputs the mode reads (lib/Import/Schema.cpp:353-377)."""
    if name == "BINARY_SELECT":
        return 3
    return 2 if name in _PW_BINARY or name.endswith("_BWD") else 1
BSQ_AUTO, BSQ_GENERIC, BSQ_ROW32, BSQ_COL32 = range(4)
BSD_AUTO, BSD_GENERIC, BSD_PACKED = range(3)
CONV_AUTO, CONV_DIRECT, CONV_IGEMM_FFMA, CONV_UMMA_BF16, CONV_UMMA_F32X3, CONV_UMMA_F32X3_CLUSTER = range(6)
MATMUL_AUTO, MATMUL_FFMA, MATMUL_UMMA_BF16, MATMUL_UMMA_MXF8, MATMUL_UMMA_F32X3, MATMUL_UMMA_F32X3_CLUSTER = range(6)
MATMUL_FP8_AUTO, MATMUL_FP8_SCALAR, MATMUL_FP8_UMMA = range(3)
SDPA_AUTO, SDPA_ROWWISE, SDPA_PAGED_DECODE, SDPA_UMMA, SDPA_PAGED_DECODE_UMMA = range(5)


class Tensor(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("rank", C.c_int32), ("reorder", C.c_int32), ("reserved", C.c_int32),
                ("dim", C.c_int64 * MAX_RANK), ("stride", C.c_int64 * MAX_RANK)]


def contiguous_strides(dims: Sequence[int]) -> list[int]:
    strides = [1] * len(dims)
    for i in range(len(dims) - 2, -1, -1):
        strides[i] = strides[i + 1] * dims[i + 1]
    return strides


def tensor(dtype: int, dims: Sequence[int], strides: Optional[Sequence[int]] = None, reorder: int = REORDER_NONE) -> Tensor:
    t = Tensor()
    t.dtype, t.rank, t.reorder = dtype, len(dims), reorder
    strides = list(strides) if strides is not None else contiguous_strides(dims)
    for i, (d, s) in enumerate(zip(dims, strides)):
        t.dim[i], t.stride[i] = d, s
    return t


ABSENT = Tensor()


class PlanInfo(C.Structure):
    _fields_ = [("kernel", C.c_int32), ("launches", C.c_int32), ("scratch_bytes", C.c_int64)]


class EpilogueStep(C.Structure):
    _fields_ = [("op", C.c_int32), ("operand", C.c_int32), ("relu_lower", C.c_float), ("relu_upper", C.c_float),
                ("relu_slope", C.c_float), ("reserved", C.c_int32)]


class BsqParams(C.Structure):
    _fields_ = [("x", Tensor), ("y", Tensor), ("scale", Tensor), ("block_size", C.c_int64), ("axis", C.c_int32),
                ("kernel", C.c_int32)]


class BsqPairParams(C.Structure):
    _fields_ = [("first", BsqParams), ("second", BsqParams)]


class BsdParams(C.Structure):
    _fields_ = [("x", Tensor), ("scale", Tensor), ("y", Tensor), ("block", C.c_int64 * MAX_RANK),
                ("block_count", C.c_int32), ("kernel", C.c_int32)]


class PointwiseParams(C.Structure):
    _fields_ = [("in0", Tensor), ("in1", Tensor), ("out", Tensor), ("mode", C.c_int32), ("relu_lower", C.c_float),
                ("relu_upper", C.c_float), ("relu_slope", C.c_float), ("in2", Tensor), ("elu_alpha", C.c_float),
                ("softplus_beta", C.c_float), ("swish_beta", C.c_float), ("axis", C.c_int32)]

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        for name in ("elu_alpha", "softplus_beta", "swish_beta"):
            if name not in kwargs:
                setattr(self, name, 1.0)


MAX_CONSTANTS = 16


class ConstantsParams(C.Structure):
    _fields_ = [("count", C.c_int32), ("reserved", C.c_int32), ("bits", C.c_uint64 * MAX_CONSTANTS), ("bytes", C.c_int32 * MAX_CONSTANTS)]


class ConvParams(C.Structure):
    _fields_ = [("x", Tensor), ("w", Tensor), ("y", Tensor), ("extra", Tensor * 2),
                ("pre_pad", C.c_int64 * 2), ("post_pad", C.c_int64 * 2), ("stride", C.c_int64 * 2),
                ("dilation", C.c_int64 * 2), ("reverse_filter", C.c_int32), ("epilogue_count", C.c_int32),
                ("epilogue", EpilogueStep * MAX_EPILOGUE), ("kernel", C.c_int32), ("reserved", C.c_int32),
                ("depth_pre_pad", C.c_int64), ("depth_post_pad", C.c_int64), ("depth_stride", C.c_int64), ("depth_dilation", C.c_int64)]


class ConvPairParams(C.Structure):
    _fields_ = [("first", ConvParams), ("second", ConvParams)]


class MatmulParams(C.Structure):
    _fields_ = [("a", Tensor), ("b", Tensor), ("c", Tensor), ("a_scale", Tensor), ("b_scale", Tensor),
                ("a_block", C.c_int64 * 2), ("b_block", C.c_int64 * 2), ("extra", Tensor * 2),
                ("epilogue_count", C.c_int32), ("kernel", C.c_int32), ("epilogue", EpilogueStep * MAX_EPILOGUE)]


class MatmulFp8Params(C.Structure):
    _fields_ = [("a", Tensor), ("b", Tensor), ("c", Tensor), ("kernel", C.c_int32), ("reserved", C.c_int32)]


class SdpaParams(C.Structure):
    _fields_ = [("q", Tensor), ("k", Tensor), ("v", Tensor), ("o", Tensor), ("stats", Tensor), ("max", Tensor),
                ("sum_exp", Tensor), ("seq_q", Tensor), ("seq_kv", Tensor), ("page_table_k", Tensor),
                ("page_table_v", Tensor), ("attn_scale", C.c_float), ("padding_mask", C.c_int32),
                ("has_left_bound", C.c_int32), ("has_right_bound", C.c_int32), ("left_bound", C.c_int64),
                ("right_bound", C.c_int64), ("bottom_right", C.c_int32), ("kernel", C.c_int32), ("s_kv", C.c_int64),
                ("bias", Tensor), ("alibi_mask", C.c_int32), ("reserved", C.c_int32), ("sink", Tensor), ("block_mask", Tensor),
                ("page_offsets_k", Tensor), ("page_offsets_v", Tensor),
                ("dropout_kind", C.c_int32), ("reserved2", C.c_int32), ("dropout_probability", C.c_double),
                ("dropout_mask", Tensor), ("dropout_scale", Tensor), ("seed", Tensor), ("offset", Tensor), ("rng_dump", Tensor)]


# every symbol include/dfgpu.h declares
EXPORTS = [
    "dfgpu_last_error", "dfgpu_abi_version",
    "dfgpu_query_block_scale_quantize", "dfgpu_block_scale_quantize",
    "dfgpu_query_block_scale_quantize_pair", "dfgpu_block_scale_quantize_pair",
    "dfgpu_query_block_scale_dequantize", "dfgpu_block_scale_dequantize",
    "dfgpu_query_pointwise", "dfgpu_pointwise", "dfgpu_pointwise_input_count", "dfgpu_query_constants", "dfgpu_constants",
    "dfgpu_query_conv_fprop", "dfgpu_conv_fprop",
    "dfgpu_query_conv_fprop_pair", "dfgpu_conv_fprop_pair",
    "dfgpu_query_matmul", "dfgpu_matmul",
    "dfgpu_query_matmul_fp8", "dfgpu_matmul_fp8",
    "dfgpu_query_sdpa_forward", "dfgpu_sdpa_forward", "dfgpu_sdpa_paged_decode_static",
    "dfgpu_selfcheck_e4m3", "dfgpu_debug_scale_codes", "dfgpu_debug_encode_e4m3", "dfgpu_device_status",
]


class DfgpuError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"dfgpu status {code}: {message}")
        self.code = code


_LIB: Optional[C.CDLL] = None


def library_path() -> Path:
    return Path(__file__).resolve().parent / "_build" / "libdfgpu.so"


def load() -> C.CDLL:
    """Load libdfgpu.so. There is no fallback: a missing library is an error."""
    global _LIB
    if _LIB is None:
        path = library_path()
        if not path.exists():
            raise RuntimeError(f"{path} is missing: run `python -m deepforge_b200.build` (or __graft_entry__.build())")
        lib = C.CDLL(str(path))
        lib.dfgpu_last_error.restype = C.c_char_p
        for name in EXPORTS:
            getattr(lib, name)
        _LIB = lib
    return _LIB


def _check(code: int) -> None:
    if code != 0:
        raise DfgpuError(code, load().dfgpu_last_error().decode(errors="replace"))


def _pointers(values: Iterable[Optional[int]]):
    values = [C.c_void_p(v or None) for v in values]
    return (C.c_void_p * len(values))(*values)


def _call(name: str, params, pointers: Sequence[Optional[int]], scratch: Optional[int], stream: Optional[int]) -> None:
    fn = getattr(load(), name)
    fn.restype = C.c_int
    _check(fn(C.byref(params), _pointers(pointers), C.c_void_p(scratch or None), C.c_void_p(stream or None)))


def query(name: str, params) -> PlanInfo:
    info = PlanInfo()
    fn = getattr(load(), "dfgpu_query_" + name)
    fn.restype = C.c_int
    _check(fn(C.byref(params), C.byref(info)))
    return info


def block_scale_quantize(params, x, y, scale, scratch=None, stream=None):
    _call("dfgpu_block_scale_quantize", params, [x, y, scale], scratch, stream)


def block_scale_quantize_pair(params, first, second, stream=None):
    """first, second: (x, y, scale) device pointers of the two tensors."""
    _call("dfgpu_block_scale_quantize_pair", params, [*first, *second], None, stream)


def block_scale_dequantize(params, x, scale, y, scratch=None, stream=None):
    _call("dfgpu_block_scale_dequantize", params, [x, scale, y], scratch, stream)


def constants(params, destinations, stream=None):
    _call("dfgpu_constants", params, list(destinations), None, stream)


def pointwise(params, in0, in1, out, scratch=None, stream=None, in2=0):
    _call("dfgpu_pointwise", params, [in0, in1, out, in2], scratch, stream)


def conv_fprop(params, x, w, y, extra0=None, extra1=None, scratch=None, stream=None):
    _call("dfgpu_conv_fprop", params, [x, w, y, extra0, extra1], scratch, stream)


def conv_fprop_pair(params, x, w_first, w_second, y, first_extra=(None, None), second_extra=(None, None), stream=None):
    _call("dfgpu_conv_fprop_pair", params, [x, w_first, w_second, y, *first_extra, *second_extra], None, stream)


def matmul(params, a, b, c, a_scale=None, b_scale=None, extra0=None, extra1=None, scratch=None, stream=None):
    _call("dfgpu_matmul", params, [a, b, c, a_scale, b_scale, extra0, extra1], scratch, stream)


def matmul_fp8(params, a, b, c, amax, descale_a, descale_b, scale_c, scratch=None, stream=None):
    _call("dfgpu_matmul_fp8", params, [a, b, c, amax, descale_a, descale_b, scale_c], scratch, stream)


def sdpa_forward(params, pointers: Sequence[Optional[int]], scratch=None, stream=None):
    """pointers: Q, K, V, O, Stats, Max, Sum_exp, SEQ_LEN_Q, SEQ_LEN_KV, Page_table_K, Page_table_V[, Bias[, SINK_TOKEN[, Block_mask[,
    Page_table_K offsets, Page_table_V offsets[, Dropout_mask, Dropout_scale, Seed, Offset, RNG_DUMP]]]]]."""
    assert 11 <= len(pointers) <= 21
    pointers = list(pointers) + [None] * (21 - len(pointers))
    _call("dfgpu_sdpa_forward", params, pointers, scratch, stream)


def sdpa_paged_decode_static(params, pointers: Sequence[Optional[int]], stream=None):
    """Paged decode with the library's built-in 8 MiB scratch: no caller buffer, no allocation."""
    assert len(pointers) == 11
    fn = load().dfgpu_sdpa_paged_decode_static
    fn.restype = C.c_int
    _check(fn(C.byref(params), _pointers(pointers), C.c_void_p(stream or None)))


def selfcheck_e4m3(first_bits: int, count: int, result_ptr: int, stream=None) -> None:
    fn = load().dfgpu_selfcheck_e4m3
    fn.restype = C.c_int
    _check(fn(C.c_uint32(first_bits), C.c_uint64(count), C.c_void_p(result_ptr), C.c_void_p(stream or None)))


def debug_scale_codes(amax_ptr: int, codes_ptr: int, count: int, stream=None) -> None:
    fn = load().dfgpu_debug_scale_codes
    fn.restype = C.c_int
    _check(fn(C.c_void_p(amax_ptr), C.c_void_p(codes_ptr), C.c_int64(count), C.c_void_p(stream or None)))


def debug_encode_e4m3(values_ptr: int, codes_ptr: int, count: int, stream=None) -> None:
    fn = load().dfgpu_debug_encode_e4m3
    fn.restype = C.c_int
    _check(fn(C.c_void_p(values_ptr), C.c_void_p(codes_ptr), C.c_int64(count), C.c_void_p(stream or None)))


def device_status() -> int:
    """Synchronise, then read and clear the device-side status word (0 = healthy)."""
    value = C.c_int(0)
    fn = load().dfgpu_device_status
    fn.restype = C.c_int
    _check(fn(C.byref(value)))
    return value.value
