"""Builders for cudnn-frontend v1.24.0 serialized Graph documents (JSON dicts): the five
benchmark configurations and the small graphs the tests use. Field names and layout are
exactly what the pinned Frontend serializer emits, as the reference's fixtures show
(test/fixtures/conv2d_f32.json in the reference)."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

FLT_MAX = 3.4028234663852886e38


def contiguous(dims: Sequence[int]) -> List[int]:
    strides = [1] * len(dims)
    for i in range(len(dims) - 2, -1, -1):
        strides[i] = strides[i + 1] * dims[i + 1]
    return strides


def nhwc(dims: Sequence[int]) -> List[int]:
    n, c, h, w = dims
    return [h * w * c, 1, w * c, c]


def tensor(uid: int, name: str, dims: Sequence[int], data_type: str = "FLOAT", strides: Optional[Sequence[int]] = None,
           virtual: bool = False, reordering: str = "NONE") -> dict:
    return {"name": name, "data_type": data_type, "dim": list(dims), "stride": list(strides) if strides is not None else contiguous(dims),
            "is_virtual": virtual, "pass_by_value": None, "is_pass_by_value": False, "reordering_type": reordering, "uid": uid,
            "uid_assigned": True}


def document(name: str, nodes: List[dict], tensors: List[dict], io: str = "FLOAT", intermediate: str = "FLOAT", graph_uid: int = 1) -> dict:
    return {
        "context": {"name": name, "compute_data_type": "FLOAT", "intermediate_data_type": intermediate, "io_data_type": io, "sm_count": -1,
                    "is_dynamic_shape_enabled": False, "is_override_shape_enabled": False},
        "graph_uid": graph_uid, "json_version": "1.0", "cudnn_backend_version": "not-used", "cudnn_frontend_version": 12400,
        "nodes": nodes, "tensors": {str(t["uid"]): t for t in tensors},
    }


def conv_node(name: str, x: int, w: int, y: int, pad=(1, 1), post_pad=None, stride=(1, 1), dilation=(1, 1), mode="CROSS_CORRELATION") -> dict:
    return {"tag": "CONV_FPROP", "name": name, "compute_data_type": "FLOAT", "inputs": {"X": x, "W": w}, "outputs": {"Y": y},
            "pre_padding": list(pad), "post_padding": list(post_pad if post_pad is not None else pad), "stride": list(stride),
            "dilation": list(dilation), "math_mode": mode}


def pointwise_node(name: str, mode: str, in0: int, out: int, in1: Optional[int] = None, lower=None, upper=None, slope=None,
                   in2: Optional[int] = None, axis=None, swish_beta=None, elu_alpha=None, softplus_beta=None) -> dict:
    inputs = {"IN_0": in0}
    if in1 is not None:
        inputs["IN_1"] = in1
    if in2 is not None:
        inputs["IN_2"] = in2
    return {"tag": "POINTWISE", "name": name, "compute_data_type": "FLOAT", "inputs": inputs, "outputs": {"OUT_0": out}, "mode": mode,
            "axis": axis, "relu_lower_clip": lower, "relu_upper_clip": upper, "relu_lower_clip_slope": slope, "swish_beta": swish_beta,
            "elu_alpha": elu_alpha, "softplus_beta": softplus_beta}


def scalar_pointwise(embedded: Optional[dict] = None, mode: str = "ADD", data_type: str = "FLOAT") -> dict:
    """X [2, 3] (mode) ALPHA [1, 1] -> Y, ALPHA passed by value: the reference's runtime-scalar graph
    (test/Compiler/FoundationalMathOpsTest.cpp:190-211) and, with `embedded` = the Frontend's scalar variant
    {"index": ..., "value": ...}, its embedded-scalar graph (:213-221), where ALPHA is a constant the graph owns."""
    tensors = [tensor(601, "X", [2, 3]), tensor(602, "ALPHA", [1, 1], data_type), tensor(603, "Y", [2, 3])]
    tensors[1]["is_pass_by_value"] = True
    doc = document("runtime-scalar-pointwise" if embedded is None else "embedded-scalar-pointwise",
                   [pointwise_node("runtime_scalar_add", mode, 601, 603, 602)], tensors, graph_uid=2106 if embedded is None else 2107)
    if embedded is not None:
        doc["tensors"]["602"]["pass_by_value"] = dict(embedded)
        doc["pass_by_values"] = {"602": dict(embedded)}
    return doc


def pointwise_all_modes(dims: Sequence[int] = (2, 3), data_type: str = "FLOAT") -> dict:
    """One POINTWISE node per mode of the schema, in the shape of the reference's own test graph
    (test/Compiler/FoundationalMathOpsTest.cpp:126-167): UID 101 A [rows, columns], 102 B [columns] (broadcast over rows),
    103 T [rows, 1] (the selector of BINARY_SELECT), outputs 1000 + the mode's position in the schema's list; axis 1,
    ReLU clips 0.25 / 1.0 with slope 0.2, swish beta 0.5, ELU alpha 2, softplus beta 2 on every node."""
    from .dfgpu import pointwise_input_count
    rows, columns = dims
    tensors = [tensor(101, "A", [rows, columns], data_type), tensor(102, "B", [columns], data_type), tensor(103, "T", [rows, 1], data_type)]
    nodes = []
    for position, mode in enumerate(SCHEMA_POINTWISE_MODES):
        count = pointwise_input_count(mode)
        nodes.append(pointwise_node("pointwise_" + mode, mode, 101, 1000 + position, 102 if count >= 2 else None, 0.25, 1.0, 0.2,
                                    103 if count >= 3 else None, 1, 0.5, 2.0, 2.0))
        tensors.append(tensor(1000 + position, "O_" + mode, [rows, columns], data_type))
    return document("pointwise_all_modes", nodes, tensors, io=data_type, graph_uid=2101)


# lib/Import/Schema.cpp:301-316, in the schema's order
SCHEMA_POINTWISE_MODES = (
    "ADD", "MUL", "SQRT", "MAX", "MIN", "RELU_FWD", "TANH_FWD", "SIGMOID_FWD", "ELU_FWD", "GELU_FWD", "SOFTPLUS_FWD", "SWISH_FWD",
    "RELU_BWD", "TANH_BWD", "SIGMOID_BWD", "ELU_BWD", "GELU_BWD", "SOFTPLUS_BWD", "SWISH_BWD", "ERF", "IDENTITY",
    "GELU_APPROX_TANH_BWD", "GELU_APPROX_TANH_FWD", "GEN_INDEX", "BINARY_SELECT", "EXP", "LOG", "NEG", "MOD", "POW", "ABS", "CEIL",
    "COS", "FLOOR", "RSQRT", "SIN", "LOGICAL_NOT", "TAN", "SUB", "ADD_SQUARE", "DIV", "CMP_EQ", "CMP_NEQ", "CMP_GT", "CMP_GE",
    "CMP_LT", "CMP_LE", "LOGICAL_AND", "LOGICAL_OR", "RECIPROCAL")


def matmul_node(name: str, a: int, b: int, c: int) -> dict:
    return {"tag": "MATMUL", "name": name, "compute_data_type": "FLOAT", "inputs": {"A": a, "B": b}, "outputs": {"C": c}, "padding_value": 0.0}


def matmul_fp8_node(name: str, a: int, b: int, descale_a: int, descale_b: int, scale_c: int, c: int, amax: int) -> dict:
    return {"tag": "MATMUL_FP8", "name": name, "compute_data_type": "FLOAT",
            "inputs": {"A": a, "B": b, "Descale_A": descale_a, "Descale_B": descale_b, "Scale_C": scale_c}, "outputs": {"C": c, "Amax_C": amax}}


def matmul_fp8(m: int, k: int, n: int, c_type: str = "FLOAT", batch: Sequence[int] = (1,), b_k_major: bool = False,
               a_batch: Optional[Sequence[int]] = None, b_batch: Optional[Sequence[int]] = None, a_type: str = "FP8_E4M3",
               b_type: str = "FP8_E4M3") -> dict:
    """One MATMUL_FP8 node in the shape of the reference's own test graph (test/Compiler/SpecializedOpsTest.cpp:370-390):
    UIDs 21 A, 22 B, 23 Descale_A, 24 Descale_B, 25 Scale_C, 26 C, 27 Amax_C. `b_k_major` stores B as [N, K]."""
    batch = list(batch)
    a_dims = list(a_batch if a_batch is not None else batch) + [m, k]
    b_dims = list(b_batch if b_batch is not None else batch) + [k, n]
    b_strides = None
    if b_k_major:
        b_strides = contiguous(b_dims[:-2] + [n, k])
        b_strides[-2], b_strides[-1] = b_strides[-1], b_strides[-2]
    tensors = [tensor(21, "A", a_dims, a_type), tensor(22, "B", b_dims, b_type, strides=b_strides),
               tensor(23, "Descale_A", [1]), tensor(24, "Descale_B", [1]), tensor(25, "Scale_C", [1]),
               tensor(26, "C", batch + [m, n], c_type), tensor(27, "Amax_C", [1])]
    return document("matmul-fp8", [matmul_fp8_node("matmul_fp8", 21, 22, 23, 24, 25, 26, 27)], tensors, io=c_type, graph_uid=5003)


def quantize_node(name: str, x: int, y: int, scale: int, block: int, axis: Optional[int]) -> dict:
    return {"tag": "BLOCK_SCALE_QUANTIZE", "name": name, "compute_data_type": "FLOAT", "inputs": {"X": x}, "outputs": {"Y": y, "scale": scale},
            "block_size": block, "axis": axis}


def dequantize_node(name: str, x: int, scale: int, y: int, blocks: Sequence[int]) -> dict:
    return {"tag": "BLOCK_SCALE_DEQUANTIZE", "name": name, "compute_data_type": "FLOAT", "inputs": {"X": x, "scale": scale}, "outputs": {"Y": y},
            "block_size": list(blocks), "is_negative_scale": False}


def sdpa_node(name: str, inputs: Dict[str, int], outputs: Dict[str, int], scale: float, padding: bool, stats: bool, max_seq_len_kv=None,
              left_bound=None, right_bound=None, alignment="TOP_LEFT", alibi: bool = False) -> dict:
    return {"tag": "SDPA", "name": name, "inputs": inputs, "outputs": outputs, "generate_stats": stats, "alibi_mask": alibi,
            "padding_mask": padding, "dropout_probability": None, "attn_scale_value": scale, "max_seq_len_kv": max_seq_len_kv,
            "mma_core_mode": None, "left_bound": left_bound, "right_bound": right_bound, "diagonal_alignment": alignment,
            "implementation": "AUTO", "is_mxfp8": False, "unfuse_fma": False}


# ---- the five benchmark configurations -------------------------------------------------------

def c1_conv(layout: str = "nhwc", n=1, c=64, h=56, w=56, k=64, r=3, pad=1) -> dict:
    """Single CONV_FPROP, f32. layout 'nhwc' is the form the reference accepts; 'nchw' is packed NCHW/KCRS."""
    xd, wd = [n, c, h, w], [k, c, r, r]
    p = h + 2 * pad - r + 1
    q = w + 2 * pad - r + 1
    yd = [n, k, p, q]
    strides = nhwc if layout == "nhwc" else contiguous
    tensors = [tensor(1, "X", xd, "FLOAT", strides(xd)), tensor(2, "W", wd, "FLOAT", strides(wd)), tensor(3, "Y", yd, "FLOAT", strides(yd))]
    return document("c1_conv_fprop", [conv_node("conv_fprop", 1, 2, 3, (pad, pad))], tensors)


def c2_bottleneck(n=32, h=56, w=56, c_in=256, c_mid=64, io: str = "BFLOAT16") -> dict:
    """ResNet-50 bottleneck: 1x1 conv -> +b1 -> ReLU -> 3x3 conv -> +b2 -> ReLU -> 1x1 conv -> + X."""
    xd, md = [n, c_in, h, w], [n, c_mid, h, w]
    t = [
        tensor(1, "X", xd, io, nhwc(xd)),
        tensor(2, "W1", [c_mid, c_in, 1, 1], io, nhwc([c_mid, c_in, 1, 1])),
        tensor(3, "B1", [1, c_mid, 1, 1], io, nhwc([1, c_mid, 1, 1])),
        tensor(4, "W2", [c_mid, c_mid, 3, 3], io, nhwc([c_mid, c_mid, 3, 3])),
        tensor(5, "B2", [1, c_mid, 1, 1], io, nhwc([1, c_mid, 1, 1])),
        tensor(6, "W3", [c_in, c_mid, 1, 1], io, nhwc([c_in, c_mid, 1, 1])),
        tensor(7, "Y", xd, io, nhwc(xd)),
        tensor(11, "conv1_out", md, "FLOAT", nhwc(md), True), tensor(12, "bias1_out", md, "FLOAT", nhwc(md), True),
        tensor(13, "relu1_out", md, "FLOAT", nhwc(md), True), tensor(14, "conv2_out", md, "FLOAT", nhwc(md), True),
        tensor(15, "bias2_out", md, "FLOAT", nhwc(md), True), tensor(16, "relu2_out", md, "FLOAT", nhwc(md), True),
        tensor(17, "conv3_out", xd, "FLOAT", nhwc(xd), True),
    ]
    nodes = [
        conv_node("conv1", 1, 2, 11, (0, 0)), pointwise_node("bias1", "ADD", 11, 12, 3), pointwise_node("relu1", "RELU_FWD", 12, 13),
        conv_node("conv2", 13, 4, 14, (1, 1)), pointwise_node("bias2", "ADD", 14, 15, 5), pointwise_node("relu2", "RELU_FWD", 15, 16),
        conv_node("conv3", 16, 6, 17, (0, 0)), pointwise_node("residual", "ADD", 17, 7, 1),
    ]
    return document("c2_bottleneck", nodes, t, io=io)


def c3_quantize_matmul(m=4096, k=4096, n=4096, io: str = "BFLOAT16", c_type: str = "BFLOAT16", block=32) -> dict:
    """quantize A (blocks along K) and B (blocks along K) to MXFP8, dequantize, MATMUL."""
    t = [
        tensor(1, "A", [m, k], io), tensor(2, "B", [k, n], io),
        tensor(3, "Aq", [m, k], "FP8_E4M3"), tensor(4, "SFA", [m, k // block], "FP8_E8M0"),
        tensor(5, "Bq", [k, n], "FP8_E4M3"), tensor(6, "SFB", [k // block, n], "FP8_E8M0"),
        tensor(7, "Adq", [m, k], "FLOAT", None, True), tensor(8, "Bdq", [k, n], "FLOAT", None, True),
        tensor(9, "C", [m, n], c_type),
    ]
    nodes = [
        quantize_node("quantize_a", 1, 3, 4, block, 1), quantize_node("quantize_b", 2, 5, 6, block, 0),
        dequantize_node("dequantize_a", 3, 4, 7, [1, block]), dequantize_node("dequantize_b", 5, 6, 8, [block, 1]),
        matmul_node("matmul", 7, 8, 9),
    ]
    return document("c3_quantize_matmul", nodes, t, io=io)


def c4_sdpa(b=8, h=32, s=2048, d=128, io: str = "BFLOAT16", causal: bool = True, stats: bool = True) -> dict:
    dims = [b, h, s, d]
    t = [tensor(1, "Q", dims, io), tensor(2, "K", dims, io), tensor(3, "V", dims, io), tensor(4, "O", dims, io)]
    outputs = {"O": 4}
    if stats:
        t.append(tensor(5, "Stats", [b, h, s, 1], "FLOAT"))
        outputs["Stats"] = 5
    node = sdpa_node("sdpa", {"Q": 1, "K": 2, "V": 3}, outputs, d ** -0.5, False, stats, right_bound=0 if causal else None)
    return document("c4_sdpa", [node], t, io=io)


def c5_paged_decode(batch=64, hq=32, hkv=8, d=128, pages=16384, block=64, max_len=8192, io: str = "BFLOAT16", compact: bool = False) -> dict:
    """compact: the page tables are stored back to back with only the slots each sequence needs (ragged batch prefix):
    tensors 9 (INT64) and 10 (INT32) hold the per-sequence offsets into them, [batch + 1, 1, 1, 1]."""
    table = max_len // block
    t = [
        tensor(1, "Q", [batch, hq, 1, d], io), tensor(2, "K", [pages, hkv, block, d], io), tensor(3, "V", [pages, hkv, block, d], io),
        tensor(4, "O", [batch, hq, 1, d], io), tensor(5, "SEQ_LEN_Q", [batch, 1, 1, 1], "INT32"), tensor(6, "SEQ_LEN_KV", [batch, 1, 1, 1], "INT32"),
        tensor(7, "Page_table_K", [batch, 1, table, 1], "INT32"), tensor(8, "Page_table_V", [batch, 1, table, 1], "INT32"),
    ]
    if compact:
        t[6].update(ragged_offset_uid=9, ragged_offset_name="Page_table_K_offsets")
        t[7].update(ragged_offset_uid=10, ragged_offset_name="Page_table_V_offsets")
        t += [tensor(9, "Page_table_K_offsets", [batch + 1, 1, 1, 1], "INT64"), tensor(10, "Page_table_V_offsets", [batch + 1, 1, 1, 1], "INT32")]
    node = sdpa_node("paged_decode", {"Q": 1, "K": 2, "V": 3, "SEQ_LEN_Q": 5, "SEQ_LEN_KV": 6, "Page_table_K": 7, "Page_table_V": 8},
                     {"O": 4}, d ** -0.5, True, False, max_seq_len_kv=max_len)
    return document("c5_paged_decode", [node], t, io=io)
