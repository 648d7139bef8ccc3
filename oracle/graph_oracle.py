"""Evaluate a serialized graph document on the CPU with the oracle, node by node --
TEST INFRASTRUCTURE ONLY (parity checker and timed CPU baseline; never the product path).

Every floating tensor is held as f32: a BFLOAT16/HALF graph input is widened exactly and
the graph is run as its all-FLOAT twin, which is the reference's own semantics (it accepts
only FLOAT tensors outside the block-scale tags). Block-scale quantize reads its input in
the tensor's real storage type, so codes and scales are bit-exact checks.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import numpy as np

import df_oracle_binding as oracle
from deepforge_b200 import dfgpu, synthetic

FLT_MAX = 3.4028234663852886e38
_FLOATING = {"FLOAT", "BFLOAT16", "HALF"}
_CODE = {"FP8_E4M3": dfgpu.E4M3, "FP8_E5M2": dfgpu.E5M2, "FP8_E8M0": dfgpu.E8M0, "INT32": dfgpu.I32, "UINT8": dfgpu.U8, "INT64": dfgpu.I64,
         "FP4_E2M1": dfgpu.FP4, "INT4": dfgpu.I4}
_STORAGE = {"FLOAT": dfgpu.F32, "BFLOAT16": dfgpu.BF16, "HALF": dfgpu.F16}


def widen(array: np.ndarray, data_type: str) -> np.ndarray:
    """Host array in storage dtype -> what the oracle holds (f32 for floating tensors)."""
    if data_type == "BFLOAT16":
        return synthetic.bf16_bits_to_f32(np.ascontiguousarray(array).view(np.uint16).reshape(-1))
    if data_type == "HALF":
        return np.ascontiguousarray(array).view(np.float16).reshape(-1).astype(np.float32)
    if data_type == "FLOAT":
        return np.ascontiguousarray(array).view(np.float32).reshape(-1).copy()
    if data_type == "INT32":
        return np.ascontiguousarray(array).view(np.int32).reshape(-1).copy()
    if data_type == "INT64":
        return np.ascontiguousarray(array).view(np.int64).reshape(-1).copy()
    return np.ascontiguousarray(array).view(np.uint8).reshape(-1).copy()


def _span(t: dict) -> int:
    if t["reordering_type"] != "NONE":
        return int(np.prod(t["dim"]))
    return sum((d - 1) * s for d, s in zip(t["dim"], t["stride"])) + 1


def _desc(t: dict, as_storage: bool = False):
    if t["data_type"] in _FLOATING:
        dtype = _STORAGE[t["data_type"]] if as_storage else dfgpu.F32
    else:
        dtype = _CODE[t["data_type"]]
    reorder = dfgpu.REORDER_F8_128x4 if t["reordering_type"] == "F8_128x4" else dfgpu.REORDER_NONE
    return dfgpu.tensor(dtype, t["dim"], t["stride"], reorder)


def _alloc(t: dict) -> np.ndarray:
    if t["data_type"] in _FLOATING:
        return np.zeros(_span(t), dtype=np.float32)
    return np.zeros(_span(t), dtype=np.int32 if t["data_type"] == "INT32" else np.uint8)


def embedded_scalar(described: dict) -> np.ndarray:
    """The value of an embedded pass-by-value payload as the tensor's type holds it, widened to f32 for the floating
    types (lib/Compiler/FoundationalGraph.cpp:2165-2214: FLOAT is an f32 bit pattern, HALF / BFLOAT16 / DOUBLE a JSON
    number narrowed to the type, INT32 / INT64 integers)."""
    payload, data_type = described["pass_by_value"], described["data_type"]
    if data_type == "FLOAT":
        return np.array([int(payload["value"], 16)], np.uint32).view(np.float32)
    if data_type == "HALF":
        return np.array([payload["value"]], np.float64).astype(np.float16).astype(np.float32)
    if data_type == "BFLOAT16":
        from deepforge_b200 import synthetic
        return synthetic.bf16_bits_to_f32(synthetic.to_bf16_bits(np.array([payload["value"]], np.float32)))
    if data_type == "DOUBLE":
        return np.array([payload["value"]], np.float64)
    return np.array([payload["value"]], np.int32 if data_type == "INT32" else np.int64)


def run(document: dict, inputs: Dict[int, np.ndarray], matmul_rows: Optional[Tuple[int, int]] = None,
        sdpa_bh: Optional[Tuple[int, int]] = None, sdpa_q_step: int = 1, storage_inputs: Optional[Dict[int, np.ndarray]] = None,
        round_to_bf16: Tuple[int, ...] = (), threads: int = 1) -> Dict[int, np.ndarray]:
    """inputs: uid -> widened arrays (see widen()). storage_inputs: uid -> raw storage-dtype arrays
    for tensors a BLOCK_SCALE_QUANTIZE reads (so bf16/f16 inputs are decoded by the oracle itself).
    round_to_bf16: UIDs of intermediate tensors to round to bf16 once produced -- the "staged"
    oracle for a chain of bf16 tensor-core contractions, each of which reads bf16 operands.
    threads: host threads for the convolutions, matmuls and SDPA (batch, head) pairs; each output element is
    computed by one thread with the same arithmetic, so the results do not depend on it."""
    tensors = {int(k): v for k, v in document["tensors"].items()}
    values: Dict[int, np.ndarray] = dict(inputs)
    for uid, described in tensors.items():   # graph-owned constants win over anything the caller passes for their UID
        if described.get("pass_by_value") is not None:
            values[uid] = embedded_scalar(described)
    for node in document["nodes"]:
        tag = node["tag"]
        ins, outs = node["inputs"], node["outputs"]
        if tag == "CONV_FPROP":
            x, w, y = ins["X"], ins["W"], outs["Y"]
            values[y] = _alloc(tensors[y])
            attrs = oracle.conv_attrs(node["pre_padding"], node["post_padding"], node["stride"], node["dilation"], node["math_mode"] == "CONVOLUTION")
            oracle.conv_generic(_desc(tensors[x]), values[x], _desc(tensors[w]), values[w], _desc(tensors[y]), values[y], attrs, threads=threads)
        elif tag == "POINTWISE":
            out = outs["OUT_0"]
            values[out] = _alloc(tensors[out])
            mode = dfgpu.PW_MODES[node["mode"]]
            a, b, c = ins["IN_0"], ins.get("IN_1"), ins.get("IN_2")

            def number(key, default):
                value = node.get(key)
                return default if value is None else value
            oracle.pointwise_general(mode, _desc(tensors[a]), values[a], _desc(tensors[b]) if b is not None else None,
                                     values[b] if b is not None else None, _desc(tensors[c]) if c is not None else None,
                                     values[c] if c is not None else None, _desc(tensors[out]), values[out],
                                     number("relu_lower_clip", 0.0), number("relu_upper_clip", FLT_MAX),
                                     number("relu_lower_clip_slope", 0.0), number("elu_alpha", 1.0), number("softplus_beta", 1.0),
                                     number("swish_beta", 1.0), number("axis", 0), threads=threads)
        elif tag == "MATMUL":
            a, b, c = ins["A"], ins["B"], outs["C"]
            values[c] = _alloc(tensors[c])
            lo, hi = matmul_rows if matmul_rows else (0, -1)
            oracle.matmul(_desc(tensors[a]), values[a], _desc(tensors[b]), values[b], _desc(tensors[c]), values[c], lo, hi, threads=threads)
        elif tag == "MATMUL_FP8":
            a, b, c, amax = ins["A"], ins["B"], outs["C"], outs["Amax_C"]
            values[c] = _alloc(tensors[c])
            scalars = [float(np.asarray(values[ins[name]], dtype=np.float32).reshape(-1)[0]) for name in ("Descale_A", "Descale_B", "Scale_C")]
            result = oracle.matmul_fp8(_desc(tensors[a]), values[a], _desc(tensors[b]), values[b], _desc(tensors[c]), values[c], *scalars)
            values[amax] = np.full(_span(tensors[amax]), result, dtype=np.float32)
        elif tag == "BLOCK_SCALE_QUANTIZE":
            x, y, scale = ins["X"], outs["Y"], outs["scale"]
            values[y], values[scale] = _alloc(tensors[y]), _alloc(tensors[scale])
            axis = node["axis"] if node["axis"] is not None else -1
            if storage_inputs and x in storage_inputs:
                oracle.block_scale_quantize(_desc(tensors[x], True), storage_inputs[x], _desc(tensors[y]), values[y], _desc(tensors[scale]), values[scale], node["block_size"], axis)
            else:
                oracle.block_scale_quantize(_desc(tensors[x]), values[x], _desc(tensors[y]), values[y], _desc(tensors[scale]), values[scale], node["block_size"], axis)
        elif tag == "BLOCK_SCALE_DEQUANTIZE":
            x, scale, y = ins["X"], ins["scale"], outs["Y"]
            values[y] = _alloc(tensors[y])
            oracle.block_scale_dequantize(_desc(tensors[x]), values[x], _desc(tensors[scale]), values[scale], _desc(tensors[y]), values[y], node["block_size"])
        elif tag == "SDPA":
            p = oracle.SdpaParams()
            arrays = []
            for name, field in (("Q", "q"), ("K", "k"), ("V", "v")):
                uid = ins[name]
                if storage_inputs and uid in storage_inputs and uid not in values:
                    # large K/V pools stay in their storage type; the oracle widens per element
                    setattr(p, field, _desc(tensors[uid], True))
                    arrays.append(storage_inputs[uid])
                else:
                    setattr(p, field, _desc(tensors[uid]))
                    arrays.append(values[uid])
            p.o = _desc(tensors[outs["O"]])
            values[outs["O"]] = _alloc(tensors[outs["O"]])
            arrays.append(values[outs["O"]])
            for name, field in (("Stats", "stats"), ("Max", "max"), ("Sum_exp", "sum_exp")):
                if name in outs:
                    setattr(p, field, _desc(tensors[outs[name]]))
                    values[outs[name]] = _alloc(tensors[outs[name]])
                    arrays.append(values[outs[name]])
                else:
                    arrays.append(None)
            for name, field in (("SEQ_LEN_Q", "seq_q"), ("SEQ_LEN_KV", "seq_kv"), ("Page_table_K", "page_table_k"), ("Page_table_V", "page_table_v")):
                if name in ins:
                    setattr(p, field, _desc(tensors[ins[name]]))
                    arrays.append(values[ins[name]])
                else:
                    arrays.append(None)
            if "Bias" in ins:
                p.bias = _desc(tensors[ins["Bias"]])
                arrays.append(values[ins["Bias"]])
            else:
                arrays.append(None)
            if "SINK_TOKEN" in ins:
                p.sink = _desc(tensors[ins["SINK_TOKEN"]])
                arrays.append(values[ins["SINK_TOKEN"]])
            else:
                arrays.append(None)
            if "Block_mask" in ins:
                p.block_mask = _desc(tensors[ins["Block_mask"]])
                arrays.append(values[ins["Block_mask"]])
            else:
                arrays.append(None)
            for name, field in (("Page_table_K", "page_offsets_k"), ("Page_table_V", "page_offsets_v")):
                # a compact page table names its batch prefix in the table's own tensor entry
                offsets_uid = tensors[ins[name]].get("ragged_offset_uid") if name in ins else None
                if offsets_uid is not None:
                    setattr(p, field, _desc(tensors[offsets_uid], True))
                    arrays.append(storage_inputs[offsets_uid] if storage_inputs and offsets_uid in storage_inputs else values[offsets_uid])
                else:
                    arrays.append(None)
            # dropout: a probability with Seed and Offset (and optionally RNG_DUMP), or the caller's Dropout_mask and Dropout_scale
            for name in ("Dropout_mask", "Dropout_scale", "Seed", "Offset"):
                arrays.append((storage_inputs[ins[name]] if storage_inputs and ins[name] in storage_inputs else values[ins[name]]) if name in ins else None)
            if node.get("dropout_probability") is not None:
                p.dropout_kind, p.dropout_probability = 1, float(node["dropout_probability"])
            elif "Dropout_mask" in ins:
                p.dropout_kind = 2
                p.dropout_mask = _desc(tensors[ins["Dropout_mask"]])
            if "RNG_DUMP" in outs:
                p.rng_dump = _desc(tensors[outs["RNG_DUMP"]])
                values[outs["RNG_DUMP"]] = _alloc(tensors[outs["RNG_DUMP"]])
                arrays.append(values[outs["RNG_DUMP"]])
            else:
                arrays.append(None)
            p.alibi_mask = int(bool(node.get("alibi_mask")))
            p.attn_scale = node["attn_scale_value"] if node["attn_scale_value"] is not None else 1.0
            p.padding_mask = int(node["padding_mask"])
            if node["left_bound"] is not None:
                p.has_left_bound, p.left_bound = 1, node["left_bound"]
            if node["right_bound"] is not None:
                p.has_right_bound, p.right_bound = 1, node["right_bound"]
            p.bottom_right = int(node["diagonal_alignment"] == "BOTTOM_RIGHT")
            k_t = tensors[ins["K"]]
            if node["max_seq_len_kv"] is not None:
                p.s_kv = node["max_seq_len_kv"]
            elif "Page_table_K" in ins:
                p.s_kv = tensors[ins["Page_table_K"]]["dim"][2] * k_t["dim"][2]
            else:
                p.s_kv = k_t["dim"][2]
            q_t = tensors[ins["Q"]]
            lo, hi = sdpa_bh if sdpa_bh else (0, q_t["dim"][0] * q_t["dim"][1])
            oracle.sdpa_forward(p, arrays, lo, hi, sdpa_q_step, threads=threads)
        else:
            raise NotImplementedError(tag)
        for uid in outs.values():
            if uid in round_to_bf16:
                values[uid] = synthetic.round_to_bf16(values[uid])
    return values
