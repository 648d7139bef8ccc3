"""MATMUL_FP8 without a GPU: the oracle against the reference's own known answer
(test/Compiler/SpecializedOpsTest.cpp:889-914), kernel-selection plans, the argument table and the
rejections the reference's validate_matmul_fp8 makes (lib/Compiler/SpecializedGraph.cpp:409-496)."""
import copy
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "oracle"))
import df_oracle_binding as oracle  # noqa: E402
import graph_oracle  # noqa: E402
from deepforge_b200 import dfgpu, graphs, runtime  # noqa: E402
from deepforge_b200.runtime import DeepForgeError  # noqa: E402


def test_oracle_reproduces_the_reference_known_answer():
    # A = [[1, 2], [3, 4]], B = [[1, -1], [2, 1]] as E4M3 codes, descales 0.5 and 2, Scale_C 1
    doc = graphs.matmul_fp8(2, 2, 2)
    values = {21: np.array([0x38, 0x40, 0x44, 0x48], dtype=np.uint8), 22: np.array([0x38, 0xb8, 0x40, 0x38], dtype=np.uint8),
              23: np.array([0.5], dtype=np.float32), 24: np.array([2.0], dtype=np.float32), 25: np.array([1.0], dtype=np.float32)}
    out = graph_oracle.run(doc, values)
    assert out[26].tolist() == [5.0, 1.0, 11.0, 1.0]
    assert out[27].tolist() == [11.0]
    # Amax_C is taken before Scale_C, C after it
    values[25] = np.array([0.25], dtype=np.float32)
    out = graph_oracle.run(doc, values)
    assert out[26].tolist() == [1.25, 0.25, 2.75, 0.25] and out[27].tolist() == [11.0]


def test_oracle_amax_keeps_nan_and_c_encodes_like_the_reference():
    doc = graphs.matmul_fp8(1, 2, 2, c_type="FP8_E4M3")
    values = {21: np.array([0x7f, 0x38], dtype=np.uint8), 22: np.array([0x38, 0x38, 0x38, 0x38], dtype=np.uint8),
              23: np.array([1.0], dtype=np.float32), 24: np.array([1.0], dtype=np.float32), 25: np.array([1.0], dtype=np.float32)}
    out = graph_oracle.run(doc, values)
    assert np.isnan(out[27][0]) and out[26].tolist() == [0x7f, 0x7f]
    # saturation at 448 and the negative that rounds to zero (-> +0)
    values[21] = np.array([0x38, 0x38], dtype=np.uint8)   # 1, 1
    values[22] = np.array([0x40, 0xb8, 0x40, 0x38], dtype=np.uint8)  # [[2, -1], [2, 1]] -> sums 4, 0
    values[25] = np.array([1000.0], dtype=np.float32)
    assert graph_oracle.run(doc, values)[26].tolist() == [0x7e, 0x00]
    values[22] = np.array([0x38, 0xb8, 0x38, 0x30], dtype=np.uint8)  # [[1, -1], [1, 0.5]] -> sums 2, -0.5
    values[25] = np.array([2.0 ** -12], dtype=np.float32)
    assert graph_oracle.run(doc, values)[26].tolist() == [0x00, 0x00]  # 2^-11 ties to even (zero); -2^-13 rounds to +0


def test_e5m2_codec_matches_the_reference_known_answers():
    """test/Compiler/SpecializedOpsTest.cpp:642-659 (decode 0x3c, 0x40, 0xc0, 0x38) and :716-735 (1, 2, -4, 8 divided by
    their block scales 2^-14, 2^-12 encode to 0x74, 0x78, 0xf4, 0x78); encoding rules of lib/Compiler/Numeric.cpp:396-425."""
    lib = oracle.lib()
    assert [lib.dfo_decode_e5m2(code) for code in (0x3c, 0x40, 0xc0, 0x38)] == [1.0, 2.0, -2.0, 0.5]
    assert [lib.dfo_encode_e5m2(value) for value in (16384.0, 32768.0, -16384.0, 32768.0)] == [0x74, 0x78, 0xf4, 0x78]
    assert lib.dfo_decode_e5m2(0x7c) == float("inf") and np.isnan(lib.dfo_decode_e5m2(0x7e)) and lib.dfo_decode_e5m2(0x01) == 2.0 ** -16
    assert lib.dfo_encode_e5m2(float("inf")) == 0x7b and lib.dfo_encode_e5m2(-1e9) == 0xfb and lib.dfo_encode_e5m2(57344.0) == 0x7b
    assert lib.dfo_encode_e5m2(float("nan")) == 0x7f and lib.dfo_encode_e5m2(-0.0) == 0x80 and lib.dfo_encode_e5m2(-2.0 ** -18) == 0x00
    assert lib.dfo_encode_e5m2(1.125) == 0x3c and lib.dfo_encode_e5m2(1.375) == 0x3e  # ties go to the even code
    for code in range(256):  # every finite code survives a round trip
        if (code & 0x7f) < 0x7c:
            assert lib.dfo_encode_e5m2(lib.dfo_decode_e5m2(code)) == code


def test_plans_and_argument_table():
    small = runtime.compile_graph(graphs.matmul_fp8(2, 2, 2))
    assert small.launch_count == 1 and small.workspace_size == 0
    assert f"matmul_fp8 kernel={dfgpu.MATMUL_FP8_SCALAR}" in small.plan_text()
    assert [a["uid"] for a in small.arguments()] == [21, 22, 23, 24, 25, 26, 27]
    access = {a["uid"]: a["access"] for a in small.arguments()}
    assert access[26] != "read" and access[27] != "read" and all(access[uid] == "read" for uid in (21, 22, 23, 24, 25))
    for c_type in ("FLOAT", "BFLOAT16", "FP8_E4M3"):
        for b_k_major in (False, True):
            big = runtime.compile_graph(graphs.matmul_fp8(256, 256, 384, c_type=c_type, b_k_major=b_k_major))
            assert f"matmul_fp8 kernel={dfgpu.MATMUL_FP8_UMMA}" in big.plan_text()
    # what the tcgen05 kernel does not take goes to the general one: HALF output, K not a multiple of 128, batches
    for doc in (graphs.matmul_fp8(256, 256, 256, c_type="HALF"), graphs.matmul_fp8(256, 192, 256), graphs.matmul_fp8(128, 128, 128, batch=(2,))):
        assert f"matmul_fp8 kernel={dfgpu.MATMUL_FP8_SCALAR}" in runtime.compile_graph(doc).plan_text()
    # E5M2 operands run on the same tensor-core kernel; an E5M2 output goes to the general one
    mixed = runtime.compile_graph(graphs.matmul_fp8(256, 256, 256, a_type="FP8_E5M2", b_type="FP8_E4M3", c_type="BFLOAT16"))
    assert f"matmul_fp8 kernel={dfgpu.MATMUL_FP8_UMMA}" in mixed.plan_text()
    assert f"matmul_fp8 kernel={dfgpu.MATMUL_FP8_SCALAR}" in runtime.compile_graph(graphs.matmul_fp8(256, 256, 256, c_type="FP8_E5M2")).plan_text()
    off = runtime.compile_graph(graphs.matmul_fp8(256, 256, 256), options=runtime.NO_TENSOR_CORES)
    assert f"matmul_fp8 kernel={dfgpu.MATMUL_FP8_SCALAR}" in off.plan_text()


def _mutated(change):
    doc = copy.deepcopy(graphs.matmul_fp8(4, 8, 4))
    change(doc)
    return doc


def _drop_input(name):
    def change(doc):
        del doc["nodes"][0]["inputs"][name]
    return change


def _set(uid, field, value):
    def change(doc):
        doc["tensors"][str(uid)][field] = value
    return change


def _add_override(doc):
    doc["tensors"]["28"] = graphs.tensor(28, "M_override", [1, 1, 1], "INT32")
    doc["nodes"][0]["inputs"]["M_override"] = 28


@pytest.mark.parametrize("change,code", [
    (_drop_input("Scale_C"), 8),                       # DFE_INVALID_VALUE: MATMUL_FP8 requires A, B, two descales, Scale_C, C, and Amax_C
    (_set(23, "dim", [2]), 15),                        # scale tensors must contain one FLOAT element
    (_set(27, "dim", [1, 2]), 15),                     # Amax_C must contain one FLOAT element
    (_set(24, "data_type", "HALF"), 10),               # scales are FLOAT
    (_set(21, "data_type", "FLOAT"), 10),              # A must be FP8
    (_set(26, "dim", [1, 4, 5]), 15),                  # M, N, K inconsistent
    (_set(21, "dim", [3, 4, 8]), 15),                  # batch not broadcast-compatible
    (_add_override, 20),                               # extent overrides are not executable here
])
def test_rejections(change, code):
    doc = _mutated(change)
    for uid in ("21", "26", "23", "27"):  # keep the strides those of a packed tensor of the new extents
        t = doc["tensors"][uid]
        t["stride"] = graphs.contiguous(t["dim"])
    with pytest.raises(DeepForgeError) as error:
        runtime.compile_graph(doc)
    assert error.value.code == code, str(error.value)
