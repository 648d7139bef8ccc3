"""MATMUL_FP8 on the GPU through Executable.execute, against the CPU oracle evaluating the same document.

The synthetic operands keep every partial sum exactly representable in f32 (workloads.matmul_fp8), so the
result does not depend on the order of the additions and both kernels -- the general one, which adds in the
reference's k order, and the tcgen05 one -- are held to the oracle bit for bit: C as FLOAT, C rounded to
BFLOAT16 / HALF, C as E4M3 codes, and Amax_C."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "oracle"))
import graph_oracle  # noqa: E402
from deepforge_b200 import dfgpu, harness, runtime, synthetic, workloads  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _device_healthy():
    yield
    assert dfgpu.device_status() == 0


def run_both(wl, options=0, overrides=None):
    session = harness.Session(wl, options=options)
    for uid, array in (overrides or {}).items():
        session.dev[uid].copy_(torch.from_numpy(np.ascontiguousarray(array).reshape(-1).view(np.uint8).copy()))
    session.run()
    inputs = {uid: graph_oracle.widen(session.raw(uid), wl.tensor(uid)["data_type"]) for uid in wl.inputs}
    return session, graph_oracle.run(wl.document, inputs)


def as_stored(reference_f32, data_type):
    """The oracle holds a floating C as f32; the device stored its rounding."""
    if data_type == "BFLOAT16":
        return synthetic.bf16_bits_to_f32(synthetic.to_bf16_bits(reference_f32))
    if data_type == "HALF":
        return reference_f32.astype(np.float16).astype(np.float32)
    return reference_f32


def check(session, reference, c_type):
    actual = session.output(26)
    expected = reference[26] if c_type.startswith("FP8") else as_stored(reference[26], c_type)
    assert np.array_equal(actual, expected), f"{int(np.sum(actual != expected))} of {actual.size} elements differ"
    assert session.output(27).tobytes() == reference[27].astype(np.float32).tobytes()


def test_reference_known_answer():
    """test/Compiler/SpecializedOpsTest.cpp:889-914 of the reference."""
    wl = workloads.matmul_fp8(2, 2, 2, c_type="FLOAT", scalars=(0.5, 2.0, 1.0))
    session, _ = run_both(wl, overrides={21: np.array([0x38, 0x40, 0x44, 0x48], dtype=np.uint8), 22: np.array([0x38, 0xb8, 0x40, 0x38], dtype=np.uint8)})
    assert session.output(26).tolist() == [5.0, 1.0, 11.0, 1.0]
    assert session.output(27).tolist() == [11.0]


@pytest.mark.parametrize("c_type", ["FLOAT", "BFLOAT16", "HALF", "FP8_E4M3"])
@pytest.mark.parametrize("shape", [dict(m=5, k=7, n=3), dict(m=33, k=70, n=17, batch=(2, 3), a_batch=(1, 3), b_batch=(2, 1)), dict(m=16, k=128, n=48, b_k_major=True)])
def test_general_kernel_matches_oracle(c_type, shape):
    wl = workloads.matmul_fp8(c_type=c_type, **shape)
    session, reference = run_both(wl)
    assert f"kernel={dfgpu.MATMUL_FP8_SCALAR}" in session.exe.plan_text()
    check(session, reference, c_type)


@pytest.mark.parametrize("c_type", ["FLOAT", "BFLOAT16", "FP8_E4M3"])
@pytest.mark.parametrize("shape", [dict(m=128, k=128, n=128), dict(m=256, k=1024, n=384, b_k_major=True), dict(m=384, k=512, n=256), dict(m=2560, k=128, n=2048)])
def test_tcgen05_kernel_matches_oracle(c_type, shape):
    """The last shape has more tiles than SMs, so the persistent loop and the half-tile tail both run."""
    wl = workloads.matmul_fp8(c_type=c_type, **shape)
    session, reference = run_both(wl)
    assert f"kernel={dfgpu.MATMUL_FP8_UMMA}" in session.exe.plan_text()
    check(session, reference, c_type)
    # and the general kernel on the same problem
    if shape["m"] <= 384:
        session, _ = run_both(wl, options=runtime.NO_TENSOR_CORES)
        check(session, reference, c_type)


@pytest.mark.parametrize("a_type,b_type", [("FP8_E5M2", "FP8_E5M2"), ("FP8_E5M2", "FP8_E4M3"), ("FP8_E4M3", "FP8_E5M2")])
@pytest.mark.parametrize("shape,c_type", [(dict(m=9, k=33, n=5), "FLOAT"), (dict(m=9, k=33, n=5), "FP8_E5M2"), (dict(m=256, k=512, n=384), "BFLOAT16"),
                                          (dict(m=128, k=256, n=128, b_k_major=True), "FP8_E4M3"), (dict(m=128, k=128, n=256), "FP8_E5M2")])
def test_e5m2_operands_and_output(a_type, b_type, shape, c_type):
    wl = workloads.matmul_fp8(c_type=c_type, a_type=a_type, b_type=b_type, **shape)
    session, reference = run_both(wl)
    tensor_core = shape["m"] >= 128 and c_type != "FP8_E5M2"
    assert f"kernel={dfgpu.MATMUL_FP8_UMMA if tensor_core else dfgpu.MATMUL_FP8_SCALAR}" in session.exe.plan_text()
    check(session, reference, c_type)


def test_e5m2_output_saturates_and_keeps_nan():
    wl = workloads.matmul_fp8(8, 16, 8, c_type="FP8_E5M2", scalars=(1.0, 1.0, 65536.0))
    codes = wl.inputs[21]()
    codes[5] = 0x7f
    session, reference = run_both(wl, overrides={21: codes})
    actual = session.output(26)
    assert np.array_equal(actual, reference[26])
    assert np.all(actual[:8] == 0x7f) and np.any((actual[8:] & 0x7f) == 0x7b) and np.all((actual[8:] & 0x7f) <= 0x7b)
    wl = workloads.matmul_fp8(8, 16, 8, c_type="FP8_E5M2", scalars=(1.0, 1.0, 2.0 ** -22))
    session, reference = run_both(wl)
    assert np.array_equal(session.output(26), reference[26]) and not np.any(session.output(26) == 0x80)


@pytest.mark.parametrize("shape", [dict(m=4, k=8, n=4), dict(m=128, k=128, n=128)])
def test_nan_saturation_and_signed_zero(shape):
    wl = workloads.matmul_fp8(c_type="FP8_E4M3", scalars=(1.0, 1.0, 1024.0), **shape)
    codes = wl.inputs[21]()
    codes[3] = 0x7f  # one NaN in row 0 of A
    session, reference = run_both(wl, overrides={21: codes})
    actual = session.output(26)
    assert np.array_equal(actual, reference[26])
    n = shape["n"]
    assert np.all(actual[:n] == 0x7f) and np.isnan(session.output(27)[0]) and np.isnan(reference[27][0])
    assert np.all((actual[n:] & 0x7f) <= 0x7e) and np.any((actual[n:] & 0x7f) == 0x7e)  # saturated, never the NaN code
    # tiny results: negatives that round to zero give +0
    wl = workloads.matmul_fp8(c_type="FP8_E4M3", scalars=(1.0, 1.0, 2.0 ** -16), **shape)
    session, reference = run_both(wl)
    assert np.array_equal(session.output(26), reference[26])
    assert not np.any(session.output(26) == 0x80)


def test_inexact_sums_within_the_f32_gate():
    """Operands over the whole exponent range: the tensor core adds in its own order, so C is held to the f32
    contraction gate (max |d| <= 1e-4 max |ref|) and Amax_C to the same relative bound."""
    wl = workloads.matmul_fp8(256, 1024, 256, c_type="FLOAT", exact=False, scalars=(1.0, 1.0, 1.0))
    session, reference = run_both(wl)
    assert f"kernel={dfgpu.MATMUL_FP8_UMMA}" in session.exe.plan_text()
    scale = float(np.max(np.abs(reference[26])))
    assert float(np.max(np.abs(session.output(26) - reference[26]))) <= 1e-4 * scale
    assert abs(float(session.output(27)[0]) - float(reference[27][0])) <= 1e-4 * scale


def test_requesting_the_tcgen05_kernel_for_an_uncovered_shape_fails():
    params = dfgpu.MatmulFp8Params()
    params.a = dfgpu.tensor(dfgpu.E4M3, [100, 128], [128, 1])
    params.b = dfgpu.tensor(dfgpu.E4M3, [128, 128], [128, 1])
    params.c = dfgpu.tensor(dfgpu.F32, [100, 128], [128, 1])
    params.kernel = dfgpu.MATMUL_FP8_UMMA
    with pytest.raises(dfgpu.DfgpuError) as error:
        dfgpu.query("matmul_fp8", params)
    assert error.value.code == 20
