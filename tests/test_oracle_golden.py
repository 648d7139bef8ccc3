"""Pins the CPU oracle against the known answers the reference's own tests hold.

Sources (paths inside the reference project):
  test/Compiler/SpecializedOpsTest.cpp:625-887   block-scale codes, scales, F8_128x4
  test/Compiler/CompilerTest.cpp:76-113,195-200  single-node conv vs an f64 reference
  test/Compiler/TrainingConvOpsTest.cpp:439-481  conv -> RELU exact case
  test/Compiler/FoundationalMathOpsTest.cpp:294-322,1090-1125  batched matmul + bias
  test/Compiler/SequenceOpsTest.cpp:371-509      SDPA in-test oracle (f64), tolerance 8e-5*(1+|ref|)
  test/Compiler/SequenceOpsTest.cpp:1945-2009,2149-2158  paged K/V tables, invalid page ids
"""
import ctypes as C
import math

import numpy as np
import pytest

import oracle
from deepforge_b200 import dfgpu
from deepforge_b200.dfgpu import BF16, E4M3, E5M2, E8M0, F16, F32, FP4, I4, I32, REORDER_F8_128x4, tensor

INF = float("inf")
NAN = float("nan")


# ---- codecs ------------------------------------------------------------------------

def test_e4m3_decode_table_and_roundtrip():
    lib = oracle.lib()
    assert lib.dfo_decode_e4m3(0x38) == 1.0
    assert lib.dfo_decode_e4m3(0x40) == 2.0
    assert lib.dfo_decode_e4m3(0xb8) == -1.0
    assert lib.dfo_decode_e4m3(0x7e) == 448.0
    assert lib.dfo_decode_e4m3(0x01) == 2.0 ** -9
    assert math.isnan(lib.dfo_decode_e4m3(0x7f)) and math.isnan(lib.dfo_decode_e4m3(0xff))
    for code in range(256):
        if (code & 0x7f) == 0x7f:
            continue
        assert lib.dfo_encode_e4m3(lib.dfo_decode_e4m3(code)) == code, hex(code)


def test_e4m3_encode_corner_cases():
    lib = oracle.lib()
    assert lib.dfo_encode_e4m3(0.0) == 0x00
    assert lib.dfo_encode_e4m3(-0.0) == 0x80
    # a non-zero negative that rounds to zero is +0 in the reference's search
    assert lib.dfo_encode_e4m3(-1e-6) == 0x00
    assert lib.dfo_encode_e4m3(-(2.0 ** -10)) == 0x00
    assert lib.dfo_encode_e4m3(-(2.0 ** -10) * 1.0001) == 0x81
    assert lib.dfo_encode_e4m3(2.0 ** -10) == 0x00  # tie to even
    assert lib.dfo_encode_e4m3(3 * 2.0 ** -10) == 0x02  # tie between 1 and 2 -> even
    assert lib.dfo_encode_e4m3(448.0) == 0x7e
    assert lib.dfo_encode_e4m3(464.0) == 0x7e
    assert lib.dfo_encode_e4m3(1e9) == 0x7e
    assert lib.dfo_encode_e4m3(-1e9) == 0xfe
    assert lib.dfo_encode_e4m3(INF) == 0x7e
    assert lib.dfo_encode_e4m3(-INF) == 0xfe
    assert lib.dfo_encode_e4m3(NAN) == 0x7f
    assert lib.dfo_encode_e4m3(-NAN) == 0x7f


def test_e8m0_codes():
    lib = oracle.lib()
    assert lib.dfo_encode_e8m0(1.0) == 127
    assert lib.dfo_encode_e8m0(2.0 ** -7) == 120
    assert lib.dfo_encode_e8m0(INF) == 0xfe
    assert lib.dfo_encode_e8m0(NAN) == 0xff
    assert lib.dfo_encode_e8m0(0.0) == 0
    assert lib.dfo_decode_e8m0(127) == 1.0 and lib.dfo_decode_e8m0(128) == 2.0
    assert math.isnan(lib.dfo_decode_e8m0(0xff))


def test_f8_128x4_offsets():
    lib = oracle.lib()
    assert lib.dfo_f8_128x4_offset(0, 32, 0, 128, 4) == 4
    assert lib.dfo_f8_128x4_offset(0, 127, 0, 128, 4) == 508


# ---- block scale -----------------------------------------------------------------------

def test_block_dequantize_known_answer():
    x = np.array([0x38, 0x40, 0xb8, 0x30], dtype=np.uint8)
    scale = np.array([127, 128], dtype=np.uint8)
    y = np.full(4, -99.0, dtype=np.float32)
    oracle.block_scale_dequantize(tensor(E4M3, [1, 4]), x, tensor(E8M0, [1, 2]), scale, tensor(F32, [1, 4]), y, [2])
    assert y.tolist() == [1.0, 2.0, -2.0, 1.0]


def test_block_quantize_known_answer():
    x = np.array([1.0, 2.0, -4.0, 8.0], dtype=np.float32)
    y = np.zeros(4, dtype=np.uint8)
    scale = np.zeros(2, dtype=np.uint8)
    oracle.block_scale_quantize(tensor(F32, [1, 4]), x, tensor(E4M3, [1, 4]), y, tensor(E8M0, [1, 2]), scale, 2, 1)
    assert scale.tolist() == [120, 122]
    assert y.tolist() == [0x70, 0x78, 0xf0, 0x78]


def test_block_quantize_exceptional_scales():
    x = np.array([INF, 0.0, NAN, 0.0], dtype=np.float32)
    y = np.zeros(4, dtype=np.uint8)
    scale = np.zeros(2, dtype=np.uint8)
    oracle.block_scale_quantize(tensor(F32, [1, 4]), x, tensor(E4M3, [1, 4]), y, tensor(E8M0, [1, 2]), scale, 2, 1)
    assert scale.tolist() == [0xfe, 0xff]
    assert y.tolist() == [0x7e, 0x00, 0x7f, 0x7f]


def test_e5m2_block_scale_known_answers():
    """FP8_E5M2 codes (test/Compiler/SpecializedOpsTest.cpp:640-659 dequantize, :716-735 quantize): the scale rule divides by 57344."""
    x = np.array([0x3c, 0x40, 0xc0, 0x38], dtype=np.uint8)
    scale = np.array([127, 128], dtype=np.uint8)
    y = np.full(4, -99.0, dtype=np.float32)
    oracle.block_scale_dequantize(tensor(E5M2, [1, 4]), x, tensor(E8M0, [1, 2]), scale, tensor(F32, [1, 4]), y, [2])
    assert y.tolist() == [1.0, 2.0, -4.0, 1.0]
    x = np.array([1.0, 2.0, -4.0, 8.0], dtype=np.float32)
    codes = np.zeros(4, dtype=np.uint8)
    scale = np.zeros(2, dtype=np.uint8)
    oracle.block_scale_quantize(tensor(F32, [1, 4]), x, tensor(E5M2, [1, 4]), codes, tensor(E8M0, [1, 2]), scale, 2, 1)
    assert scale.tolist() == [113, 115]
    assert codes.tolist() == [0x74, 0x78, 0xf4, 0x78]


def test_packed_four_bit_known_answers():
    """FP4_E2M1 codes with FP8_E4M3 scales through quantize and dequantize (test/Compiler/SpecializedOpsTest.cpp:736-754: 1, 2, -3, 6 come back
    as 1.03125, 2.0625, -3, 6) and signed INT4 nibbles with HALF scales into BFLOAT16 (:661-681), two codes per byte, low nibble first."""
    x = np.array([1.0, 2.0, -3.0, 6.0], dtype=np.float32)
    codes = np.zeros(2, dtype=np.uint8)
    scale = np.zeros(2, dtype=np.uint8)
    oracle.block_scale_quantize(tensor(F32, [1, 4]), x, tensor(FP4, [1, 4]), codes, tensor(E4M3, [1, 2]), scale, 2, 1)
    y = np.full(4, -99.0, dtype=np.float32)
    oracle.block_scale_dequantize(tensor(FP4, [1, 4]), codes, tensor(E4M3, [1, 2]), scale, tensor(F32, [1, 4]), y, [2])
    assert y.tolist() == [1.03125, 2.0625, -3.0, 6.0]
    nibbles = np.array([0xf8, 0x70], dtype=np.uint8)
    half_scales = np.array([0x3800, 0x4000], dtype=np.uint16)
    out = np.full(4, 0xffff, dtype=np.uint16)
    oracle.block_scale_dequantize(tensor(I4, [1, 4]), nibbles, tensor(F16, [1, 2]), half_scales, tensor(BF16, [1, 4]), out, [2])
    assert out.tolist() == [0xc080, 0xbf00, 0x0000, 0x4160]
    lib = oracle.lib()
    lib.dfo_decode_e2m1.restype = C.c_float
    assert [lib.dfo_decode_e2m1(code) for code in range(16)] == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    encode = lambda v: lib.dfo_encode_e2m1(C.c_float(v))
    assert [encode(v) for v in (0.0, -0.0, 0.25, 0.75, 1.25, 2.5, 5.0, 6.0, 7.0, -100.0, float("inf"), float("nan"), -0.2)] == \
        [0x0, 0x8, 0x0, 0x2, 0x2, 0x4, 0x6, 0x7, 0x7, 0xf, 0x7, 0x7, 0x0]


def test_bf16_fp8_f16_roundtrip_bits():
    x = np.array([0x3f80, 0x4000, 0xc080, 0x4100], dtype=np.uint16)
    packed = np.zeros(4, dtype=np.uint8)
    scale = np.zeros(2, dtype=np.uint8)
    y = np.full(4, 0xffff, dtype=np.uint16)
    oracle.block_scale_quantize(tensor(BF16, [1, 4]), x, tensor(E4M3, [1, 4]), packed, tensor(E8M0, [1, 2]), scale, 2, 1)
    oracle.block_scale_dequantize(tensor(E4M3, [1, 4]), packed, tensor(E8M0, [1, 2]), scale, tensor(F16, [1, 4]), y, [2])
    assert y.tolist() == [0x3c00, 0x4000, 0xc400, 0x4800]


def _f8_offset(m, k, m_extent=128, k_extent=4):
    return oracle.lib().dfo_f8_128x4_offset(0, m, k, m_extent, k_extent)


def test_reordered_dequantize():
    x = np.full(128 * 32, 0x38, dtype=np.uint8)
    scale = np.full(128 * 4, 127, dtype=np.uint8)
    scale[_f8_offset(32, 0)] = 128
    scale[_f8_offset(127, 0)] = 126
    y = np.full(128 * 32, -99.0, dtype=np.float32)
    sd = tensor(E8M0, [128, 4], [4, 1], REORDER_F8_128x4)
    oracle.block_scale_dequantize(tensor(E4M3, [128, 32]), x, sd, scale, tensor(F32, [128, 32]), y, [32])
    expected = np.ones((128, 32), dtype=np.float32)
    expected[32] = 2.0
    expected[127] = 0.5
    assert np.array_equal(y.reshape(128, 32), expected)


def test_transposed_reordered_dequantize():
    x = np.full(32 * 128, 0x38, dtype=np.uint8)
    scale = np.full(4 * 128, 127, dtype=np.uint8)
    scale[_f8_offset(32, 0)] = 128
    scale[_f8_offset(127, 0)] = 126
    y = np.full(32 * 128, -99.0, dtype=np.float32)
    sd = tensor(E8M0, [4, 128], [1, 4], REORDER_F8_128x4)
    oracle.block_scale_dequantize(tensor(E4M3, [32, 128]), x, sd, scale, tensor(F32, [32, 128]), y, [32, 1])
    expected = np.ones((32, 128), dtype=np.float32)
    expected[:, 32] = 2.0
    expected[:, 127] = 0.5
    assert np.array_equal(y.reshape(32, 128), expected)


def test_reordered_quantize_initialises_padded_slots():
    x = np.full((128, 32), 448.0, dtype=np.float32)
    x[32] = 224.0
    x[127] = 112.0
    y = np.zeros(128 * 32, dtype=np.uint8)
    scale = np.zeros(128 * 4, dtype=np.uint8)
    sd = tensor(E8M0, [128, 4], [4, 1], REORDER_F8_128x4)
    oracle.block_scale_quantize(tensor(F32, [128, 32]), x, tensor(E4M3, [128, 32]), y, sd, scale, 32, 1)
    assert np.all(y == 0x7e)
    for m in range(128):
        for k in range(4):
            expected = 127
            if k == 0 and m == 32:
                expected = 126
            if k == 0 and m == 127:
                expected = 125
            assert scale[_f8_offset(m, k)] == expected


def test_scale_rule_is_ceil_power_of_two():
    # amax 448 -> 1.0 exactly; just above -> doubles; 224 -> 0.5
    values = np.array([448.0, 448.5, 224.0, 3.0, 0.0, 1e-45, INF], dtype=np.float32)
    codes = oracle.block_scale_code_many(values)
    assert codes.tolist()[:4] == [127, 128, 126, 127 + math.ceil(math.log2(3.0 / 448.0))]
    assert codes[4] == 127  # amax 0 -> scale 1.0
    assert codes[5] == 127  # amax/448 underflows to 0 -> scale 1.0
    assert codes[6] == 0xfe


# ---- conv ------------------------------------------------------------------------------

def _np_conv_nhwc(x, w, pads, stride=(1, 1), dilation=(1, 1)):
    """f64 reference, the shape of CompilerTest.cpp:76-113."""
    n, h, wd, c = x.shape
    k, r, s, _ = w.shape
    top, left, bottom, right = pads
    oh = (h + top + bottom - (dilation[0] * (r - 1) + 1)) // stride[0] + 1
    ow = (wd + left + right - (dilation[1] * (s - 1) + 1)) // stride[1] + 1
    xp = np.zeros((n, h + top + bottom, wd + left + right, c), dtype=np.float64)
    xp[:, top:top + h, left:left + wd] = x
    y = np.zeros((n, oh, ow, k), dtype=np.float64)
    for ir in range(r):
        for is_ in range(s):
            patch = xp[:, ir * dilation[0]:ir * dilation[0] + oh * stride[0]:stride[0],
                       is_ * dilation[1]:is_ * dilation[1] + ow * stride[1]:stride[1]]
            y += np.einsum("nhwc,kc->nhwk", patch, w[:, ir, is_].astype(np.float64))
    return y


def _reference_test_inputs(count_x, count_w):
    x = np.array([((i * 7) % 19 - 9) / 7.0 for i in range(count_x)], dtype=np.float32)
    w = np.array([((i * 5) % 13 - 6) / 5.0 for i in range(count_w)], dtype=np.float32)
    return x, w


@pytest.mark.parametrize("shape", [
    # (n, h, w, c, k, r, s, (top, left, bottom, right)) -- the three conv fixtures of the reference
    (1, 5, 5, 3, 5, 3, 3, (1, 0, 1, 2)),
    (1, 5, 5, 17, 5, 3, 3, (1, 0, 1, 2)),
    (1, 5, 5, 3, 5, 3, 3, (0, 0, 0, 0)),
    (1, 17, 33, 29, 30, 3, 3, (1, 1, 1, 1)),
])
def test_conv_mvp_matches_f64_reference(shape):
    n, h, wd, c, k, r, s, pads = shape
    x, w = _reference_test_inputs(n * h * wd * c, k * r * s * c)
    reference = _np_conv_nhwc(x.reshape(n, h, wd, c), w.reshape(k, r, s, c), pads)
    for vf in (0, 8, 16):
        y = oracle.conv_mvp(x, w, n, h, wd, c, k, r, s, pads, vector_width=vf)
        assert np.all(np.abs(y - reference) <= 1e-4 + 1e-3 * np.abs(reference)), vf
    # the generic restatement on the same NHWC strides agrees too
    xd = tensor(F32, [n, c, h, wd], [h * wd * c, 1, wd * c, c])
    wdsc = tensor(F32, [k, c, r, s], [r * s * c, 1, s * c, c])
    oh, ow = reference.shape[1], reference.shape[2]
    yd = tensor(F32, [n, k, oh, ow], [oh * ow * k, 1, ow * k, k])
    y = np.zeros(n * oh * ow * k, dtype=np.float32)
    attrs = oracle.conv_attrs([pads[0], pads[1]], [pads[2], pads[3]], [1, 1], [1, 1])
    oracle.conv_generic(xd, x, wdsc, w, yd, y, attrs)
    assert np.all(np.abs(y.reshape(reference.shape) - reference) <= 1e-4 + 1e-3 * np.abs(reference))


def test_conv_special_values():
    # zero -> 0, NaN -> NaN, +Inf -> +Inf (VariantMatrixTest.cpp:216-275); the single-node
    # path multiplies materialised zero padding, so Inf next to a border gives NaN there.
    x = np.zeros((1, 3, 3, 1), dtype=np.float32)
    w = np.ones((1, 3, 3, 1), dtype=np.float32)
    assert np.all(oracle.conv_mvp(x, w, 1, 3, 3, 1, 1, 3, 3, (1, 1, 1, 1)) == 0.0)
    x[0, 1, 1, 0] = NAN
    assert np.all(np.isnan(oracle.conv_mvp(x, w, 1, 3, 3, 1, 1, 3, 3, (1, 1, 1, 1))))
    x[0, 1, 1, 0] = INF
    assert np.all(oracle.conv_mvp(x, w, 1, 3, 3, 1, 1, 3, 3, (1, 1, 1, 1)) == INF)
    w2 = w.copy()
    w2[0, 0, 0, 0] = INF  # the padded tap of the corner output multiplies 0 * Inf
    y = oracle.conv_mvp(np.ones_like(x), w2, 1, 3, 3, 1, 1, 3, 3, (1, 1, 1, 1))
    assert math.isnan(y[0, 0, 0, 0]) and y[0, 2, 2, 0] == INF


def test_conv_then_relu_exact():
    x = np.arange(1, 10, dtype=np.float32)
    w = np.array([1.0, -2.0, 0.5, 1.0], dtype=np.float32)
    xd = tensor(F32, [1, 1, 3, 3])
    wd = tensor(F32, [1, 1, 2, 2])
    yd = tensor(F32, [1, 1, 2, 2])
    conv = np.zeros(4, dtype=np.float32)
    oracle.conv_generic(xd, x, wd, w, yd, conv, oracle.conv_attrs([0, 0], [0, 0], [1, 1], [1, 1]))
    out = np.zeros(4, dtype=np.float32)
    oracle.pointwise(dfgpu.PW_RELU_FWD, yd, conv, None, None, yd, out)
    expected = []
    for p in range(2):
        for q in range(2):
            total = sum(x[(p + r) * 3 + q + s] * w[r * 2 + s] for r in range(2) for s in range(2))
            expected.append(max(float(total), 0.0))
    assert out.tolist() == expected


def test_grouped_strided_dilated_conv_against_f64():
    rng = np.random.default_rng(5)
    n, c, h, wd, k, r, s, groups = 2, 4, 9, 8, 6, 3, 2, 2
    x = rng.standard_normal((n, c, h, wd)).astype(np.float32)
    w = rng.standard_normal((k, c // groups, r, s)).astype(np.float32)
    pre, post, stride, dilation = [1, 2], [2, 0], [2, 1], [1, 2]
    oh = (h + pre[0] + post[0] - (dilation[0] * (r - 1) + 1)) // stride[0] + 1
    ow = (wd + pre[1] + post[1] - (dilation[1] * (s - 1) + 1)) // stride[1] + 1
    y = np.zeros((n, k, oh, ow), dtype=np.float32)
    oracle.conv_generic(tensor(F32, x.shape), x, tensor(F32, w.shape), w, tensor(F32, y.shape), y,
                        oracle.conv_attrs(pre, post, stride, dilation))
    reference = np.zeros_like(y, dtype=np.float64)
    for ik in range(k):
        g = ik // (k // groups)
        for ic in range(c // groups):
            for ir in range(r):
                for is_ in range(s):
                    for p in range(oh):
                        ih = p * stride[0] + ir * dilation[0] - pre[0]
                        if not 0 <= ih < h:
                            continue
                        for q in range(ow):
                            iw = q * stride[1] + is_ * dilation[1] - pre[1]
                            if 0 <= iw < wd:
                                reference[:, ik, p, q] += x[:, g * (c // groups) + ic, ih, iw].astype(np.float64) * w[ik, ic, ir, is_]
    assert np.all(np.abs(y - reference) <= 2e-5 * (1 + np.abs(reference)))


# ---- matmul ---------------------------------------------------------------------------------

def test_batched_matmul_with_broadcast_bias():
    a = np.array([1, 2, 3, 4, 5, 6, -1, 0, 1, 2, -2, 1], dtype=np.float32)
    b = np.array([1, 2, 0, 1, 1, 0], dtype=np.float32)
    bias = np.array([0.5, -1.0], dtype=np.float32)
    c = np.zeros(8, dtype=np.float32)
    out = np.full(8, -99.0, dtype=np.float32)
    cd = tensor(F32, [2, 2, 2])
    oracle.matmul(tensor(F32, [2, 2, 3]), a, tensor(F32, [1, 3, 2]), b, cd, c)
    oracle.pointwise(dfgpu.PW_ADD, cd, c, tensor(F32, [2]), bias, cd, out)
    assert out.tolist() == [4.5, 3.0, 10.5, 12.0, 0.5, -3.0, 3.5, 1.0]


# ---- SDPA -----------------------------------------------------------------------------------

def np_attention(q, k, v, scale, seq_q=None, seq_kv=None, right_bound=None, left_bound=None, bottom_right=False):
    """f64 reference in the shape of SequenceOpsTest.cpp:371-509 (no bias/dropout/alibi)."""
    b, hq, sq, _ = q.shape
    skv = k.shape[2]
    dv = v.shape[3]
    o = np.zeros((b, hq, sq, dv))
    stats = np.zeros((b, hq, sq))
    mx = np.zeros((b, hq, sq))
    sm = np.zeros((b, hq, sq))
    for n in range(b):
        for h in range(hq):
            kh = h // (hq // k.shape[1])
            vh = h // (hq // v.shape[1])
            for iq in range(sq):
                valid = np.ones(skv, dtype=bool)
                kv = np.arange(skv)
                if seq_q is not None:
                    valid &= (iq < seq_q[n]) & (kv < seq_kv[n])
                shift = 0
                if bottom_right:
                    shift = (seq_kv[n] - seq_q[n]) if seq_q is not None else skv - sq
                if right_bound is not None:
                    valid &= (kv - iq) <= shift + right_bound
                if left_bound is not None:
                    valid &= (kv - iq) > shift - left_bound
                scores = (k[n, kh].astype(np.float64) @ q[n, h, iq].astype(np.float64)) * scale
                scores = np.where(valid, scores.astype(np.float32).astype(np.float64), -np.inf)
                m = scores.max() if valid.any() else -np.inf
                e = np.where(valid, np.exp(scores - m), 0.0) if valid.any() else np.zeros(skv)
                total = e.sum()
                mx[n, h, iq], sm[n, h, iq] = m, total
                stats[n, h, iq] = m + (np.log(total) if total > 0 else -np.inf)
                if total > 0:
                    o[n, h, iq] = (e / total) @ v[n, vh].astype(np.float64)
    return o, stats, mx, sm


def _sdpa_params(q, k, v, o, scale, s_kv, **kw):
    p = oracle.SdpaParams()
    p.q, p.k, p.v, p.o = (tensor(F32, t.shape) for t in (q, k, v, o))
    p.attn_scale = scale
    p.s_kv = s_kv
    for key, value in kw.items():
        setattr(p, key, value)
    return p


def _close(actual, expected, tol=8e-5):
    expected = np.asarray(expected)
    finite = np.isfinite(expected)
    assert np.array_equal(actual[~finite], expected[~finite].astype(actual.dtype))
    assert np.all(np.abs(actual[finite] - expected[finite]) <= tol * (1 + np.abs(expected[finite])))


def test_sdpa_gqa_padding_window_stats():
    rng = np.random.default_rng(11)
    q = rng.standard_normal((2, 4, 5, 8)).astype(np.float32)
    k = rng.standard_normal((2, 2, 7, 8)).astype(np.float32)
    v = rng.standard_normal((2, 1, 7, 6)).astype(np.float32)
    o = np.full((2, 4, 5, 6), -99.0, dtype=np.float32)
    stats = np.zeros((2, 4, 5, 1), dtype=np.float32)
    mx = np.zeros_like(stats)
    sm = np.zeros_like(stats)
    seq_q = np.array([5, 3], dtype=np.int32)
    seq_kv = np.array([7, 4], dtype=np.int32)
    for bottom_right in (False, True):
        p = _sdpa_params(q, k, v, o, 0.3, 7, padding_mask=1, has_right_bound=1, right_bound=1, has_left_bound=1,
                         left_bound=3, bottom_right=int(bottom_right))
        p.stats = p.max = p.sum_exp = tensor(F32, stats.shape)
        p.seq_q = p.seq_kv = tensor(I32, [2, 1, 1, 1])
        oracle.sdpa_forward(p, [q, k, v, o, stats, mx, sm, seq_q, seq_kv, None, None])
        ro, rs, rm, rsum = np_attention(q, k, v, 0.3, seq_q, seq_kv, right_bound=1, left_bound=3, bottom_right=bottom_right)
        _close(o, ro)
        _close(stats[..., 0], rs)
        _close(mx[..., 0], rm)
        _close(sm[..., 0], rsum)
        # padded query rows are written as zeros, fully masked rows give -inf stats
        assert np.all(o[1, :, 3:] == 0.0)
        assert np.all(stats[1, :, 3:, 0] == -INF)


def _paged_case():
    q = np.array([0.2, -0.3, -0.5, 0.4], dtype=np.float32).reshape(2, 1, 1, 2)
    k = np.array([0.6, -0.2, -0.4, 0.9, 0.1, 0.5, -0.3, 0.8, 0.7, -0.6, 0.2, 0.4], dtype=np.float32).reshape(2, 1, 3, 2)
    v = np.array([0.3, -0.7, 0.8, 0.2, -0.6, 0.4, 0.5, -0.1, -0.2, 0.9, 0.6, -0.8], dtype=np.float32).reshape(2, 1, 3, 2)
    page_k = np.array([2, 0, 3, 1], dtype=np.int32)
    page_v = np.array([1, 3, 0, 2], dtype=np.int32)

    def container(logical, table):
        c = np.full((4, 1, 2, 2), -17.0, dtype=np.float32)
        for b in range(2):
            for s in range(3):
                c[table[b * 2 + s // 2], 0, s % 2] = logical[b, 0, s]
        return c

    return q, k, v, page_k, page_v, container(k, page_k), container(v, page_v)


def test_paged_sdpa_equals_contiguous_and_guards_invalid_pages():
    q, k, v, page_k, page_v, kc, vc = _paged_case()
    o = np.full((2, 1, 1, 2), -99.0, dtype=np.float32)
    seq_q = np.array([1, 1], dtype=np.int32)
    seq_kv = np.array([3, 3], dtype=np.int32)
    p = _sdpa_params(q, kc, vc, o, 0.5, 3, padding_mask=1)
    p.seq_q = p.seq_kv = tensor(I32, [2, 1, 1, 1])
    p.page_table_k = p.page_table_v = tensor(I32, [2, 1, 2, 1])
    oracle.sdpa_forward(p, [q, kc, vc, o, None, None, None, seq_q, seq_kv, page_k, page_v])
    reference, _, _, _ = np_attention(q, k, v, 0.5, seq_q, seq_kv)
    _close(o, reference)
    page_k[:2] = [-1, 99]
    page_v[:2] = [-1, 99]
    o[:] = -99.0
    oracle.sdpa_forward(p, [q, kc, vc, o, None, None, None, seq_q, seq_kv, page_k, page_v])
    assert o[0, 0, 0, 0] == 0.0 and o[0, 0, 0, 1] == 0.0


def test_compact_page_tables_equal_contiguous_and_prefix_rule():
    """test/Compiler/SequenceOpsTest.cpp:2031-2147: exact-allocation packed page tables (K offsets INT64 {0,2,3}, V offsets
    INT32 {0,2,3}, sequence lengths {3,1}, two tokens per page) give the contiguous result, and a K segment shorter
    than its sequence demands ({0,1,3}) is rejected with DFE_INVALID_VARIANT_PACK."""
    from deepforge_b200.dfgpu import I64
    q, k, v, _, _, _, _ = _paged_case()
    seq_q = np.array([1, 1], dtype=np.int32)
    seq_kv = np.array([3, 1], dtype=np.int32)
    packed_k, packed_v = np.array([2, 0, 1], dtype=np.int32), np.array([1, 3, 2], dtype=np.int32)
    offsets_k, offsets_v = np.array([0, 2, 3], dtype=np.int64), np.array([0, 2, 3], dtype=np.int32)

    def container(logical, table, offsets):
        c = np.full((4, 1, 2, 2), -17.0, dtype=np.float32)
        for b in range(2):
            for s in range(int(seq_kv[b])):
                c[table[int(offsets[b]) + s // 2], 0, s % 2] = logical[b, 0, s]
        return c

    kc, vc = container(k, packed_k, offsets_k), container(v, packed_v, offsets_v)
    o = np.full((2, 1, 1, 2), -99.0, dtype=np.float32)
    p = _sdpa_params(q, kc, vc, o, 0.5, 3, padding_mask=1)
    p.seq_q = p.seq_kv = tensor(I32, [2, 1, 1, 1])
    p.page_table_k = p.page_table_v = tensor(I32, [2, 1, 2, 1])
    p.page_offsets_k, p.page_offsets_v = tensor(I64, [3, 1, 1, 1]), tensor(I32, [3, 1, 1, 1])
    arrays = [q, kc, vc, o, None, None, None, seq_q, seq_kv, packed_k, packed_v, None, None, None, offsets_k, offsets_v]
    assert oracle.validate_page_prefix(p, arrays, 0) == 0 and oracle.validate_page_prefix(p, arrays, 1) == 0
    oracle.sdpa_forward(p, arrays)
    reference, _, _, _ = np_attention(q, k, v, 0.5, seq_q, seq_kv)
    _close(o, reference)
    for bad in ([0, 1, 3], [1, 2, 3], [0, 3, 2], [0, 2, 5], [0, -1, 3]):  # short segment, non-zero start, decreasing, past the bound (2 x 2), negative
        arrays[14] = np.array(bad, dtype=np.int64)
        assert oracle.validate_page_prefix(p, arrays, 0) == 17, bad
    arrays[14] = offsets_k
    arrays[8] = np.array([5, 1], dtype=np.int32)  # a sequence longer than the table's logical bound
    assert oracle.validate_page_prefix(p, arrays, 0) == 17


def test_static_loop_nest_forms_are_bit_identical_to_the_flat_loops():
    """dfo_conv_generic_nhwc and the vectorisable branch of dfo_matmul run the same chain of f32 operations per output
    element as the literal restatements (c, then taps; k in order; one multiply and one add per step), so their
    results must agree bit for bit, whatever the thread count."""
    from deepforge_b200 import dfgpu
    T = dfgpu.tensor
    rng = np.random.default_rng(5)

    def nhwc(n, c, h, w):
        return T(dfgpu.F32, [n, c, h, w], [h * w * c, 1, w * c, c])

    for n, c, h, w, k, r, pad, stride, dilation, reverse in [(2, 5, 7, 6, 9, 3, 1, 1, 1, False), (1, 4, 9, 9, 3, 3, 2, 2, 1, True), (1, 16, 6, 5, 8, 1, 0, 1, 1, False),
                                                             (1, 3, 11, 8, 4, 3, 2, 1, 2, False)]:
        x = rng.standard_normal(n * c * h * w).astype(np.float32)
        x[::7] *= 1e4
        weights = rng.standard_normal(k * c * r * r).astype(np.float32)
        p = (h + 2 * pad - (dilation * (r - 1) + 1)) // stride + 1
        q = (w + 2 * pad - (dilation * (r - 1) + 1)) // stride + 1
        flat, fast = np.zeros(n * k * p * q, np.float32), np.zeros(n * k * p * q, np.float32)
        attrs = oracle.conv_attrs([pad, pad], [pad, pad], [stride, stride], [dilation, dilation], reverse)
        xd, wd, yd = nhwc(n, c, h, w), T(dfgpu.F32, [k, c, r, r], [r * r * c, 1, r * c, c]), nhwc(n, k, p, q)
        oracle.conv_generic_flat(xd, x, wd, weights, yd, flat, attrs)
        oracle.conv_generic(xd, x, wd, weights, yd, fast, attrs, threads=3)
        assert np.array_equal(flat.view(np.uint32), fast.view(np.uint32))
    m, kk, nn = 37, 200, 130
    a, b = rng.standard_normal(m * kk).astype(np.float32), rng.standard_normal(kk * nn).astype(np.float32)
    fast, flat = np.zeros(m * nn, np.float32), np.zeros(m * nn, np.float32)
    oracle.matmul(T(dfgpu.F32, [m, kk]), a, T(dfgpu.F32, [kk, nn]), b, T(dfgpu.F32, [m, nn]), fast, threads=4)
    transposed = np.ascontiguousarray(b.reshape(kk, nn).T).reshape(-1)  # column-major B takes the flat loop
    oracle.matmul(T(dfgpu.F32, [m, kk]), a, T(dfgpu.F32, [kk, nn], [1, kk]), transposed, T(dfgpu.F32, [m, nn]), flat)
    assert np.array_equal(flat.view(np.uint32), fast.view(np.uint32))


def test_device_side_generator_reproduces_the_host_stream():
    import torch
    from deepforge_b200 import synthetic, workloads
    seed, uid, count = 20261130, 2, 1 << 15
    host = workloads._normal(seed, uid, count, "BFLOAT16")()
    device = synthetic.normal_on_device(torch.device("cpu"), seed, uid, count, chunk=1 << 12).view(torch.uint16).numpy()
    assert np.array_equal(host, device)
    assert np.array_equal(synthetic.normal_on_device(torch.device("cpu"), seed, uid, 1000, bf16=False).numpy(), synthetic.normal(seed, uid, 1000))


# ---- POINTWISE: every mode of the schema -----------------------------------------------

def _oracle_pointwise(mode_name, a, b, t, **scalars):
    import pointwise_reference as reference
    rows, columns = a.shape
    out = np.full((rows, columns), -99.0, np.float32)
    count = dfgpu.pointwise_input_count(mode_name)
    oracle.pointwise_general(dfgpu.PW_MODES[mode_name], tensor(F32, [rows, columns]), a,
                             tensor(F32, [columns]) if count >= 2 else None, b if count >= 2 else None,
                             tensor(F32, [rows, 1]) if count >= 3 else None, t if count >= 3 else None,
                             tensor(F32, [rows, columns]), out,
                             lower=reference.RELU_LOWER, upper=reference.RELU_UPPER, slope=reference.RELU_SLOPE,
                             elu_alpha=reference.ELU_ALPHA, softplus_beta=reference.SOFTPLUS_BETA, swish_beta=reference.SWISH_BETA,
                             axis=1, **scalars)
    return out


@pytest.mark.parametrize("mode_name", dfgpu.PW_MODE_NAMES)
def test_pointwise_modes_match_the_reference_test_oracle(mode_name):
    """test/Compiler/FoundationalMathOpsTest.cpp:440-545,617-640: the reference's inputs, formulas and tolerance."""
    import pointwise_reference as reference
    a, b, t = reference.A.reshape(2, 3).copy(), reference.B.copy(), reference.T.copy()
    out = _oracle_pointwise(mode_name, a, b, t)
    reference.assert_close(mode_name, out, reference.expected(mode_name, a, b, t))


@pytest.mark.parametrize("mode_name", dfgpu.PW_MODE_NAMES)
def test_pointwise_modes_on_seeded_values(mode_name):
    """The same formulas on 64 x 48 seeded values in [-3, 3] (both signs, fractions, exact ties and zeros)."""
    import pointwise_reference as reference
    rng = np.random.default_rng(1234)
    a = np.round(rng.uniform(-3.0, 3.0, (64, 48)) * 8).astype(np.float32) / 8   # multiples of 1/8: ties between A and B exist
    b = np.round(rng.uniform(-3.0, 3.0, 48) * 8).astype(np.float32) / 8
    t = (rng.integers(0, 2, 64) * rng.uniform(-2.0, 2.0, 64)).astype(np.float32)
    a[0, :4] = [0.0, -0.0, 2.5, -2.5]
    b[:4] = [0.0, 1.0, 2.5, 0.0]
    out = _oracle_pointwise(mode_name, a, b, t)
    # f32 rounding of |values| up to e^3 and 3^3 stays far inside the reference's tolerance; POW's poles give infinities
    reference.assert_close(mode_name, out, reference.expected(mode_name, a, b, t))


def test_pointwise_softplus_is_stable_for_large_inputs():
    """test/Compiler/FoundationalMathOpsTest.cpp:169-186 (single_softplus_graph): max(x, 0) + log1p-form, no overflow."""
    x = np.array([1000.0, -1000.0], np.float32)
    out = np.zeros(2, np.float32)
    oracle.pointwise_general(dfgpu.PW_MODES["SOFTPLUS_FWD"], tensor(F32, [2]), x, None, None, None, None, tensor(F32, [2]), out)
    assert out[0] == 1000.0 and out[1] == 0.0
