"""tcgen05 GEMM / implicit-GEMM convolution against the CPU oracle (bf16 storage, f32 accumulate).

Tolerance for bf16 contractions: |d| <= 1e-2 + 2e-2*|ref|. With an f32 output the only
difference from the oracle is accumulation order, so the f32 rule max|d| <= 1e-4*max|ref| holds."""
import numpy as np
import pytest

import gpu_util as g
import oracle
from deepforge_b200 import dfgpu, synthetic
from deepforge_b200.dfgpu import BF16, E4M3, E8M0, F32, tensor
from test_gpu_contractions import check_bf16, check_f32, nhwc_strides, run_conv, step

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _device_healthy():
    yield
    assert dfgpu.device_status() == 0, "a bounded wait expired inside a kernel"


def run_matmul(m, n, k, out_dtype=BF16, b_k_major=False, bias=False, relu=False, seed=4):
    a = synthetic.round_to_bf16(synthetic.normal(seed, 1, m * k))
    b = synthetic.round_to_bf16(synthetic.normal(seed, 2, k * n))
    b_strides = [1, k] if b_k_major else [n, 1]
    ref = np.zeros(m * n, dtype=np.float32)
    cd = tensor(F32, [m, n])
    oracle.matmul(tensor(F32, [m, k]), a, tensor(F32, [k, n], b_strides), b, cd, ref)
    p = dfgpu.MatmulParams()
    p.a, p.b, p.c = tensor(BF16, [m, k]), tensor(BF16, [k, n], b_strides), tensor(out_dtype, [m, n])
    p.kernel = dfgpu.MATMUL_UMMA_BF16
    extra = None
    count = 0
    if bias:
        bv = synthetic.round_to_bf16(synthetic.uniform(seed, 3, n, -1.0, 1.0))
        p.extra[0] = tensor(BF16, [n])
        p.epilogue[count] = step(dfgpu.EPI_ADD, 0)
        count += 1
        extra = g.to_device(synthetic.to_bf16_bits(bv))
        tmp = np.zeros_like(ref)
        oracle.pointwise(dfgpu.PW_ADD, cd, ref, tensor(F32, [n]), bv, cd, tmp)
        ref = tmp
    if relu:
        p.epilogue[count] = step(dfgpu.EPI_RELU)
        count += 1
        tmp = np.zeros_like(ref)
        oracle.pointwise(dfgpu.PW_RELU_FWD, cd, ref, None, None, cd, tmp)
        ref = tmp
    p.epilogue_count = count
    assert dfgpu.query("matmul", p).kernel == dfgpu.MATMUL_UMMA_BF16
    da, db = g.to_device(synthetic.to_bf16_bits(a)), g.to_device(synthetic.to_bf16_bits(b))
    dc = g.device_zeros(m * n * dfgpu.DTYPE_BYTES[out_dtype], 0x7f)
    dfgpu.matmul(p, g.ptr(da), g.ptr(db), g.ptr(dc), extra0=g.ptr(extra))
    if out_dtype == BF16:
        out = synthetic.bf16_bits_to_f32(g.to_host(dc, np.uint16))
    else:
        out = g.to_host(dc, np.float32)
    return out, ref


@pytest.mark.parametrize("m,n,k", [(128, 64, 64), (256, 128, 128), (200, 64, 192), (384, 256, 320), (130, 192, 64)])
@pytest.mark.parametrize("b_k_major", [False, True])
def test_matmul_umma_f32_out(m, n, k, b_k_major):
    out, ref = run_matmul(m, n, k, F32, b_k_major)
    check_f32(out, ref)


def test_matmul_umma_bf16_out_bias_relu():
    out, ref = run_matmul(256, 128, 256, BF16, False, bias=True, relu=True)
    check_bf16(out, ref)


def conv_case(n, c, h, w, k, r, pad, epilogue=(), extras=(), ydtype=BF16, seed=6, one_tile_per_cta=False):
    x_dims, w_dims = [n, c, h, w], [k, c, r, r]
    p_out = h + 2 * pad - r + 1
    q_out = w + 2 * pad - r + 1
    y_dims = [n, k, p_out, q_out]
    return run_conv(BF16, x_dims, w_dims, [pad, pad], [pad, pad], [1, 1], [1, 1], dfgpu.CONV_UMMA_BF16,
                    nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides(y_dims), epilogue=epilogue,
                    extras=extras, seed=seed, reserved=int(one_tile_per_cta))


@pytest.mark.parametrize("n,c,h,w,k,r,pad", [
    (2, 64, 8, 8, 64, 1, 0),      # 1x1, M = 128 exactly
    (1, 128, 7, 9, 64, 1, 0),     # 1x1 with an M tail
    (2, 64, 14, 14, 64, 3, 1),    # 3x3 same, 9 rows per tile, ragged last tile
    (1, 64, 56, 56, 64, 3, 1),    # the bottleneck's 3x3 geometry
    (2, 128, 10, 12, 128, 3, 0),  # no padding, two K slices per tap
    (1, 64, 6, 5, 256, 3, 2),     # wide padding, BN = 256
])
@pytest.mark.parametrize("one_tile_per_cta", [False, True])
def test_conv_umma_matches_oracle(n, c, h, w, k, r, pad, one_tile_per_cta):
    # both forms of the kernel: the persistent one (TMA-store epilogue) and one tile per CTA
    info, out, ref = conv_case(n, c, h, w, k, r, pad, one_tile_per_cta=one_tile_per_cta)
    assert info.kernel == dfgpu.CONV_UMMA_BF16
    check_bf16(out, ref)


@pytest.mark.parametrize("n,c,h,w,k,r,pad", [
    (2, 128, 28, 28, 64, 3, 1),   # two channel blocks per filter row, 4 rows of pitch 30 per tile
    (1, 64, 28, 28, 128, 3, 1),   # 128 output channels in one N tile
    (3, 64, 56, 56, 256, 3, 1),   # two N tiles share each activation tile
])
def test_conv_umma_halo_form(n, c, h, w, k, r, pad):
    """Filters wider than one tap on the persistent kernel: each filter row's input rows are loaded once with
    their padded columns and the three taps read that slot from shifted start rows; GEMM rows that fall on the
    padding columns are computed and dropped."""
    info, out, ref = conv_case(n, c, h, w, k, r, pad, epilogue=[step(dfgpu.EPI_RELU)], seed=12)
    assert info.kernel == dfgpu.CONV_UMMA_BF16
    check_bf16(out, ref)


def test_conv_umma_halo_form_one_by_three_filter():
    n, c, h, w, k = 2, 64, 16, 28, 64
    x_dims, w_dims, y_dims = [n, c, h, w], [k, c, 1, 3], [n, k, h, w]
    info, out, ref = run_conv(BF16, x_dims, w_dims, [0, 1], [0, 1], [1, 1], [1, 1], dfgpu.CONV_UMMA_BF16,
                              nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides(y_dims), seed=13)
    check_bf16(out, ref)


@pytest.mark.parametrize("one_tile_per_cta", [False, True])
@pytest.mark.parametrize("n,c,h,w,k,r,pad", [(2, 64, 12, 12, 256, 1, 0), (3, 64, 16, 16, 64, 3, 1), (40, 64, 28, 28, 128, 1, 0)])
def test_conv_umma_fused_bias_relu_and_residual(n, c, h, w, k, r, pad, one_tile_per_cta):
    bias = synthetic.uniform(3, 5, k, -0.1, 0.1)
    residual = synthetic.normal(3, 6, n * k * h * w)
    y_strides = nhwc_strides([n, k, h, w])
    info, out, ref = conv_case(n, c, h, w, k, r, pad,
                               epilogue=[step(dfgpu.EPI_ADD, 0), step(dfgpu.EPI_RELU), step(dfgpu.EPI_ADD, 1)],
                               extras=[([1, k, 1, 1], [k, 1, k, k], bias), ([n, k, h, w], y_strides, residual)],
                               one_tile_per_cta=one_tile_per_cta)
    assert info.kernel == dfgpu.CONV_UMMA_BF16
    check_bf16(out, ref)


def test_conv_umma_many_tiles_per_cta():
    # 1568 tiles on 148 SMs: every CTA of the persistent kernel walks ~10 tiles through both accumulators
    info, out, ref = conv_case(16, 64, 112, 112, 64, 1, 0, epilogue=[step(dfgpu.EPI_RELU)], seed=9)
    check_bf16(out, ref)


def run_matmul_mxf8(m, n, k, out_dtype=F32, b_k_major=False, bias_relu=False, seed=9, kernel=None):
    """A [m, k] with blocks along K, B [k, n] with blocks along K, quantized by the oracle; the reference is the
    oracle's dequantize + f32 matmul of the same codes and scales."""
    rng = np.random.default_rng(seed)
    # row / column magnitudes spread over many powers of two so that the scale bytes differ from block to block
    a = (synthetic.normal(seed, 1, m * k).reshape(m, k) * np.exp2(rng.integers(-6, 7, size=(m, k // 32)).repeat(32, axis=1))).astype(np.float32).reshape(-1)
    b = (synthetic.normal(seed, 2, k * n).reshape(k, n) * np.exp2(rng.integers(-6, 7, size=(k // 32, n)).repeat(32, axis=0))).astype(np.float32).reshape(-1)
    aq, sa = np.zeros(m * k, dtype=np.uint8), np.zeros(m * k // 32, dtype=np.uint8)
    bq, sb = np.zeros(k * n, dtype=np.uint8), np.zeros(k * n // 32, dtype=np.uint8)
    oracle.block_scale_quantize(tensor(F32, [m, k]), a, tensor(E4M3, [m, k]), aq, tensor(E8M0, [m, k // 32]), sa, 32, 1)
    oracle.block_scale_quantize(tensor(F32, [k, n]), b, tensor(E4M3, [k, n]), bq, tensor(E8M0, [k // 32, n]), sb, 32, 0)
    af, bf = np.zeros(m * k, dtype=np.float32), np.zeros(k * n, dtype=np.float32)
    oracle.block_scale_dequantize(tensor(E4M3, [m, k]), aq, tensor(E8M0, [m, k // 32]), sa, tensor(F32, [m, k]), af, [1, 32])
    oracle.block_scale_dequantize(tensor(E4M3, [k, n]), bq, tensor(E8M0, [k // 32, n]), sb, tensor(F32, [k, n]), bf, [32, 1])
    ref = np.zeros(m * n, dtype=np.float32)
    cd = tensor(F32, [m, n])
    oracle.matmul(tensor(F32, [m, k]), af, tensor(F32, [k, n]), bf, cd, ref)
    p = dfgpu.MatmulParams()
    b_strides = [1, k] if b_k_major else [n, 1]
    p.a, p.b, p.c = tensor(E4M3, [m, k]), tensor(E4M3, [k, n], b_strides), tensor(out_dtype, [m, n])
    p.a_scale, p.b_scale = tensor(E8M0, [m, k // 32]), tensor(E8M0, [k // 32, n])
    p.a_block[0], p.a_block[1], p.b_block[0], p.b_block[1] = 1, 32, 32, 1
    p.kernel = dfgpu.MATMUL_UMMA_MXF8 if kernel is None else kernel
    extra = None
    if bias_relu:
        bv = synthetic.round_to_bf16(synthetic.uniform(seed, 3, n, -1.0, 1.0))
        p.extra[0] = tensor(BF16, [n])
        p.epilogue[0] = step(dfgpu.EPI_ADD, 0)
        p.epilogue[1] = step(dfgpu.EPI_RELU)
        p.epilogue_count = 2
        extra = g.to_device(synthetic.to_bf16_bits(bv))
        tmp = np.zeros_like(ref)
        oracle.pointwise(dfgpu.PW_ADD, cd, ref, tensor(F32, [n]), bv, cd, tmp)
        ref = np.zeros_like(tmp)
        oracle.pointwise(dfgpu.PW_RELU_FWD, cd, tmp, None, None, cd, ref)
    assert dfgpu.query("matmul", p).kernel == p.kernel
    b_codes = np.ascontiguousarray(bq.reshape(k, n).T).reshape(-1) if b_k_major else bq
    d = [g.to_device(v) for v in (aq, b_codes, sa, sb)]
    dc = g.device_zeros(m * n * dfgpu.DTYPE_BYTES[out_dtype], 0x7f)
    dfgpu.matmul(p, g.ptr(d[0]), g.ptr(d[1]), g.ptr(dc), g.ptr(d[2]), g.ptr(d[3]), extra0=g.ptr(extra))
    if out_dtype == BF16:
        return synthetic.bf16_bits_to_f32(g.to_host(dc, np.uint16)), ref
    return g.to_host(dc, np.float32), ref


@pytest.mark.parametrize("b_k_major", [False, True])
@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (128, 256, 256), (256, 384, 512), (384, 512, 1024), (256, 256, 128), (512, 256, 384)])
def test_matmul_mxf8_f32_out(m, n, k, b_k_major):
    """Block-scaled tensor-core matmul on E4M3 codes and E8M0 scales: products and scales are exact, so
    with an f32 output only the order of the f32 additions differs from the oracle. The inputs span 2^-6..2^6
    per block, so sums cancel heavily and the bound is the f32-contraction rule max|d| <= 1e-4 * max|ref|
    (a per-element relative bound is meaningless for outputs that are the small difference of huge terms)."""
    out, ref = run_matmul_mxf8(m, n, k, F32, b_k_major)
    assert np.all(np.isfinite(out))
    assert float(np.max(np.abs(out - ref))) <= 1e-4 * float(np.max(np.abs(ref)))


def test_matmul_mxf8_bf16_out_bias_relu_many_tiles_per_cta():
    """160 tiles of 128 x 256 on 148 SMs: some CTAs run two tiles through the same accumulator."""
    out, ref = run_matmul_mxf8(2560, 2048, 256, BF16, False, bias_relu=True)
    check_bf16(out, ref)
