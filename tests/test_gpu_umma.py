"""tcgen05 GEMM / implicit-GEMM convolution against the CPU oracle (bf16 storage, f32 accumulate).

Tolerance for bf16 contractions: |d| <= 1e-2 + 2e-2*|ref|. With an f32 output the only
difference from the oracle is accumulation order, so the f32 rule max|d| <= 1e-4*max|ref| holds."""
import numpy as np
import pytest

import gpu_util as g
import oracle
from deepforge_b200 import dfgpu, synthetic
from deepforge_b200.dfgpu import BF16, F32, tensor
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
