"""POINTWISE, CONV_FPROP and MATMUL kernels against the CPU oracle, through the C ABI.

Tolerances: f32 graphs max|d| <= 1e-4 * max|ref| (and the reference's own
1e-4 + 1e-3*|ref| per element); bf16 storage |d| <= 1e-2 + 2e-2*|ref|."""
import numpy as np
import pytest

import gpu_util as g
import oracle
from deepforge_b200 import dfgpu, synthetic
from deepforge_b200.dfgpu import BF16, E4M3, E8M0, F32, tensor

pytestmark = pytest.mark.gpu
FLT_MAX = 3.4028234663852886e38


def check_f32(actual, reference):
    scale = max(float(np.max(np.abs(reference))), 1e-30)
    assert float(np.max(np.abs(actual - reference))) <= 1e-4 * scale
    assert np.all(np.abs(actual - reference) <= 1e-4 + 1e-3 * np.abs(reference))


def check_bf16(actual, reference):
    assert np.all(np.abs(actual - reference) <= 1e-2 + 2e-2 * np.abs(reference))


def host_array(values, dtype):
    return synthetic.to_bf16_bits(values) if dtype == BF16 else np.ascontiguousarray(values, dtype=np.float32)


def read_back(buffer, dtype, shape):
    if dtype == BF16:
        return synthetic.bf16_bits_to_f32(g.to_host(buffer, np.uint16)).reshape(shape)
    return g.to_host(buffer, np.float32, shape)


def nhwc_strides(dims):
    n, c, h, w = dims
    return [h * w * c, 1, w * c, c]


def step(op, operand=0, lower=0.0, upper=FLT_MAX, slope=0.0):
    s = dfgpu.EpilogueStep()
    s.op, s.operand, s.relu_lower, s.relu_upper, s.relu_slope = op, operand, lower, upper, slope
    return s


@pytest.mark.parametrize("mode", [dfgpu.PW_ADD, dfgpu.PW_MUL, dfgpu.PW_SUB, dfgpu.PW_RELU_FWD, dfgpu.PW_IDENTITY])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_pointwise_broadcast(mode, dtype):
    shape = [2, 6, 5, 4]
    a = synthetic.normal(1, 1, int(np.prod(shape)))
    a[3] = np.nan
    a[5] = np.inf
    b = synthetic.normal(1, 2, 6)
    ad, bd, od = tensor(dtype, shape), tensor(dtype, [1, 6, 1, 1]), tensor(dtype, shape)
    ha, hb = host_array(a, dtype), host_array(b, dtype)
    width = dfgpu.DTYPE_BYTES[dtype]
    ref = np.zeros(a.size * width, dtype=np.uint8)
    oracle.pointwise(mode, ad, ha, bd, hb, od, ref, 0.25, 1.5, 0.1)
    p = dfgpu.PointwiseParams()
    p.in0, p.in1, p.out, p.mode = ad, bd, od, mode
    p.relu_lower, p.relu_upper, p.relu_slope = 0.25, 1.5, 0.1
    da, db, do = g.to_device(ha), g.to_device(hb), g.device_zeros(ref.size)
    dfgpu.pointwise(p, g.ptr(da), g.ptr(db), g.ptr(do))
    out = g.to_host(do, np.uint8)
    view = np.uint32 if dtype == F32 else np.uint16
    a_bits, r_bits = out.view(view), ref.view(view)
    nan = np.isnan(read_back(do, dtype, shape)).reshape(-1)
    assert np.array_equal(a_bits[~nan], r_bits[~nan])


# modes whose value goes through exp, log, pow, erf, tanh or the trigonometric functions: CUDA's and the host's math
# libraries round those differently (both within a few ulp), everything else is the same bits
LIBM_MODES = {"POW", "EXP", "LOG", "COS", "SIN", "TAN", "ERF", "TANH_FWD", "TANH_BWD", "SIGMOID_FWD", "SIGMOID_BWD", "ELU_FWD",
              "ELU_BWD", "SOFTPLUS_FWD", "SOFTPLUS_BWD", "SWISH_FWD", "SWISH_BWD", "GELU_FWD", "GELU_BWD", "GELU_APPROX_TANH_FWD",
              "GELU_APPROX_TANH_BWD"}


def pointwise_operands(rows, columns):
    rng = np.random.default_rng(99)
    a = (np.round(rng.uniform(-3.0, 3.0, (rows, columns)) * 8) / 8).astype(np.float32)   # multiples of 1/8: A == B happens
    b = (np.round(rng.uniform(-3.0, 3.0, (rows, columns)) * 8) / 8).astype(np.float32)
    t = (rng.integers(0, 2, (rows, columns)) * rng.uniform(-2.0, 2.0, (rows, columns))).astype(np.float32)
    a[0, :8] = [0.0, -0.0, 0.0, -0.0, 2.5, -2.5, np.nan, np.inf]
    b[0, :8] = [0.0, 0.0, -0.0, -0.0, 2.5, 0.0, 1.0, -1.0]
    return a, b, t


@pytest.mark.parametrize("layout", ["packed_f32", "packed_bf16", "packed_f16", "broadcast_f32", "broadcast_f16_to_f32"])
@pytest.mark.parametrize("mode_name", dfgpu.PW_MODE_NAMES)
def test_pointwise_every_mode_against_the_oracle(mode_name, layout):
    """lib/Compiler/FoundationalGraph.cpp:2581-2955: all 50 modes, through both general kernels (four packed values per
    thread; one element per thread with broadcast, strides and mixed storage types) and the five dedicated ones."""
    rows, columns = 24, 40
    a, b, t = pointwise_operands(rows, columns)
    count = dfgpu.pointwise_input_count(mode_name)
    in_type = {"packed_f32": F32, "packed_bf16": BF16, "packed_f16": dfgpu.F16, "broadcast_f32": F32, "broadcast_f16_to_f32": dfgpu.F16}[layout]
    out_type = {"packed_bf16": BF16, "packed_f16": dfgpu.F16}.get(layout, F32)
    if layout.startswith("packed"):
        bd, td = tensor(in_type, [rows, columns]), tensor(in_type, [rows, columns])
    else:   # B along the columns, T down the rows, A with padded rows
        b, t = b[:1].copy(), t[:, :1].copy()
        bd, td = tensor(in_type, [columns]), tensor(in_type, [rows, 1])
    ad = tensor(in_type, [rows, columns]) if layout.startswith("packed") else tensor(in_type, [rows, columns], [columns + 3, 1])
    od = tensor(out_type, [rows, columns])

    def stored(values, descriptor):
        if in_type == BF16:
            bits = synthetic.to_bf16_bits(values)
        elif in_type == dfgpu.F16:
            bits = np.ascontiguousarray(values, dtype=np.float16).view(np.uint16)
        else:
            bits = np.ascontiguousarray(values, dtype=np.float32)
        if descriptor.rank == 2 and int(descriptor.stride[0]) != int(descriptor.dim[1]):
            padded = np.zeros((rows, int(descriptor.stride[0])), bits.dtype)
            padded[:, :columns] = bits.reshape(rows, columns)
            return np.ascontiguousarray(padded)
        return np.ascontiguousarray(bits)
    ha, hb, ht = stored(a, ad), stored(b, bd), stored(t, td)
    width = dfgpu.DTYPE_BYTES[out_type]
    ref = np.zeros(rows * columns * width, dtype=np.uint8)
    scalars = dict(lower=-0.5, upper=1.25, slope=0.125, elu_alpha=1.5, softplus_beta=0.75, swish_beta=1.75, axis=1)
    oracle.pointwise_general(dfgpu.PW_MODES[mode_name], ad, ha, bd if count >= 2 else None, hb if count >= 2 else None,
                             td if count >= 3 else None, ht if count >= 3 else None, od, ref, **scalars)
    p = dfgpu.PointwiseParams()
    p.in0, p.out, p.mode = ad, od, dfgpu.PW_MODES[mode_name]
    if count >= 2:
        p.in1 = bd
    if count >= 3:
        p.in2 = td
    p.relu_lower, p.relu_upper, p.relu_slope = scalars["lower"], scalars["upper"], scalars["slope"]
    p.elu_alpha, p.softplus_beta, p.swish_beta, p.axis = scalars["elu_alpha"], scalars["softplus_beta"], scalars["swish_beta"], 1
    da, db, dt, do = g.to_device(ha), g.to_device(hb), g.to_device(ht), g.device_zeros(ref.size)
    dfgpu.pointwise(p, g.ptr(da), g.ptr(db) if count >= 2 else 0, g.ptr(do), in2=g.ptr(dt) if count >= 3 else 0)
    out = g.to_host(do, np.uint8)
    if out_type == F32:
        got, want = out.view(np.float32), ref.view(np.float32)
    elif out_type == dfgpu.F16:
        got, want = out.view(np.float16).astype(np.float32), ref.view(np.float16).astype(np.float32)
    else:
        got, want = synthetic.bf16_bits_to_f32(out.view(np.uint16)), synthetic.bf16_bits_to_f32(ref.view(np.uint16))
    assert np.array_equal(np.isnan(got), np.isnan(want))
    finite = ~np.isnan(want)
    if mode_name in LIBM_MODES:
        infinite = np.isinf(want)
        assert np.array_equal(got[infinite], want[infinite])
        ok = finite & ~infinite
        if out_type == F32:
            assert np.all(np.abs(got[ok] - want[ok]) <= 2e-6 + 2e-6 * np.abs(want[ok])), float(np.max(np.abs(got[ok] - want[ok])))
        else:   # one bf16 (f16) step where the f32 values straddle a rounding boundary
            step = 2.0 ** -7 if out_type == BF16 else 2.0 ** -10
            assert np.all(np.abs(got[ok] - want[ok]) <= step * np.abs(want[ok]) + (1e-30 if out_type == BF16 else 2.0 ** -24))
    else:
        view = np.uint32 if out_type == F32 else np.uint16
        assert np.array_equal(out.view(view)[finite], ref.view(view)[finite])


def test_relu_default_clips_inf_to_flt_max_and_keeps_nan():
    x = np.array([-1.0, 0.5, np.inf, np.nan, -np.inf], dtype=np.float32)
    d = tensor(F32, [5])
    p = dfgpu.PointwiseParams()
    p.in0, p.out, p.mode, p.relu_lower, p.relu_upper, p.relu_slope = d, d, dfgpu.PW_RELU_FWD, 0.0, FLT_MAX, 0.0
    dx, do = g.to_device(x), g.device_zeros(20)
    dfgpu.pointwise(p, g.ptr(dx), 0, g.ptr(do))
    out = g.to_host(do, np.float32)
    # -inf takes the lower branch: 0 + 0 * (-inf - 0) = NaN, exactly as the reference's formula gives
    assert out[0] == 0.0 and out[1] == 0.5 and out[2] == np.float32(FLT_MAX) and np.isnan(out[3]) and np.isnan(out[4])


def run_conv(dtype, x_dims, w_dims, pre, post, stride, dilation, kernel, x_strides=None, w_strides=None, y_strides=None,
             reverse=False, epilogue=(), extras=(), seed=1, reserved=0):
    n, c, h, w = x_dims
    k, cg, r, s = w_dims
    oh = (h + pre[0] + post[0] - (dilation[0] * (r - 1) + 1)) // stride[0] + 1
    ow = (w + pre[1] + post[1] - (dilation[1] * (s - 1) + 1)) // stride[1] + 1
    y_dims = [n, k, oh, ow]
    xd, wd, yd = tensor(dtype, x_dims, x_strides), tensor(dtype, w_dims, w_strides), tensor(dtype, y_dims, y_strides)
    x = synthetic.normal(seed, 1, int(np.prod(x_dims)))
    wv = synthetic.normal(seed, 2, int(np.prod(w_dims)), std=(2.0 / (cg * r * s)) ** 0.5)
    hx, hw = host_array(x, dtype), host_array(wv, dtype)
    # oracle: f32 restatement on the (possibly bf16-rounded) values
    fx = synthetic.round_to_bf16(x) if dtype == BF16 else x
    fw = synthetic.round_to_bf16(wv) if dtype == BF16 else wv
    fxd, fwd, fyd = tensor(F32, x_dims, x_strides), tensor(F32, w_dims, w_strides), tensor(F32, y_dims, y_strides)
    ref = np.zeros(int(np.prod(y_dims)), dtype=np.float32)
    oracle.conv_generic(fxd, fx, fwd, fw, fyd, ref, oracle.conv_attrs(pre, post, stride, dilation, reverse))
    p = dfgpu.ConvParams()
    p.x, p.w, p.y = xd, wd, yd
    for i in range(2):
        p.pre_pad[i], p.post_pad[i], p.stride[i], p.dilation[i] = pre[i], post[i], stride[i], dilation[i]
    p.reverse_filter, p.kernel = int(reverse), kernel
    p.reserved = reserved
    extra_dev = [None, None]
    for i, (dims, strides, values) in enumerate(extras):
        p.extra[i] = tensor(dtype, dims, strides)
        extra_dev[i] = g.to_device(host_array(values, dtype))
    p.epilogue_count = len(epilogue)
    for i, e in enumerate(epilogue):
        p.epilogue[i] = e
        tmp = np.zeros_like(ref)
        if e.op == dfgpu.EPI_ADD:
            dims, strides, values = extras[e.operand]
            ev = synthetic.round_to_bf16(values) if dtype == BF16 else values
            oracle.pointwise(dfgpu.PW_ADD, fyd, ref, tensor(F32, dims, strides), np.ascontiguousarray(ev, dtype=np.float32), fyd, tmp)
        else:
            oracle.pointwise(dfgpu.PW_RELU_FWD, fyd, ref, None, None, fyd, tmp, e.relu_lower, e.relu_upper, e.relu_slope)
        ref = tmp
    dx, dw = g.to_device(hx), g.to_device(hw)
    dy = g.device_zeros(ref.size * dfgpu.DTYPE_BYTES[dtype])
    info = dfgpu.query("conv_fprop", p)
    scratch = g.device_zeros(info.scratch_bytes, 0xA5) if info.scratch_bytes else None
    dfgpu.conv_fprop(p, g.ptr(dx), g.ptr(dw), g.ptr(dy), g.ptr(extra_dev[0]), g.ptr(extra_dev[1]), scratch=g.ptr(scratch))
    out = read_back(dy, dtype, -1)
    return info, out, ref


@pytest.mark.parametrize("kernel", [dfgpu.CONV_DIRECT, dfgpu.CONV_IGEMM_FFMA])
@pytest.mark.parametrize("c,k,h,w", [(1, 1, 5, 5), (7, 8, 6, 9), (17, 33, 29, 30), (64, 64, 14, 14), (31, 15, 8, 8)])
def test_conv_f32_nhwc_tails(kernel, c, k, h, w):
    x_dims, w_dims = [2, c, h, w], [k, c, 3, 3]
    info, out, ref = run_conv(F32, x_dims, w_dims, [1, 1], [1, 1], [1, 1], [1, 1], kernel,
                              nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides([2, k, h, w]))
    assert info.kernel == kernel
    check_f32(out, ref)


@pytest.mark.parametrize("kernel", [dfgpu.CONV_DIRECT, dfgpu.CONV_IGEMM_FFMA])
def test_conv_f32_nchw_asymmetric_strided_dilated(kernel):
    info, out, ref = run_conv(F32, [2, 6, 11, 9], [10, 6, 3, 2], [1, 0], [2, 1], [2, 1], [1, 2], kernel, reverse=True)
    check_f32(out, ref)


def test_conv_grouped_direct():
    info, out, ref = run_conv(F32, [2, 8, 9, 8], [6, 4, 3, 2], [1, 2], [2, 0], [2, 1], [1, 2], dfgpu.CONV_AUTO)
    assert info.kernel == dfgpu.CONV_DIRECT
    check_f32(out, ref)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_conv_fused_bias_relu_residual(dtype):
    x_dims, w_dims = [2, 16, 7, 7], [16, 16, 3, 3]
    bias = synthetic.uniform(3, 5, 16, -0.1, 0.1)
    residual = synthetic.normal(3, 6, 2 * 16 * 7 * 7)
    y_strides = nhwc_strides([2, 16, 7, 7])
    info, out, ref = run_conv(dtype, x_dims, w_dims, [1, 1], [1, 1], [1, 1], [1, 1], dfgpu.CONV_IGEMM_FFMA,
                              nhwc_strides(x_dims), nhwc_strides(w_dims), y_strides,
                              epilogue=[step(dfgpu.EPI_ADD, 0), step(dfgpu.EPI_RELU), step(dfgpu.EPI_ADD, 1)],
                              extras=[([1, 16, 1, 1], [16, 1, 16, 16], bias), ([2, 16, 7, 7], y_strides, residual)])
    (check_f32 if dtype == F32 else check_bf16)(out, ref)


def test_conv_benchmark_shape_c1_both_layouts():
    """1x64x56x56 (*) 64x64x3x3, pad 1: the reference's 'large' profile (NHWC) and the NCHW-strided form."""
    x_dims, w_dims, y_dims = [1, 64, 56, 56], [64, 64, 3, 3], [1, 64, 56, 56]
    info, out, ref = run_conv(F32, x_dims, w_dims, [1, 1], [1, 1], [1, 1], [1, 1], dfgpu.CONV_AUTO,
                              nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides(y_dims), seed=20261126)
    check_f32(out, ref)
    info, out, ref = run_conv(F32, x_dims, w_dims, [1, 1], [1, 1], [1, 1], [1, 1], dfgpu.CONV_AUTO, seed=20261126)
    assert info.kernel == dfgpu.CONV_UMMA_F32X3_CLUSTER  # (the same one-launch tcgen05 kernel, reading and writing NCHW value by value)
    check_f32(out, ref)
    # mixed: channels-last X, NCHW filter and output
    info, out, ref = run_conv(F32, x_dims, w_dims, [1, 1], [1, 1], [1, 1], [1, 1], dfgpu.CONV_AUTO, nhwc_strides(x_dims), seed=20261126)
    assert info.kernel == dfgpu.CONV_UMMA_F32X3_CLUSTER
    check_f32(out, ref)


def test_conv_benchmark_shape_c1_in_one_launch_on_tensor_cores():
    """The benchmark convolution has 25 output tiles for 148 SMs: AUTO resolves it to the one-launch tcgen05 form (a thread-block cluster per
    tile, the filter taps shared out between its CTAs, no scratch), which holds the f32 gates against the oracle and agrees with the CUDA-core
    kernel far inside them. So do the shapes below, by id: one unit per CTA, several units per CTA (the operand buffers are reused), two
    channel chunks per tap, two tiles along K, a ragged last tile, images that end inside a tile, no padding, and bias + ReLU."""
    x_dims, w_dims, y_dims = [1, 64, 56, 56], [64, 64, 3, 3], [1, 64, 56, 56]
    info, out, ref = run_conv(F32, x_dims, w_dims, [1, 1], [1, 1], [1, 1], [1, 1], dfgpu.CONV_AUTO,
                              nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides(y_dims), seed=20261126)
    assert info.kernel == dfgpu.CONV_UMMA_F32X3_CLUSTER and info.launches == 1 and info.scratch_bytes == 0
    check_f32(out, ref)
    info2, out2, _ = run_conv(F32, x_dims, w_dims, [1, 1], [1, 1], [1, 1], [1, 1], dfgpu.CONV_IGEMM_FFMA,
                              nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides(y_dims), seed=20261126)
    assert float(np.max(np.abs(out - out2))) <= 3e-5 * float(np.max(np.abs(ref)))
    cases = (([3, 128, 14, 14], [64, 128, 1, 1], 0), ([2, 64, 28, 28], [128, 64, 3, 3], 1), ([1, 64, 9, 20], [64, 64, 5, 5], 2),
             ([4, 64, 40, 40], [64, 64, 3, 3], 1), ([2, 192, 11, 13], [64, 192, 3, 3], 0), ([5, 64, 7, 7], [256, 64, 1, 1], 0),
             # channel counts that do not fill a 64-channel unit or a 64-channel tile (C a multiple of 8, K of 4): zero-filled
             ([1, 32, 32, 32], [32, 32, 3, 3], 1), ([2, 72, 9, 9], [20, 72, 3, 3], 1), ([1, 8, 10, 10], [4, 8, 5, 5], 2), ([3, 136, 6, 5], [132, 136, 1, 1], 0),
             # more tiles than SMs: one CTA per tile walks all nine taps, the tiles run in waves; and a single output pixel
             ([8, 64, 56, 56], [64, 64, 3, 3], 1), ([1, 8, 1, 1], [4, 8, 1, 1], 0),
             # channel counts that are no multiple of 8 or 4 (the last group of a unit is read value by value and zero-filled)
             ([2, 17, 29, 30], [33, 17, 3, 3], 1), ([1, 31, 8, 8], [15, 31, 3, 3], 1), ([2, 7, 6, 9], [8, 7, 3, 3], 1))
    for x_dims, w_dims, pad in cases:
        n, c, h, w = x_dims
        k, _, r, s_ = w_dims
        y_dims = [n, k, h + 2 * pad - r + 1, w + 2 * pad - s_ + 1]
        bias = synthetic.uniform(3, 5, k, -0.1, 0.1)
        info, out, ref = run_conv(F32, x_dims, w_dims, [pad, pad], [pad, pad], [1, 1], [1, 1], dfgpu.CONV_UMMA_F32X3_CLUSTER,
                                  nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides(y_dims), seed=5,
                                  epilogue=[step(dfgpu.EPI_ADD, 0), step(dfgpu.EPI_RELU)], extras=[([1, k, 1, 1], [k, 1, k, k], bias)])
        assert info.kernel == dfgpu.CONV_UMMA_F32X3_CLUSTER and info.launches == 1
        check_f32(out, ref)
    # stride, dilation, asymmetric padding and a reversed filter only change which pixel and which tap a loader thread reads
    for x_dims, w_dims, pre, post, stride, dilation, reverse in (([2, 64, 28, 28], [64, 64, 3, 3], [1, 1], [1, 1], [2, 2], [1, 1], False),
                                                                   ([1, 64, 20, 17], [64, 64, 3, 3], [2, 2], [2, 2], [1, 1], [2, 2], False),
                                                                   ([2, 32, 11, 9], [16, 32, 3, 2], [1, 0], [2, 1], [2, 1], [1, 2], True),
                                                                   ([1, 64, 14, 14], [64, 64, 3, 3], [1, 1], [1, 1], [1, 1], [1, 1], True)):
        kernels = {}
        out_h = (x_dims[2] + pre[0] + post[0] - (dilation[0] * (w_dims[2] - 1) + 1)) // stride[0] + 1
        out_w = (x_dims[3] + pre[1] + post[1] - (dilation[1] * (w_dims[3] - 1) + 1)) // stride[1] + 1
        for kernel in (dfgpu.CONV_UMMA_F32X3_CLUSTER, dfgpu.CONV_AUTO):
            info, out, ref = run_conv(F32, x_dims, w_dims, pre, post, stride, dilation, kernel, nhwc_strides(x_dims), nhwc_strides(w_dims),
                                      nhwc_strides([x_dims[0], w_dims[0], out_h, out_w]), reverse=reverse, seed=11)
            kernels[kernel] = info.kernel
            check_f32(out, ref)
        assert kernels[dfgpu.CONV_UMMA_F32X3_CLUSTER] == kernels[dfgpu.CONV_AUTO] == dfgpu.CONV_UMMA_F32X3_CLUSTER
    assert dfgpu.device_status() == 0


@pytest.mark.parametrize("dtype", [BF16, F32])
def test_one_launch_form_for_convolutions_the_bf16_kernel_does_not_take(dtype):
    """A stride-2 3 x 3 convolution, a dilated one and one with 24 -> 20 channels: AUTO resolves them to the one-launch tcgen05 kernel for
    bf16 storage as for f32 (read value by value and widened), with bias + ReLU; a stride-1 64-channel bf16 convolution stays with the bf16
    tcgen05 kernel."""
    for x_dims, w_dims, pad, stride, dilation in (([2, 64, 28, 28], [64, 64, 3, 3], 1, 2, 1), ([1, 64, 20, 17], [128, 64, 3, 3], 2, 1, 2),
                                                  ([3, 24, 12, 12], [20, 24, 3, 3], 1, 1, 1)):
        n, c, h, w = x_dims
        k = w_dims[0]
        out_h = (h + 2 * pad - (dilation * 2 + 1)) // stride + 1
        out_w = (w + 2 * pad - (dilation * 2 + 1)) // stride + 1
        bias = synthetic.uniform(3, 5, k, -0.1, 0.1)
        info, out, ref = run_conv(dtype, x_dims, w_dims, [pad, pad], [pad, pad], [stride, stride], [dilation, dilation], dfgpu.CONV_AUTO,
                                  nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides([n, k, out_h, out_w]), seed=13,
                                  epilogue=[step(dfgpu.EPI_ADD, 0), step(dfgpu.EPI_RELU)], extras=[([1, k, 1, 1], [k, 1, k, k], bias)])
        assert info.kernel == dfgpu.CONV_UMMA_F32X3_CLUSTER and info.launches == 1 and info.scratch_bytes == 0
        (check_f32 if dtype == F32 else check_bf16)(out, ref)
    if dtype == BF16:
        x_dims, w_dims = [2, 64, 14, 14], [64, 64, 3, 3]
        info, out, ref = run_conv(BF16, x_dims, w_dims, [1, 1], [1, 1], [1, 1], [1, 1], dfgpu.CONV_AUTO,
                                  nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides([2, 64, 14, 14]))
        assert info.kernel == dfgpu.CONV_UMMA_BF16
        check_bf16(out, ref)
    assert dfgpu.device_status() == 0


def test_matmul_bf16_odd_shape_in_one_launch_on_tensor_cores():
    """A bf16 product the bf16 tcgen05 matmul does not take (M = 100, K = 136, N = 68) runs on the one-launch kernel."""
    out, ref = run_matmul(BF16, [100, 136], [136, 68], kernel=dfgpu.MATMUL_AUTO)
    check_bf16(out, ref)
    p = dfgpu.MatmulParams()
    p.a, p.b, p.c = tensor(BF16, [100, 136]), tensor(BF16, [136, 68]), tensor(BF16, [100, 68])
    assert dfgpu.query("matmul", p).kernel == dfgpu.MATMUL_UMMA_F32X3_CLUSTER
    assert dfgpu.device_status() == 0


def test_one_launch_forms_take_pointers_of_any_alignment():
    """f32 arguments keep the reference's 4-byte alignment: with X (or A) 4 bytes off a 16-byte boundary the one-launch kernel reads that
    operand value by value instead of as float4s; the result agrees with the CUDA-core kernel's far inside the gate."""
    x_dims, w_dims, y_dims = [1, 64, 12, 12], [64, 64, 3, 3], [1, 64, 12, 12]
    x = synthetic.normal(9, 1, int(np.prod(x_dims))).astype(np.float32)
    w = synthetic.normal(9, 2, int(np.prod(w_dims)), std=0.05).astype(np.float32)
    p = dfgpu.ConvParams()
    p.x, p.w, p.y = tensor(F32, x_dims, nhwc_strides(x_dims)), tensor(F32, w_dims, nhwc_strides(w_dims)), tensor(F32, y_dims, nhwc_strides(y_dims))
    for i in range(2):
        p.pre_pad[i], p.post_pad[i], p.stride[i], p.dilation[i] = 1, 1, 1, 1
    shifted = g.to_device(np.concatenate([np.zeros(1, np.float32), x]))
    dw = g.to_device(w)
    results = {}
    for kernel in (dfgpu.CONV_IGEMM_FFMA, dfgpu.CONV_UMMA_F32X3_CLUSTER):
        p.kernel = kernel
        dy = g.device_zeros(int(np.prod(y_dims)) * 4, 0x5A)
        dfgpu.conv_fprop(p, g.ptr(shifted) + 4, g.ptr(dw), g.ptr(dy))
        results[kernel] = g.to_host(dy, np.float32).copy()
    assert float(np.max(np.abs(results[dfgpu.CONV_IGEMM_FFMA] - results[dfgpu.CONV_UMMA_F32X3_CLUSTER]))) <= 3e-5 * float(np.max(np.abs(results[dfgpu.CONV_IGEMM_FFMA])))
    assert not np.array_equal(results[dfgpu.CONV_IGEMM_FFMA], results[dfgpu.CONV_UMMA_F32X3_CLUSTER])
    a = synthetic.normal(4, 1, 128 * 128).astype(np.float32)
    b = synthetic.normal(4, 2, 128 * 64).astype(np.float32)
    q = dfgpu.MatmulParams()
    q.a, q.b, q.c = tensor(F32, [128, 128]), tensor(F32, [128, 64]), tensor(F32, [128, 64])
    da, db = g.to_device(np.concatenate([np.zeros(1, np.float32), a])), g.to_device(b)
    for kernel in (dfgpu.MATMUL_FFMA, dfgpu.MATMUL_UMMA_F32X3_CLUSTER):
        q.kernel = kernel
        dc = g.device_zeros(128 * 64 * 4, 0x5A)
        dfgpu.matmul(q, g.ptr(da) + 4, g.ptr(db), g.ptr(dc))
        results[kernel] = g.to_host(dc, np.float32).copy()
    assert float(np.max(np.abs(results[dfgpu.MATMUL_FFMA] - results[dfgpu.MATMUL_UMMA_F32X3_CLUSTER]))) <= 2e-5 * float(np.max(np.abs(results[dfgpu.MATMUL_FFMA])))
    assert not np.array_equal(results[dfgpu.MATMUL_FFMA], results[dfgpu.MATMUL_UMMA_F32X3_CLUSTER])
    assert dfgpu.device_status() == 0


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_grouped_convolutions_in_one_launch_on_tensor_cores(dtype):
    """Groups: every 64-channel output tile belongs to one group and reads that group's input channels only (2 groups of 32 -> 32
    channels; 4 groups of 16 -> 24, so a group's last tile and unit are partly empty; 2 groups of 80 -> 72 with stride 2)."""
    for x_dims, w_dims, stride in (([2, 64, 12, 12], [64, 32, 3, 3], 1), ([1, 64, 9, 9], [96, 16, 3, 3], 1), ([2, 160, 15, 13], [144, 80, 3, 3], 2)):
        n, c, h, w = x_dims
        k = w_dims[0]
        out_h, out_w = (h + 2 - 3) // stride + 1, (w + 2 - 3) // stride + 1
        info, out, ref = run_conv(dtype, x_dims, w_dims, [1, 1], [1, 1], [stride, stride], [1, 1], dfgpu.CONV_AUTO,
                                  nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides([n, k, out_h, out_w]), seed=17)
        assert info.kernel == dfgpu.CONV_UMMA_F32X3_CLUSTER and info.launches == 1
        (check_f32 if dtype == F32 else check_bf16)(out, ref)
    assert dfgpu.device_status() == 0


def test_conv_one_launch_form_limits():
    """A reduction of more than 64 units per CTA (here 144 with one CTA per tile) is refused by id, and AUTO then takes another kernel."""
    for x_dims, w_dims, stride in (([32, 1024, 56, 56], [64, 1024, 3, 3], 1),):
        p = dfgpu.ConvParams()
        n, c, h, w = x_dims
        y_dims = [n, w_dims[0], (h + 2 - 3) // stride + 1, (w + 2 - 3) // stride + 1]
        p.x, p.w, p.y = tensor(F32, x_dims, nhwc_strides(x_dims)), tensor(F32, w_dims, nhwc_strides(w_dims)), tensor(F32, y_dims, nhwc_strides(y_dims))
        for i in range(2):
            p.pre_pad[i], p.post_pad[i], p.stride[i], p.dilation[i] = 1, 1, stride, 1
        p.kernel = dfgpu.CONV_UMMA_F32X3_CLUSTER
        with pytest.raises(dfgpu.DfgpuError) as error:
            dfgpu.query("conv_fprop", p)
        assert "one-launch tcgen05 form" in str(error.value)
        p.kernel = dfgpu.CONV_AUTO
        assert dfgpu.query("conv_fprop", p).kernel != dfgpu.CONV_UMMA_F32X3_CLUSTER


@pytest.mark.parametrize("where", ["x_inf", "x_nan", "w_inf", "x_huge", "clean"])
def test_conv_one_launch_form_with_non_finite_operands(where):
    """A cluster whose inputs hold an infinity or a NaN computes its tile on the CUDA cores: those tiles are bit for bit the CUDA-core kernel's
    own (NaNs in the same places, zero padding multiplied), the others stay on the tensor cores. Finite values up to the largest f32 stay on
    the tensor cores everywhere (the pieces are cut off, not rounded, so none rounds past the largest bf16)."""
    x_dims, w_dims, y_dims = [1, 64, 12, 12], [64, 64, 3, 3], [1, 64, 12, 12]
    x = synthetic.normal(9, 1, int(np.prod(x_dims)))
    w = synthetic.normal(9, 2, int(np.prod(w_dims)), std=0.05)
    w[::7] = np.float32(0.5)          # lower pieces of exactly zero
    if where == "x_inf": x[5 * 64 + 3] = np.inf        # pixel 5: inside the first tile's windows only
    if where == "x_nan": x[140 * 64 + 9] = np.nan      # pixel 140: seen by both tiles (rows 10..11 of the image)
    if where == "w_inf": w[1000] = -np.inf
    if where == "x_huge": x[40 * 64 + 1], w[:] = np.float32(3.395e38), np.float32(2.0 ** -20)
    p = dfgpu.ConvParams()
    p.x, p.w, p.y = tensor(F32, x_dims, nhwc_strides(x_dims)), tensor(F32, w_dims, nhwc_strides(w_dims)), tensor(F32, y_dims, nhwc_strides(y_dims))
    for i in range(2):
        p.pre_pad[i], p.post_pad[i], p.stride[i], p.dilation[i] = 1, 1, 1, 1
    dx, dw = g.to_device(x.astype(np.float32)), g.to_device(w.astype(np.float32))
    results = {}
    for kernel in (dfgpu.CONV_IGEMM_FFMA, dfgpu.CONV_UMMA_F32X3_CLUSTER):
        p.kernel = kernel
        dy = g.device_zeros(int(np.prod(y_dims)) * 4, 0x5A)
        dfgpu.conv_fprop(p, g.ptr(dx), g.ptr(dw), g.ptr(dy))
        results[kernel] = g.to_host(dy, np.uint32).copy().reshape(144, 64)
    cores, cluster = results[dfgpu.CONV_IGEMM_FFMA], results[dfgpu.CONV_UMMA_F32X3_CLUSTER]
    a, b = cluster.view(np.float32), cores.view(np.float32)
    exact_tiles = {"x_inf": [0], "x_nan": [0, 1], "w_inf": [0, 1], "x_huge": [], "clean": []}[where]
    for tile in range(2):
        rows = slice(tile * 128, min(144, tile * 128 + 128))
        if tile in exact_tiles:
            assert np.array_equal(cores[rows], cluster[rows])
        else:
            assert np.all(np.isfinite(a[rows])) and not np.array_equal(cores[rows], cluster[rows])  # (the tensor-core result stands)
            assert float(np.max(np.abs(a[rows] - b[rows]))) <= 3e-5 * float(np.max(np.abs(b[np.isfinite(b)])))
    if exact_tiles:
        assert not np.all(np.isfinite(b))
    assert dfgpu.device_status() == 0


def test_conv_split_form_runs_on_tensor_cores():
    """The three-launch split-operand tcgen05 form (six bf16 products of three-piece operands, f32 accumulation), which AUTO takes for f32
    convolutions of more tiles than SMs: it holds the f32 gates against the oracle on the benchmark convolution, a 1x1 filter, a deeper one
    with bias and ReLU, and a batch of images."""
    x_dims, w_dims, y_dims = [1, 64, 56, 56], [64, 64, 3, 3], [1, 64, 56, 56]
    info, out, ref = run_conv(F32, x_dims, w_dims, [1, 1], [1, 1], [1, 1], [1, 1], dfgpu.CONV_UMMA_F32X3,
                              nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides(y_dims), seed=20261126)
    assert info.kernel == dfgpu.CONV_UMMA_F32X3 and info.launches == 3 and info.scratch_bytes > 0
    check_f32(out, ref)
    # the CUDA-core kernel on the same inputs: the two agree far inside the gate
    info2, out2, _ = run_conv(F32, x_dims, w_dims, [1, 1], [1, 1], [1, 1], [1, 1], dfgpu.CONV_IGEMM_FFMA,
                              nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides(y_dims), seed=20261126)
    assert info2.kernel == dfgpu.CONV_IGEMM_FFMA
    assert float(np.max(np.abs(out - out2))) <= 3e-5 * float(np.max(np.abs(ref)))
    for x_dims, w_dims, pad in (([3, 128, 14, 14], [64, 128, 1, 1], 0), ([2, 64, 28, 28], [128, 64, 3, 3], 1), ([1, 64, 9, 20], [64, 64, 5, 5], 2)):
        n, c, h, w = x_dims
        y_dims = [n, w_dims[0], h, w]
        bias = synthetic.uniform(3, 5, w_dims[0], -0.1, 0.1)
        # (asked for by id: AUTO keeps convolutions below 2^24 multiply-adds on CUDA cores, where one launch beats three)
        info, out, ref = run_conv(F32, x_dims, w_dims, [pad, pad], [pad, pad], [1, 1], [1, 1], dfgpu.CONV_UMMA_F32X3,
                                  nhwc_strides(x_dims), nhwc_strides(w_dims), nhwc_strides(y_dims), seed=5,
                                  epilogue=[step(dfgpu.EPI_ADD, 0), step(dfgpu.EPI_RELU)], extras=[([1, w_dims[0], 1, 1], [w_dims[0], 1, w_dims[0], w_dims[0]], bias)])
        assert info.kernel == dfgpu.CONV_UMMA_F32X3
        check_f32(out, ref)


@pytest.mark.parametrize("where", ["x_inf", "x_nan", "w_inf", "x_huge", "clean"])
def test_conv_split_form_with_non_finite_operands(where):
    """An infinity or a NaN in X or W does not survive the split into bf16 pieces (inf * 0), so the CUDA-core kernel behind the
    tensor-core one redoes the convolution: the result is then bit for bit the CUDA-core kernel's own (NaNs in the same
    places). Finite values past the largest bf16 stay on the tensor cores."""
    x_dims, w_dims, y_dims = [1, 64, 12, 12], [64, 64, 3, 3], [1, 64, 12, 12]
    x = synthetic.normal(9, 1, int(np.prod(x_dims)))
    w = synthetic.normal(9, 2, int(np.prod(w_dims)), std=0.05)
    w[::7] = np.float32(0.5)          # lower pieces of exactly zero
    if where == "x_inf": x[5 * 64 + 3] = np.inf
    if where == "x_nan": x[77 * 64 + 9] = np.nan
    if where == "w_inf": w[1000] = -np.inf
    if where == "x_huge": x[40 * 64 + 1], w[:] = np.float32(3.395e38), np.float32(2.0 ** -20)
    p = dfgpu.ConvParams()
    p.x, p.w, p.y = tensor(F32, x_dims, nhwc_strides(x_dims)), tensor(F32, w_dims, nhwc_strides(w_dims)), tensor(F32, y_dims, nhwc_strides(y_dims))
    for i in range(2):
        p.pre_pad[i], p.post_pad[i], p.stride[i], p.dilation[i] = 1, 1, 1, 1
    dx, dw = g.to_device(x.astype(np.float32)), g.to_device(w.astype(np.float32))
    results = {}
    for kernel in (dfgpu.CONV_IGEMM_FFMA, dfgpu.CONV_UMMA_F32X3):
        p.kernel = kernel
        info = dfgpu.query("conv_fprop", p)
        dy = g.device_zeros(int(np.prod(y_dims)) * 4, 0x5A)
        scratch = g.device_zeros(info.scratch_bytes, 0xA5) if info.scratch_bytes else None
        dfgpu.conv_fprop(p, g.ptr(dx), g.ptr(dw), g.ptr(dy), scratch=g.ptr(scratch))
        results[kernel] = g.to_host(dy, np.uint32).copy()
    cores, split = results[dfgpu.CONV_IGEMM_FFMA], results[dfgpu.CONV_UMMA_F32X3]
    if where in ("x_inf", "x_nan", "w_inf"):
        assert np.array_equal(cores, split)
        assert not np.all(np.isfinite(cores.view(np.float32)))
    else:
        a, b = split.view(np.float32), cores.view(np.float32)
        assert np.all(np.isfinite(a)) and not np.array_equal(cores, split)  # (the tensor-core result stands)
        assert float(np.max(np.abs(a - b))) <= 3e-5 * float(np.max(np.abs(b)))


def test_conv_special_values_single_node_rule():
    # zero -> 0, NaN -> NaN, +Inf -> +Inf
    xd = tensor(F32, [1, 1, 3, 3])
    p = dfgpu.ConvParams()
    p.x, p.w, p.y = xd, xd, xd
    for i in range(2):
        p.pre_pad[i], p.post_pad[i], p.stride[i], p.dilation[i] = 1, 1, 1, 1
    w = np.ones(9, dtype=np.float32)
    for centre, check in ((0.0, lambda y: np.all(y == 0)), (np.nan, lambda y: np.all(np.isnan(y))), (np.inf, lambda y: np.all(y == np.inf))):
        x = np.zeros(9, dtype=np.float32)
        x[4] = centre
        dx, dw, dy = g.to_device(x), g.to_device(w), g.device_zeros(36)
        for kernel in (dfgpu.CONV_DIRECT, dfgpu.CONV_IGEMM_FFMA):
            p.kernel = kernel
            dfgpu.conv_fprop(p, g.ptr(dx), g.ptr(dw), g.ptr(dy))
            assert check(g.to_host(dy, np.float32)), (centre, kernel)


def run_matmul(dtype, a_dims, b_dims, kernel=dfgpu.MATMUL_FFMA, a_strides=None, b_strides=None, seed=2):
    rank = len(a_dims)
    c_dims = [max(x, y) for x, y in zip(a_dims[:-2], b_dims[:-2])] + [a_dims[-2], b_dims[-1]]
    a = synthetic.normal(seed, 1, int(np.prod(a_dims)))
    b = synthetic.normal(seed, 2, int(np.prod(b_dims)))
    fa = synthetic.round_to_bf16(a) if dtype == BF16 else a
    fb = synthetic.round_to_bf16(b) if dtype == BF16 else b
    ref = np.zeros(int(np.prod(c_dims)), dtype=np.float32)
    oracle.matmul(tensor(F32, a_dims, a_strides), fa, tensor(F32, b_dims, b_strides), fb, tensor(F32, c_dims), ref)
    p = dfgpu.MatmulParams()
    p.a, p.b, p.c, p.kernel = tensor(dtype, a_dims, a_strides), tensor(dtype, b_dims, b_strides), tensor(dtype, c_dims), kernel
    da, db = g.to_device(host_array(a, dtype)), g.to_device(host_array(b, dtype))
    dc = g.device_zeros(ref.size * dfgpu.DTYPE_BYTES[dtype])
    info = dfgpu.query("matmul", p)
    scratch = g.device_zeros(info.scratch_bytes, 0xA5) if info.scratch_bytes else None
    dfgpu.matmul(p, g.ptr(da), g.ptr(db), g.ptr(dc), scratch=g.ptr(scratch))
    return read_back(dc, dtype, -1), ref


@pytest.mark.parametrize("a_dims,b_dims,b_strides", [([256, 128], [128, 192], None), ([130, 96], [96, 64], None), ([200, 64], [64, 128], [1, 64]),
                                                    ([1024, 1024], [1024, 1024], None), ([2048, 512], [512, 1024], None)])
def test_matmul_f32_on_tensor_cores(a_dims, b_dims, b_strides):
    """f32 A, B, C resolve to the split-operand tcgen05 form (six bf16 products, f32 accumulation) and hold the f32 gates
    against the oracle, for N-contiguous and K-contiguous B and a last row tile that is not full."""
    p = dfgpu.MatmulParams()
    p.a, p.b, p.c = tensor(F32, a_dims), tensor(F32, b_dims, b_strides), tensor(F32, [a_dims[0], b_dims[1]])
    # AUTO: the one-launch form where it fits and pays (K >= 128; at most 148 tiles or one tile of columns), the three-launch form for other big products, else CUDA cores
    expected = {(256, 128): dfgpu.MATMUL_UMMA_F32X3_CLUSTER, (1024, 1024): dfgpu.MATMUL_UMMA_F32X3_CLUSTER,
                (2048, 512): dfgpu.MATMUL_UMMA_F32X3}.get((a_dims[0], a_dims[1]), dfgpu.MATMUL_FFMA)
    assert dfgpu.query("matmul", p).kernel == expected
    p.kernel = dfgpu.MATMUL_UMMA_F32X3
    info = dfgpu.query("matmul", p)
    assert info.kernel == dfgpu.MATMUL_UMMA_F32X3 and info.launches == 3 and info.scratch_bytes > 0
    out, ref = run_matmul(F32, a_dims, b_dims, kernel=dfgpu.MATMUL_UMMA_F32X3, b_strides=b_strides)
    check_f32(out, ref)
    cores, _ = run_matmul(F32, a_dims, b_dims, kernel=dfgpu.MATMUL_FFMA, b_strides=b_strides)
    assert float(np.max(np.abs(out - cores))) <= 2e-5 * float(np.max(np.abs(ref)))  # (each carries its own f32 accumulation error)
    assert not np.array_equal(out, cores)  # (the tensor-core result stands: no operand was infinite or NaN)


@pytest.mark.parametrize("a_dims,b_dims,b_strides", [([256, 128], [128, 192], None), ([130, 64], [64, 64], None), ([200, 64], [64, 128], [1, 64]),
                                                    ([512, 512], [512, 256], None), ([1000, 1024], [1024, 64], [1, 1024]),
                                                    ([100, 40], [40, 12], None), ([130, 136], [136, 68], None), ([130, 136], [136, 68], [1, 136])])
def test_matmul_f32_in_one_launch_on_tensor_cores(a_dims, b_dims, b_strides):
    """An unbatched f32 product of at most 148 output tiles runs on the one-launch tcgen05 kernel of the f32 convolution (as the 1 x 1
    convolution of M pixels): no scratch, N-contiguous and K-contiguous B, a last row tile that is not full, one to eight CTAs per tile, and
    a bias row + ReLU + full-size addend in the epilogue; K need only be a multiple of 8 and N of 4. AUTO takes it from K = 128 on (the CUDA-core
    kernel walks K in steps of 16)."""
    m, k, n = a_dims[0], a_dims[1], b_dims[1]
    p = dfgpu.MatmulParams()
    p.a, p.b, p.c = tensor(F32, a_dims), tensor(F32, b_dims, b_strides), tensor(F32, [m, n])
    assert dfgpu.query("matmul", p).kernel == (dfgpu.MATMUL_UMMA_F32X3_CLUSTER if k >= 128 else dfgpu.MATMUL_FFMA)
    p.kernel = dfgpu.MATMUL_UMMA_F32X3_CLUSTER
    info = dfgpu.query("matmul", p)
    assert info.kernel == dfgpu.MATMUL_UMMA_F32X3_CLUSTER and info.launches == 1 and info.scratch_bytes == 0
    out, ref = run_matmul(F32, a_dims, b_dims, kernel=dfgpu.MATMUL_UMMA_F32X3_CLUSTER, b_strides=b_strides)
    check_f32(out, ref)
    cores, _ = run_matmul(F32, a_dims, b_dims, kernel=dfgpu.MATMUL_FFMA, b_strides=b_strides)
    assert float(np.max(np.abs(out - cores))) <= 2e-5 * float(np.max(np.abs(ref)))
    assert not np.array_equal(out, cores)
    # the epilogue: C = relu(A B + bias[n]) + addend[m, n], against the CUDA-core kernel's
    bias, addend = synthetic.uniform(8, 1, n, -1.0, 1.0).astype(np.float32), synthetic.normal(8, 2, m * n).astype(np.float32)
    p.extra[0], p.extra[1] = tensor(F32, [1, n]), tensor(F32, [m, n])
    p.epilogue_count = 3
    p.epilogue[0], p.epilogue[1], p.epilogue[2] = step(dfgpu.EPI_ADD, 0), step(dfgpu.EPI_RELU), step(dfgpu.EPI_ADD, 1)
    da = g.to_device(synthetic.normal(2, 1, m * k).astype(np.float32))
    db = g.to_device(synthetic.normal(2, 2, k * n).astype(np.float32))
    d0, d1 = g.to_device(bias), g.to_device(addend)
    results = {}
    for kernel in (dfgpu.MATMUL_FFMA, dfgpu.MATMUL_UMMA_F32X3_CLUSTER):
        p.kernel = kernel
        dc = g.device_zeros(m * n * 4, 0x5A)
        dfgpu.matmul(p, g.ptr(da), g.ptr(db), g.ptr(dc), extra0=g.ptr(d0), extra1=g.ptr(d1))
        results[kernel] = g.to_host(dc, np.float32).copy()
    plain = np.maximum(ref.reshape(m, n) + bias[None, :], 0.0) + addend.reshape(m, n)
    check_f32(results[dfgpu.MATMUL_UMMA_F32X3_CLUSTER].reshape(m, n), plain)
    assert float(np.max(np.abs(results[dfgpu.MATMUL_UMMA_F32X3_CLUSTER] - results[dfgpu.MATMUL_FFMA]))) <= 2e-5 * float(np.max(np.abs(plain)))
    assert dfgpu.device_status() == 0


@pytest.mark.parametrize("a_dims,b_dims", [([4, 130, 136], [4, 136, 68]), ([4, 130, 136], [1, 136, 68]), ([1, 200, 72], [5, 72, 31]), ([3, 1, 65, 129], [3, 1, 129, 64])])
def test_matmul_batched_in_one_launch_on_tensor_cores(a_dims, b_dims):
    """One batch axis (either operand may be broadcast along it): every matrix of the batch is one image of the 1 x 1 convolution, with its
    own filter where B is batched; row, reduction and column counts that fill no tile."""
    p = dfgpu.MatmulParams()
    c_dims = [max(x, y) for x, y in zip(a_dims[:-2], b_dims[:-2])] + [a_dims[-2], b_dims[-1]]
    p.a, p.b, p.c = tensor(F32, a_dims), tensor(F32, b_dims), tensor(F32, c_dims)
    p.kernel = dfgpu.MATMUL_UMMA_F32X3_CLUSTER
    info = dfgpu.query("matmul", p)
    assert info.kernel == dfgpu.MATMUL_UMMA_F32X3_CLUSTER and info.launches == 1 and info.scratch_bytes == 0
    out, ref = run_matmul(F32, a_dims, b_dims, kernel=dfgpu.MATMUL_UMMA_F32X3_CLUSTER)
    check_f32(out, ref)
    cores, _ = run_matmul(F32, a_dims, b_dims, kernel=dfgpu.MATMUL_FFMA)
    assert float(np.max(np.abs(out - cores))) <= 2e-5 * float(np.max(np.abs(ref)))
    # two batch axes of extent > 1 stay on CUDA cores
    q = dfgpu.MatmulParams()
    q.a, q.b, q.c = tensor(F32, [3, 1, 65, 136]), tensor(F32, [1, 2, 136, 64]), tensor(F32, [3, 2, 65, 64])
    assert dfgpu.query("matmul", q).kernel == dfgpu.MATMUL_FFMA
    assert dfgpu.device_status() == 0


def test_matmul_f32_one_launch_form_with_other_strides():
    """A stored transposed, rows of B padded to 130 floats (no 16-byte row pitch) and rows of C padded to 132: the one-launch kernel
    reads A and B value by value and still stores C as float4s."""
    m, k, n = 300, 256, 128
    a_store = synthetic.normal(5, 1, k * m).astype(np.float32)            # [k, m]: A[i, j] = a_store[j * m + i]
    b_store = synthetic.normal(5, 2, k * 130).astype(np.float32)          # [k, 130]
    p = dfgpu.MatmulParams()
    p.a, p.b, p.c = tensor(F32, [m, k], [1, m]), tensor(F32, [k, n], [130, 1]), tensor(F32, [m, n], [132, 1])
    ref = (a_store.reshape(k, m).T.astype(np.float64) @ b_store.reshape(k, 130)[:, :n].astype(np.float64)).astype(np.float32)
    da, db = g.to_device(a_store), g.to_device(b_store)
    results = {}
    for kernel in (dfgpu.MATMUL_AUTO, dfgpu.MATMUL_FFMA):
        p.kernel = kernel
        if kernel == dfgpu.MATMUL_AUTO:
            assert dfgpu.query("matmul", p).kernel == dfgpu.MATMUL_UMMA_F32X3_CLUSTER
        dc = g.device_zeros(m * 132 * 4, 0x5A)
        dfgpu.matmul(p, g.ptr(da), g.ptr(db), g.ptr(dc))
        stored = g.to_host(dc, np.float32).copy().reshape(m, 132)
        assert np.all(stored[:, n:].view(np.uint32) == 0x5A5A5A5A)  # (the padding of C's rows is not touched)
        results[kernel] = stored[:, :n]
    check_f32(results[dfgpu.MATMUL_AUTO], ref)
    assert float(np.max(np.abs(results[dfgpu.MATMUL_AUTO] - results[dfgpu.MATMUL_FFMA]))) <= 2e-5 * float(np.max(np.abs(ref)))
    assert dfgpu.device_status() == 0


@pytest.mark.parametrize("b_strides", [None, [1, 128]])
def test_matmul_f32_one_launch_form_with_non_finite_operand(b_strides):
    """An infinity in A (rows 0..127 are the first tile) and a NaN in B: a cluster that sees one computes its tile on the CUDA cores, bit
    for bit the CUDA-core kernel's result; the NaN in B is in every tile's filter."""
    a_dims, b_dims = [256, 128], [128, 64]
    for where in ("a", "b"):
        a = synthetic.normal(4, 1, 256 * 128).astype(np.float32)
        b = np.full(128 * 64, 0.5, dtype=np.float32)  # (lower pieces of exactly zero: inf * 0 in the split products)
        if where == "a": a[77] = np.inf
        else: b[5 * 64 + 9] = np.nan
        p = dfgpu.MatmulParams()
        p.a, p.b, p.c = tensor(F32, a_dims), tensor(F32, b_dims, b_strides), tensor(F32, [256, 64])
        da, db = g.to_device(a), g.to_device(b)
        results = {}
        for kernel in (dfgpu.MATMUL_FFMA, dfgpu.MATMUL_UMMA_F32X3_CLUSTER):
            p.kernel = kernel
            dc = g.device_zeros(256 * 64 * 4, 0x5A)
            dfgpu.matmul(p, g.ptr(da), g.ptr(db), g.ptr(dc))
            results[kernel] = g.to_host(dc, np.uint32).copy().reshape(256, 64)
        cores, cluster = results[dfgpu.MATMUL_FFMA], results[dfgpu.MATMUL_UMMA_F32X3_CLUSTER]
        exact_rows = slice(0, 128) if where == "a" else slice(0, 256)
        assert np.array_equal(cores[exact_rows], cluster[exact_rows])
        assert not np.all(np.isfinite(cores.view(np.float32)))
        if where == "a":
            assert np.all(np.isfinite(cluster[128:].view(np.float32)))
            assert float(np.max(np.abs(cluster[128:].view(np.float32) - cores[128:].view(np.float32)))) <= 2e-5 * float(np.max(np.abs(cores[128:].view(np.float32))))
    assert dfgpu.device_status() == 0


def test_matmul_f32_split_form_with_non_finite_operand():
    """An infinity in A: the CUDA-core kernel behind the tensor-core one redoes the product, bit for bit its own result."""
    a_dims, b_dims = [128, 64], [64, 64]
    a = synthetic.normal(4, 1, 128 * 64).astype(np.float32)
    b = np.full(64 * 64, 0.5, dtype=np.float32)  # (lower pieces of exactly zero: inf * 0 in the split products)
    a[77] = np.inf
    p = dfgpu.MatmulParams()
    p.a, p.b, p.c = tensor(F32, a_dims), tensor(F32, b_dims), tensor(F32, [128, 64])
    da, db = g.to_device(a), g.to_device(b)
    results = {}
    for kernel in (dfgpu.MATMUL_FFMA, dfgpu.MATMUL_UMMA_F32X3):
        p.kernel = kernel
        info = dfgpu.query("matmul", p)
        dc = g.device_zeros(128 * 64 * 4, 0x5A)
        scratch = g.device_zeros(info.scratch_bytes, 0xA5) if info.scratch_bytes else None
        dfgpu.matmul(p, g.ptr(da), g.ptr(db), g.ptr(dc), scratch=g.ptr(scratch))
        results[kernel] = g.to_host(dc, np.uint32).copy()
    assert np.array_equal(results[dfgpu.MATMUL_FFMA], results[dfgpu.MATMUL_UMMA_F32X3])
    assert np.isinf(results[dfgpu.MATMUL_FFMA].view(np.float32)).any()


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("a_dims,b_dims", [([2, 2, 3], [1, 3, 2]), ([70, 45], [45, 33]), ([3, 1, 65, 129], [1, 2, 129, 64])])
def test_matmul_ffma(dtype, a_dims, b_dims):
    out, ref = run_matmul(dtype, a_dims, b_dims)
    (check_f32 if dtype == F32 else check_bf16)(out, ref)


def test_matmul_transposed_strides():
    out, ref = run_matmul(F32, [40, 24], [24, 56], a_strides=[1, 40], b_strides=[1, 24])
    check_f32(out, ref)


def test_matmul_known_answer_with_bias_epilogue():
    a = np.array([1, 2, 3, 4, 5, 6, -1, 0, 1, 2, -2, 1], dtype=np.float32)
    b = np.array([1, 2, 0, 1, 1, 0], dtype=np.float32)
    bias = np.array([0.5, -1.0], dtype=np.float32)
    p = dfgpu.MatmulParams()
    p.a, p.b, p.c = tensor(F32, [2, 2, 3]), tensor(F32, [1, 3, 2]), tensor(F32, [2, 2, 2])
    p.extra[0] = tensor(F32, [2])
    p.epilogue_count = 1
    p.epilogue[0] = step(dfgpu.EPI_ADD, 0)
    da, db, dbias, dc = g.to_device(a), g.to_device(b), g.to_device(bias), g.device_zeros(32)
    dfgpu.matmul(p, g.ptr(da), g.ptr(db), g.ptr(dc), extra0=g.ptr(dbias))
    assert g.to_host(dc, np.float32).tolist() == [4.5, 3.0, 10.5, 12.0, 0.5, -3.0, 3.5, 1.0]


def test_matmul_with_fused_block_dequantize():
    """quantize -> (dequantize -> matmul fused): equals the oracle's dequantize + f32 matmul."""
    m, k, n = 96, 128, 80
    a = synthetic.normal(7, 1, m * k)
    b = synthetic.normal(7, 2, k * n)
    aq, sa = np.zeros(m * k, dtype=np.uint8), np.zeros(m * k // 32, dtype=np.uint8)
    bq, sb = np.zeros(k * n, dtype=np.uint8), np.zeros(k * n // 32, dtype=np.uint8)
    oracle.block_scale_quantize(tensor(F32, [m, k]), a, tensor(E4M3, [m, k]), aq, tensor(E8M0, [m, k // 32]), sa, 32, 1)
    oracle.block_scale_quantize(tensor(F32, [k, n]), b, tensor(E4M3, [k, n]), bq, tensor(E8M0, [k // 32, n]), sb, 32, 0)
    af, bf = np.zeros(m * k, dtype=np.float32), np.zeros(k * n, dtype=np.float32)
    oracle.block_scale_dequantize(tensor(E4M3, [m, k]), aq, tensor(E8M0, [m, k // 32]), sa, tensor(F32, [m, k]), af, [1, 32])
    oracle.block_scale_dequantize(tensor(E4M3, [k, n]), bq, tensor(E8M0, [k // 32, n]), sb, tensor(F32, [k, n]), bf, [32, 1])
    ref = np.zeros(m * n, dtype=np.float32)
    oracle.matmul(tensor(F32, [m, k]), af, tensor(F32, [k, n]), bf, tensor(F32, [m, n]), ref)
    p = dfgpu.MatmulParams()
    p.a, p.b, p.c = tensor(E4M3, [m, k]), tensor(E4M3, [k, n]), tensor(F32, [m, n])
    p.a_scale, p.b_scale = tensor(E8M0, [m, k // 32]), tensor(E8M0, [k // 32, n])
    p.a_block[0], p.a_block[1], p.b_block[0], p.b_block[1] = 1, 32, 32, 1
    p.kernel = dfgpu.MATMUL_FFMA
    d = [g.to_device(v) for v in (aq, bq, sa, sb)]
    dc = g.device_zeros(m * n * 4)
    dfgpu.matmul(p, g.ptr(d[0]), g.ptr(d[1]), g.ptr(dc), g.ptr(d[2]), g.ptr(d[3]))
    check_f32(g.to_host(dc, np.float32), ref)
