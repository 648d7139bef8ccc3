"""Bit-exact parity of the block-scale kernels with the CPU oracle, through the C ABI."""
import numpy as np
import pytest

import oracle
from deepforge_b200 import dfgpu, synthetic
from deepforge_b200.dfgpu import BF16, E4M3, E5M2, E8M0, F16, F32, FP4, I4, REORDER_F8_128x4, tensor

pytestmark = pytest.mark.gpu

NP_OF = {F32: np.float32, F16: np.float16, BF16: np.uint16}


def _make_x(dtype, shape, seed, special=False):
    count = int(np.prod(shape))
    values = synthetic.normal(seed, 1, count)
    mask = synthetic.outlier_mask(seed, 1, count)
    values = np.where(mask, values * 64.0, values).astype(np.float32)
    if special:
        values[::97] = 0.0
        values[5::101] = -0.0
        values[7::211] = -1e-7          # negative that rounds to zero
        values[11::257] = np.float32(448.0)
        values[13::509] = np.inf
        values[17::1021] = np.nan
        values[19::127] = 1e-30
        values[23::131] = -3.0e38
    if dtype == F32:
        return values.reshape(shape)
    if dtype == F16:
        with np.errstate(over="ignore"):
            return values.astype(np.float16).reshape(shape)
    return synthetic.to_bf16_bits(values).reshape(shape)


def _quantize_both(dtype, shape, block, axis, kernel, scale_dims=None, scale_strides=None, reorder=0, seed=3, special=False,
                   x_strides=None, code_type=E4M3):
    import gpu_util as g
    x = _make_x(dtype, shape, seed, special)
    logical = list(shape)
    logical[axis] //= block
    scale_dims = scale_dims or logical
    xd = tensor(dtype, shape, x_strides)
    yd = tensor(code_type, shape)
    sd = tensor(E8M0, scale_dims, scale_strides, reorder)
    scale_bytes = int(np.prod(scale_dims))
    y_ref = np.zeros(int(np.prod(shape)), dtype=np.uint8)
    s_ref = np.full(scale_bytes, 0xAA, dtype=np.uint8)
    oracle.block_scale_quantize(xd, x, yd, y_ref, sd, s_ref, block, axis)

    p = dfgpu.BsqParams()
    p.x, p.y, p.scale, p.block_size, p.axis, p.kernel = xd, yd, sd, block, axis, kernel
    info = dfgpu.query("block_scale_quantize", p)
    dx = g.to_device(x)
    dy = g.device_zeros(y_ref.size, 0x55)
    ds = g.device_zeros(scale_bytes, 0xAA)
    dfgpu.block_scale_quantize(p, g.ptr(dx), g.ptr(dy), g.ptr(ds))
    y = g.to_host(dy, np.uint8)
    s = g.to_host(ds, np.uint8)
    return info, x, y, s, y_ref, s_ref


@pytest.mark.parametrize("dtype", [F32, F16, BF16])
def test_e5m2_codes_match_oracle_and_the_reference_known_answers(dtype):
    """FP8_E5M2 codes run on the general kernels: the scale rule divides by 57344 (known answers of test/Compiler/SpecializedOpsTest.cpp:640-659
    and :716-735), and codes and scales equal the oracle's bit for bit on ordinary and special values, blocks along either axis, plain and
    F8_128x4 scale layouts; dequantize likewise."""
    import gpu_util as g
    if dtype == F32:
        p = dfgpu.BsqParams()
        p.x, p.y, p.scale, p.block_size, p.axis = tensor(F32, [1, 4]), tensor(E5M2, [1, 4]), tensor(E8M0, [1, 2]), 2, 1
        assert dfgpu.query("block_scale_quantize", p).kernel == dfgpu.BSQ_GENERIC
        dx, dy, ds = g.to_device(np.array([1.0, 2.0, -4.0, 8.0], dtype=np.float32)), g.device_zeros(4), g.device_zeros(2)
        dfgpu.block_scale_quantize(p, g.ptr(dx), g.ptr(dy), g.ptr(ds))
        assert g.to_host(ds, np.uint8).tolist() == [113, 115] and g.to_host(dy, np.uint8).tolist() == [0x74, 0x78, 0xf4, 0x78]
        q = dfgpu.BsdParams()
        q.x, q.scale, q.y, q.block_count = tensor(E5M2, [1, 4]), tensor(E8M0, [1, 2]), tensor(F32, [1, 4]), 1
        q.block[0] = 2
        dx, ds, dy = g.to_device(np.array([0x3c, 0x40, 0xc0, 0x38], dtype=np.uint8)), g.to_device(np.array([127, 128], dtype=np.uint8)), g.device_zeros(16)
        dfgpu.block_scale_dequantize(q, g.ptr(dx), g.ptr(ds), g.ptr(dy))
        assert g.to_host(dy, np.float32).tolist() == [1.0, 2.0, -4.0, 1.0]
    for shape, block, axis, special, reorder, scale_dims in (([128, 256], 32, 1, False, 0, None), ([128, 256], 32, 1, True, 0, None), ([256, 64], 32, 0, True, 0, None),
                                                              ([3, 40, 48], 8, 2, True, 0, None), ([128, 128], 32, 1, True, REORDER_F8_128x4, [128, 4])):
        info, x, y, s, y_ref, s_ref = _quantize_both(dtype, shape, block, axis, dfgpu.BSQ_AUTO, scale_dims=scale_dims, reorder=reorder, special=special, code_type=E5M2)
        assert info.kernel == dfgpu.BSQ_GENERIC
        assert np.array_equal(s, s_ref) and np.array_equal(y, y_ref)
        if reorder:
            continue
        # and back: the general dequantize kernel on the E5M2 codes against the oracle, bit for bit
        blocks = [1] * len(shape)
        blocks[axis] = block
        out_type = dtype
        width = dfgpu.DTYPE_BYTES[out_type]
        ref = np.zeros(int(np.prod(shape)) * width, dtype=np.uint8)
        logical = list(shape)
        logical[axis] //= block
        oracle.block_scale_dequantize(tensor(E5M2, shape), y_ref, tensor(E8M0, logical), s_ref, tensor(out_type, shape), ref, blocks)
        q = dfgpu.BsdParams()
        q.x, q.scale, q.y, q.block_count = tensor(E5M2, shape), tensor(E8M0, logical), tensor(out_type, shape), len(shape)
        for i, b in enumerate(blocks):
            q.block[i] = b
        dx, ds, dy = g.to_device(y_ref), g.to_device(s_ref), g.device_zeros(ref.size, 0x11)
        dfgpu.block_scale_dequantize(q, g.ptr(dx), g.ptr(ds), g.ptr(dy))
        out = g.to_host(dy, np.uint8)
        view = np.uint32 if width == 4 else np.uint16
        a, b = out.view(view), ref.view(view)
        as_float = (out.view(np.float32) if out_type == F32 else out.view(np.float16).astype(np.float32) if out_type == F16
                    else synthetic.bf16_bits_to_f32(out.view(np.uint16)))
        nan = np.isnan(as_float)
        assert np.array_equal(a[~nan], b[~nan]) and nan.any() == special


@pytest.mark.parametrize("dtype", [F32, F16, BF16])
def test_packed_four_bit_codes_match_oracle_and_the_reference_known_answers(dtype):
    """FP4_E2M1 codes (two to a byte) with FP8_E4M3 scales, and INT4 with floating scales, on the general kernels: the reference's known
    answers (test/Compiler/SpecializedOpsTest.cpp:661-681, :736-754) and bit-exact parity with the oracle on ordinary and special values,
    blocks along the contiguous axis and across it (neighbouring threads then share bytes)."""
    import gpu_util as g
    if dtype == F32:
        p = dfgpu.BsqParams()
        p.x, p.y, p.scale, p.block_size, p.axis = tensor(F32, [1, 4]), tensor(FP4, [1, 4]), tensor(E4M3, [1, 2]), 2, 1
        assert dfgpu.query("block_scale_quantize", p).kernel == dfgpu.BSQ_GENERIC
        dx, dy, ds = g.to_device(np.array([1.0, 2.0, -3.0, 6.0], dtype=np.float32)), g.device_zeros(4), g.device_zeros(4)
        dfgpu.block_scale_quantize(p, g.ptr(dx), g.ptr(dy), g.ptr(ds))
        q = dfgpu.BsdParams()
        q.x, q.scale, q.y, q.block_count = tensor(FP4, [1, 4]), tensor(E4M3, [1, 2]), tensor(F32, [1, 4]), 1
        q.block[0] = 2
        dout = g.device_zeros(16)
        dfgpu.block_scale_dequantize(q, g.ptr(dy), g.ptr(ds), g.ptr(dout))
        assert g.to_host(dout, np.float32).tolist() == [1.03125, 2.0625, -3.0, 6.0]
        q.x, q.scale, q.y = tensor(I4, [1, 4]), tensor(F16, [1, 2]), tensor(BF16, [1, 4])
        dx, ds, dout = g.to_device(np.array([0xf8, 0x70, 0, 0], dtype=np.uint8)), g.to_device(np.array([0x3800, 0x4000], dtype=np.uint16)), g.device_zeros(8)
        dfgpu.block_scale_dequantize(q, g.ptr(dx), g.ptr(ds), g.ptr(dout))
        assert g.to_host(dout, np.uint16).tolist() == [0xc080, 0xbf00, 0x0000, 0x4160]
    for shape, block, axis, special in (([64, 128], 16, 1, False), ([64, 128], 32, 1, True), ([96, 40], 32, 0, True), ([3, 20, 24], 4, 1, True)):
        count = int(np.prod(shape))
        x = _make_x(dtype, shape, 31, special)
        logical = list(shape)
        logical[axis] //= block
        xd, yd, sd = tensor(dtype, shape), tensor(FP4, shape), tensor(E4M3, logical)
        y_ref, s_ref = np.zeros(count // 2, dtype=np.uint8), np.zeros(int(np.prod(logical)), dtype=np.uint8)
        oracle.block_scale_quantize(xd, x, yd, y_ref, sd, s_ref, block, axis)
        p = dfgpu.BsqParams()
        p.x, p.y, p.scale, p.block_size, p.axis = xd, yd, sd, block, axis
        dx, dy, ds = g.to_device(x), g.device_zeros(count // 2, 0x55), g.device_zeros(s_ref.size, 0xAA)
        dfgpu.block_scale_quantize(p, g.ptr(dx), g.ptr(dy), g.ptr(ds))
        assert np.array_equal(g.to_host(ds, np.uint8), s_ref) and np.array_equal(g.to_host(dy, np.uint8), y_ref)
        # back through the general dequantize kernel, and the same nibbles read as INT4 with bf16 scales
        blocks = [1] * len(shape)
        blocks[axis] = block
        for code_type, scale_type, scales in ((FP4, E4M3, s_ref), (I4, BF16, synthetic.to_bf16_bits(synthetic.uniform(31, 3, s_ref.size, -2.0, 2.0)))):
            width = dfgpu.DTYPE_BYTES[dtype]
            ref = np.zeros(count * width, dtype=np.uint8)
            oracle.block_scale_dequantize(tensor(code_type, shape), y_ref, tensor(scale_type, logical), scales, tensor(dtype, shape), ref, blocks)
            q = dfgpu.BsdParams()
            q.x, q.scale, q.y, q.block_count = tensor(code_type, shape), tensor(scale_type, logical), tensor(dtype, shape), len(shape)
            for i, b in enumerate(blocks):
                q.block[i] = b
            dcodes, dscales, dout = g.to_device(y_ref), g.to_device(scales), g.device_zeros(ref.size, 0x11)
            dfgpu.block_scale_dequantize(q, g.ptr(dcodes), g.ptr(dscales), g.ptr(dout))
            out = g.to_host(dout, np.uint8)
            view = np.uint32 if width == 4 else np.uint16
            as_float = (out.view(np.float32) if dtype == F32 else out.view(np.float16).astype(np.float32) if dtype == F16
                        else synthetic.bf16_bits_to_f32(out.view(np.uint16)))
            nan = np.isnan(as_float)
            assert np.array_equal(out.view(view)[~nan], ref.view(view)[~nan])


def test_known_answers_through_the_abi():
    import gpu_util as g
    p = dfgpu.BsqParams()
    p.x, p.y, p.scale = tensor(F32, [1, 4]), tensor(E4M3, [1, 4]), tensor(E8M0, [1, 2])
    p.block_size, p.axis = 2, 1
    for values, scales, codes in (
        ([1.0, 2.0, -4.0, 8.0], [120, 122], [0x70, 0x78, 0xf0, 0x78]),
        ([np.inf, 0.0, np.nan, 0.0], [0xfe, 0xff], [0x7e, 0x00, 0x7f, 0x7f]),
    ):
        dx = g.to_device(np.array(values, dtype=np.float32))
        dy, ds = g.device_zeros(4), g.device_zeros(2)
        dfgpu.block_scale_quantize(p, g.ptr(dx), g.ptr(dy), g.ptr(ds))
        assert g.to_host(ds, np.uint8).tolist() == scales
        assert g.to_host(dy, np.uint8).tolist() == codes
    q = dfgpu.BsdParams()
    q.x, q.scale, q.y = tensor(E4M3, [1, 4]), tensor(E8M0, [1, 2]), tensor(F32, [1, 4])
    q.block[0], q.block_count = 2, 1
    dx = g.to_device(np.array([0x38, 0x40, 0xb8, 0x30], dtype=np.uint8))
    ds = g.to_device(np.array([127, 128], dtype=np.uint8))
    dy = g.device_zeros(16)
    dfgpu.block_scale_dequantize(q, g.ptr(dx), g.ptr(ds), g.ptr(dy))
    assert g.to_host(dy, np.float32).tolist() == [1.0, 2.0, -2.0, 1.0]


@pytest.mark.parametrize("dtype", [F32, F16, BF16])
@pytest.mark.parametrize("kernel", [dfgpu.BSQ_GENERIC, dfgpu.BSQ_ROW32])
def test_row_blocks_match_oracle(dtype, kernel):
    info, x, y, s, y_ref, s_ref = _quantize_both(dtype, [96, 256], 32, 1, kernel, special=True)
    assert info.kernel == kernel
    assert np.array_equal(s, s_ref)
    assert np.array_equal(y, y_ref)


@pytest.mark.parametrize("dtype", [F32, F16, BF16])
@pytest.mark.parametrize("kernel", [dfgpu.BSQ_GENERIC, dfgpu.BSQ_COL32])
def test_column_blocks_match_oracle(dtype, kernel):
    info, x, y, s, y_ref, s_ref = _quantize_both(dtype, [3, 128, 72], 32, 1, kernel, special=True, seed=9)
    assert info.kernel == kernel
    assert np.array_equal(s, s_ref)
    assert np.array_equal(y, y_ref)


@pytest.mark.parametrize("shape,axis", [([1000, 1056], 1), ([2, 96, 1000], 1), ([7, 32], 1), ([64, 8], 0), ([9, 3200, 264], 1)])
def test_ragged_bf16_tiles_match_oracle(shape, axis):
    """Sizes that leave the streaming kernel a partial last tile (row form: elements % 8192 != 0; column form: N % 256
    != 0) and more tiles than one pass of the grid (the last case walks its ring of stages around)."""
    info, x, y, s, y_ref, s_ref = _quantize_both(BF16, shape, 32, axis, dfgpu.BSQ_AUTO, special=True, seed=31)
    assert info.kernel == (dfgpu.BSQ_ROW32 if axis == len(shape) - 1 else dfgpu.BSQ_COL32)
    assert np.array_equal(s, s_ref)
    assert np.array_equal(y, y_ref)


@pytest.mark.parametrize("axis", [1, 0])
def test_every_bf16_amax_pattern(axis):
    """One block per bf16 magnitude pattern (0 .. 0x7fff: zero, subnormals, every exponent and fraction, infinity and
    the NaNs) as that block's largest |x|, the other elements anywhere below it with random signs: the bf16 kernels
    derive the scale code from the pattern's bits and multiply in bf16, and must still equal the oracle bit for bit."""
    import gpu_util as g
    rng = np.random.default_rng(77)
    top = np.arange(0x8000, dtype=np.uint32)
    magnitude = (rng.random((0x8000, 32)) * (top[:, None] + 1)).astype(np.uint32)
    magnitude = np.minimum(magnitude, top[:, None])
    magnitude[np.arange(0x8000), rng.integers(0, 32, 0x8000)] = top
    bits = (magnitude | (rng.integers(0, 2, magnitude.shape).astype(np.uint32) << 15)).astype(np.uint16)
    if axis == 1:
        x = bits.reshape(1024, 1024)          # block b = elements 32b .. 32b+31 of the flattened tensor
        sdims = [1024, 32]
    else:
        x = np.ascontiguousarray(bits.reshape(32, 1024, 32).transpose(0, 2, 1)).reshape(1024, 1024)  # block (kb, n) down the rows
        sdims = [32, 1024]
    xd, yd, sd = tensor(BF16, [1024, 1024]), tensor(E4M3, [1024, 1024]), tensor(E8M0, sdims)
    y_ref = np.zeros(1024 * 1024, dtype=np.uint8)
    s_ref = np.zeros(32768, dtype=np.uint8)
    oracle.block_scale_quantize(xd, x, yd, y_ref, sd, s_ref, 32, axis)
    p = dfgpu.BsqParams()
    p.x, p.y, p.scale, p.block_size, p.axis = xd, yd, sd, 32, axis
    dx, dy, ds = g.to_device(x), g.device_zeros(y_ref.size, 0x55), g.device_zeros(32768, 0xAA)
    dfgpu.block_scale_quantize(p, g.ptr(dx), g.ptr(dy), g.ptr(ds))
    assert np.array_equal(g.to_host(ds, np.uint8), s_ref)
    assert np.array_equal(g.to_host(dy, np.uint8), y_ref)


@pytest.mark.parametrize("shapes", [(([300, 1056], 1), ([96, 1000], 0)), (([64, 264], 0), ([2, 64, 72], 1)), (([33, 64], 1), ([9, 32], 1))])
def test_quantize_pair_matches_oracle(shapes):
    """Two tensors through dfgpu_block_scale_quantize_pair (one grid): each result equals the oracle's for that tensor
    alone, for row+column, column+column and row+row pairs with ragged last tiles."""
    import gpu_util as g
    pair = dfgpu.BsqPairParams()
    device, expected = [], []
    for index, (shape, axis) in enumerate(shapes):
        x = _make_x(BF16, shape, 40 + index, special=True)
        logical = list(shape)
        logical[axis] //= 32
        xd, yd, sd = tensor(BF16, shape), tensor(E4M3, shape), tensor(E8M0, logical)
        y_ref = np.zeros(int(np.prod(shape)), dtype=np.uint8)
        s_ref = np.zeros(int(np.prod(logical)), dtype=np.uint8)
        oracle.block_scale_quantize(xd, x, yd, y_ref, sd, s_ref, 32, axis)
        p = pair.first if index == 0 else pair.second
        p.x, p.y, p.scale, p.block_size, p.axis = xd, yd, sd, 32, axis
        device.append((g.to_device(x), g.device_zeros(y_ref.size, 0x55), g.device_zeros(s_ref.size, 0xAA)))
        expected.append((y_ref, s_ref))
    assert dfgpu.query("block_scale_quantize_pair", pair).launches == 1
    dfgpu.block_scale_quantize_pair(pair, [g.ptr(t) for t in device[0]], [g.ptr(t) for t in device[1]])
    for (dx, dy, ds), (y_ref, s_ref) in zip(device, expected):
        assert np.array_equal(g.to_host(ds, np.uint8), s_ref)
        assert np.array_equal(g.to_host(dy, np.uint8), y_ref)
    assert dfgpu.device_status() == 0


@pytest.mark.parametrize("block,axis,shape", [(2, 1, [5, 6]), (16, 0, [32, 7]), (64, 2, [2, 3, 128]), (8, 1, [4, 24, 5])])
def test_generic_blocks_match_oracle(block, axis, shape):
    info, x, y, s, y_ref, s_ref = _quantize_both(F32, shape, block, axis, dfgpu.BSQ_AUTO, special=True, seed=21)
    assert np.array_equal(s, s_ref)
    assert np.array_equal(y, y_ref)


def test_strided_input_uses_generic_kernel():
    # X is a [64, 64] window of a [64, 80] buffer
    info, x, y, s, y_ref, s_ref = _quantize_both(BF16, [64, 64], 32, 1, dfgpu.BSQ_AUTO, seed=4)
    assert info.kernel == dfgpu.BSQ_ROW32
    import gpu_util as g
    full = _make_x(BF16, [64, 80], 4)
    xd = tensor(BF16, [64, 64], [80, 1])
    yd, sd = tensor(E4M3, [64, 64]), tensor(E8M0, [64, 2])
    y_ref = np.zeros(64 * 64, dtype=np.uint8)
    s_ref = np.zeros(128, dtype=np.uint8)
    oracle.block_scale_quantize(xd, full, yd, y_ref, sd, s_ref, 32, 1)
    p = dfgpu.BsqParams()
    p.x, p.y, p.scale, p.block_size, p.axis = xd, yd, sd, 32, 1
    assert dfgpu.query("block_scale_quantize", p).kernel == dfgpu.BSQ_GENERIC
    dx, dy, ds = g.to_device(full), g.device_zeros(64 * 64), g.device_zeros(128)
    dfgpu.block_scale_quantize(p, g.ptr(dx), g.ptr(dy), g.ptr(ds))
    assert np.array_equal(g.to_host(dy, np.uint8), y_ref) and np.array_equal(g.to_host(ds, np.uint8), s_ref)


@pytest.mark.parametrize("kernel", [dfgpu.BSQ_GENERIC, dfgpu.BSQ_ROW32])
def test_reordered_scale_with_padding_slots(kernel):
    # the reference's 128x32 case: logical scale [128,1] inside an F8_128x4 [128,4] tensor
    info, x, y, s, y_ref, s_ref = _quantize_both(F32, [128, 32], 32, 1, kernel, scale_dims=[128, 4], scale_strides=[4, 1],
                                                 reorder=REORDER_F8_128x4, seed=8)
    assert info.launches == 2  # fill + quantize
    assert np.array_equal(s, s_ref) and np.array_equal(y, y_ref)
    assert np.count_nonzero(s == 0x7f) >= 128 * 3


@pytest.mark.parametrize("kernel", [dfgpu.BSQ_GENERIC, dfgpu.BSQ_ROW32])
def test_reordered_scale_full_grid(kernel):
    info, x, y, s, y_ref, s_ref = _quantize_both(BF16, [256, 256], 32, 1, kernel, scale_dims=[256, 8], scale_strides=[8, 1],
                                                 reorder=REORDER_F8_128x4, seed=12, special=True)
    assert np.array_equal(s, s_ref) and np.array_equal(y, y_ref)


@pytest.mark.parametrize("kernel", [dfgpu.BSQ_GENERIC, dfgpu.BSQ_COL32])
def test_transposed_reordered_scale(kernel):
    # B-style operand [K, N], blocks along K, scale [K/32, N] stored with N as the 128-row axis
    info, x, y, s, y_ref, s_ref = _quantize_both(BF16, [128, 256], 32, 0, kernel, scale_dims=[4, 256], scale_strides=[1, 4],
                                                 reorder=REORDER_F8_128x4, seed=14, special=True)
    assert np.array_equal(s, s_ref) and np.array_equal(y, y_ref)


def test_reference_reordered_known_answer():
    import gpu_util as g
    x = np.full((128, 32), 448.0, dtype=np.float32)
    x[32] = 224.0
    x[127] = 112.0
    p = dfgpu.BsqParams()
    p.x, p.y = tensor(F32, [128, 32]), tensor(E4M3, [128, 32])
    p.scale = tensor(E8M0, [128, 4], [4, 1], REORDER_F8_128x4)
    p.block_size, p.axis = 32, 1
    dx, dy, ds = g.to_device(x), g.device_zeros(128 * 32), g.device_zeros(512)
    dfgpu.block_scale_quantize(p, g.ptr(dx), g.ptr(dy), g.ptr(ds))
    y, s = g.to_host(dy, np.uint8), g.to_host(ds, np.uint8)
    assert np.all(y == 0x7e)
    off = oracle.lib().dfo_f8_128x4_offset
    for m in range(128):
        for k in range(4):
            expected = 126 if (k == 0 and m == 32) else 125 if (k == 0 and m == 127) else 127
            assert s[off(0, m, k, 128, 4)] == expected


def test_exhaustive_e4m3_encoder_sweep():
    """All 2^32 f32 bit patterns: the production encoder equals the literal candidate search."""
    import torch
    result = torch.zeros(2, dtype=torch.int64, device="cuda")
    for chunk in range(16):
        dfgpu.selfcheck_e4m3(chunk << 28, 1 << 28, result.data_ptr())
    torch.cuda.synchronize()
    bad, witness = result.cpu().tolist()
    assert bad == 0, f"{bad} disagreements, e.g. bits {witness - 1:#010x}"


def test_encoder_matches_oracle_on_boundaries_and_samples():
    import gpu_util as g
    codes = np.arange(256, dtype=np.uint8)
    lib = oracle.lib()
    decoded = np.array([lib.dfo_decode_e4m3(int(c)) for c in codes if (c & 0x7f) != 0x7f], dtype=np.float32)
    mids = ((decoded[:-1].astype(np.float64) + decoded[1:].astype(np.float64)) / 2).astype(np.float32)
    around = np.concatenate([decoded, mids, np.nextafter(mids, np.float32(np.inf)), np.nextafter(mids, np.float32(-np.inf)),
                             np.nextafter(decoded, np.float32(np.inf)), np.nextafter(decoded, np.float32(-np.inf))])
    bits = synthetic.raw_u64(77, 1, 1 << 20).astype(np.uint32)
    samples = np.concatenate([around, bits.view(np.float32),
                              np.array([0.0, -0.0, np.inf, -np.inf, np.nan, -np.nan, 1e-45, -1e-45, 2.0 ** -10, -(2.0 ** -10)], dtype=np.float32)])
    expected = oracle.encode_e4m3_many(samples)
    dv, dc = g.to_device(samples), g.device_zeros(samples.size)
    dfgpu.debug_encode_e4m3(g.ptr(dv), g.ptr(dc), samples.size)
    assert np.array_equal(g.to_host(dc, np.uint8), expected)


def test_scale_rule_for_every_16bit_amax():
    """All 65,536 bf16 and f16 patterns as block amax go through the E8M0 rule bit-exactly."""
    import gpu_util as g
    patterns = np.arange(1 << 16, dtype=np.uint16)
    bf = synthetic.bf16_bits_to_f32(patterns)
    with np.errstate(invalid="ignore"):
        half = patterns.view(np.float16).astype(np.float32)
    amax = np.abs(np.concatenate([bf, half])).astype(np.float32)
    expected = oracle.block_scale_code_many(amax)
    da, dc = g.to_device(amax), g.device_zeros(amax.size)
    dfgpu.debug_scale_codes(g.ptr(da), g.ptr(dc), amax.size)
    assert np.array_equal(g.to_host(dc, np.uint8), expected)


@pytest.mark.parametrize("ydtype", [F32, F16, BF16])
@pytest.mark.parametrize("blocks,shape,kernel", [([1, 32], [64, 128], dfgpu.BSD_PACKED), ([32, 1], [64, 128], dfgpu.BSD_PACKED),
                                                 ([1, 32], [64, 128], dfgpu.BSD_GENERIC), ([2], [3, 4], dfgpu.BSD_GENERIC),
                                                 ([4, 2], [2, 8, 6], dfgpu.BSD_GENERIC)])
def test_dequantize_matches_oracle(ydtype, blocks, shape, kernel):
    import gpu_util as g
    count = int(np.prod(shape))
    codes = (synthetic.raw_u64(5, 2, count) & np.uint64(0xff)).astype(np.uint8)
    scale_dims = list(shape)
    for i, b in enumerate(blocks):
        axis = len(shape) - len(blocks) + i
        scale_dims[axis] = shape[axis] // b
    scount = int(np.prod(scale_dims))
    scales = (100 + synthetic.raw_u64(5, 3, scount) % np.uint64(60)).astype(np.uint8)
    scales[::17] = 0xff
    scales[1::19] = 0
    scales[2::23] = 254
    xd, sd, yd = tensor(E4M3, shape), tensor(E8M0, scale_dims), tensor(ydtype, shape)
    width = dfgpu.DTYPE_BYTES[ydtype]
    ref = np.zeros(count * width, dtype=np.uint8)
    oracle.block_scale_dequantize(xd, codes, sd, scales, yd, ref, blocks)
    p = dfgpu.BsdParams()
    p.x, p.scale, p.y = xd, sd, yd
    for i, b in enumerate(blocks):
        p.block[i] = b
    p.block_count, p.kernel = len(blocks), kernel
    assert dfgpu.query("block_scale_dequantize", p).kernel == kernel
    dx, ds, dy = g.to_device(codes), g.to_device(scales), g.device_zeros(count * width)
    dfgpu.block_scale_dequantize(p, g.ptr(dx), g.ptr(ds), g.ptr(dy))
    out = g.to_host(dy, np.uint8)
    if ydtype == F32:
        a, b = out.view(np.uint32), ref.view(np.uint32)
    else:
        a, b = out.view(np.uint16), ref.view(np.uint16)
    nan_a = np.isnan(out.view(NP_OF[ydtype])) if ydtype != BF16 else np.isnan(synthetic.bf16_bits_to_f32(a))
    nan_b = np.isnan(ref.view(NP_OF[ydtype])) if ydtype != BF16 else np.isnan(synthetic.bf16_bits_to_f32(b))
    assert np.array_equal(nan_a, nan_b)
    assert np.array_equal(a[~nan_a], b[~nan_b])


def test_full_size_quantize_properties():
    """The benchmark's 4096x4096 bf16 operands: A-style and B-style. Checked against the
    oracle on a slab, and through size-independent properties on the whole matrix:
    every |x / scale| <= 448 unless saturated, scale code == rule(amax), decode(code)*scale
    within half an E4M3 step of x."""
    import gpu_util as g
    n = 4096
    seed = 20261125 + 3
    values = synthetic.normal(seed, 1, n * n)
    values = np.where(synthetic.outlier_mask(seed, 1, n * n), values * 64.0, values).astype(np.float32)
    bits = synthetic.to_bf16_bits(values).reshape(n, n)
    x32 = synthetic.bf16_bits_to_f32(bits)
    dx = g.to_device(bits)
    for axis, kernel in ((1, dfgpu.BSQ_ROW32), (0, dfgpu.BSQ_COL32)):
        sdims = [n, n // 32] if axis == 1 else [n // 32, n]
        p = dfgpu.BsqParams()
        p.x, p.y, p.scale, p.block_size, p.axis = tensor(BF16, [n, n]), tensor(E4M3, [n, n]), tensor(E8M0, sdims), 32, axis
        assert dfgpu.query("block_scale_quantize", p).kernel == kernel
        dy, ds = g.device_zeros(n * n), g.device_zeros(n * n // 32)
        dfgpu.block_scale_quantize(p, g.ptr(dx), g.ptr(dy), g.ptr(ds))
        y = g.to_host(dy, np.uint8, (n, n))
        s = g.to_host(ds, np.uint8, sdims)
        blocks = np.abs(x32).reshape(n, n // 32, 32).max(axis=2) if axis == 1 else np.abs(x32).reshape(n // 32, 32, n).max(axis=1)
        assert np.array_equal(s, oracle.block_scale_code_many(blocks))
        # oracle slab: 64 rows (A) or 64 columns' worth of blocks via the first 64 K-rows (B)
        rows = 64
        sub = np.ascontiguousarray(bits[:rows])
        y_ref = np.zeros(rows * n, dtype=np.uint8)
        s_rows = rows if axis == 1 else rows // 32
        s_ref = np.zeros(s_rows * (n // 32 if axis == 1 else n), dtype=np.uint8)
        oracle.block_scale_quantize(tensor(BF16, [rows, n]), sub, tensor(E4M3, [rows, n]), y_ref,
                                    tensor(E8M0, [rows, n // 32] if axis == 1 else [rows // 32, n]), s_ref, 32, axis)
        assert np.array_equal(y[:rows].reshape(-1), y_ref)
        assert np.array_equal(s[:s_rows].reshape(-1), s_ref)
        # round trip through the dequantize kernel
        q = dfgpu.BsdParams()
        q.x, q.scale, q.y = tensor(E4M3, [n, n]), tensor(E8M0, sdims), tensor(F32, [n, n])
        q.block[0], q.block[1], q.block_count = (1, 32, 2) if axis == 1 else (32, 1, 2)
        dz = g.device_zeros(n * n * 4)
        dfgpu.block_scale_dequantize(q, g.ptr(dy), g.ptr(ds), g.ptr(dz))
        z = g.to_host(dz, np.float32, (n, n))
        scale_full = np.repeat(np.ldexp(1.0, s.astype(np.int32) - 127), 32, axis=1 if axis == 1 else 0)
        assert np.all(np.abs(z - x32) <= scale_full * 16.0 + 0)  # coarse: half a top-binade step (32/2)
        rel = np.abs(z - x32) <= np.maximum(np.abs(x32) * 0.0625, scale_full * 2.0 ** -10)
        assert np.all(rel)
