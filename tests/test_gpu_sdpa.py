"""SDPA forward kernels (row-wise general kernel, paged decode) against the CPU oracle."""
import numpy as np
import pytest

import gpu_util as g
import oracle
from deepforge_b200 import dfgpu, synthetic
from deepforge_b200.dfgpu import BF16, F32, I32, tensor

pytestmark = pytest.mark.gpu
INF = float("inf")


def close_f32(actual, expected, tol=8e-5):
    finite = np.isfinite(expected)
    assert np.array_equal(actual[~finite], expected[~finite])
    assert np.all(np.abs(actual[finite] - expected[finite]) <= tol * (1 + np.abs(expected[finite])))


def close_bf16(actual, expected):
    assert np.all(np.abs(actual - expected) <= 1e-2 + 2e-2 * np.abs(expected))


def both(dtype, q_dims, k_dims, v_dims, s_kv, scale, kernel, seq=None, tables=None, stats=True, seed=5, q_step=1, bh_range=None,
         bias_dims=None, sink=False, block_mask=None, compact=None, **flags):
    """Run oracle (f32 restatement on dtype-rounded inputs) and the GPU kernel on the same data.
    compact: (slots per batch entry, K offsets as int64, V offsets as int32) when `tables` are compact 1-D page tables."""
    b, hq, sq, _ = q_dims
    o_dims = [b, hq, sq, v_dims[3]]
    row_dims = [b, hq, sq, 1]
    raw = [synthetic.normal(seed, i + 1, int(np.prod(d))) for i, d in enumerate((q_dims, k_dims, v_dims))]
    rounded = [synthetic.round_to_bf16(a) if dtype == BF16 else a for a in raw]
    host = [synthetic.to_bf16_bits(a) if dtype == BF16 else a for a in raw]

    def fill(params, t):
        params.q, params.k, params.v, params.o = (tensor(t, d) for d in (q_dims, k_dims, v_dims, o_dims))
        if stats:
            params.stats = params.max = params.sum_exp = tensor(F32, row_dims)
        params.attn_scale, params.s_kv = scale, s_kv
        if seq is not None:
            params.padding_mask = 1
            params.seq_q = params.seq_kv = tensor(I32, [b, 1, 1, 1])
        if tables is not None and compact is None:
            params.page_table_k = tensor(I32, [b, 1, tables[0].shape[1], 1])
            params.page_table_v = tensor(I32, [b, 1, tables[1].shape[1], 1])
        if compact is not None:
            params.page_table_k = params.page_table_v = tensor(I32, [b, 1, compact[0], 1])
            params.page_offsets_k, params.page_offsets_v = tensor(dfgpu.I64, [b + 1, 1, 1, 1]), tensor(I32, [b + 1, 1, 1, 1])
        if bias_dims is not None:
            params.bias = tensor(F32, bias_dims)
        if sink:
            params.sink = tensor(F32, [1, hq, 1, 1])
        if block_mask is not None:
            params.block_mask = tensor(dfgpu.U8, list(block_mask.shape))
        for key, value in flags.items():
            setattr(params, key, value)

    bias = synthetic.normal(seed, 9, int(np.prod(bias_dims))) if bias_dims is not None else None
    sink_values = (2.0 * synthetic.normal(seed, 10, hq)).astype(np.float32) if sink else None
    op = oracle.SdpaParams()
    fill(op, F32)
    o_ref = np.full(int(np.prod(o_dims)), -99.0, dtype=np.float32)
    rows_ref = [np.full(int(np.prod(row_dims)), -99.0, dtype=np.float32) for _ in range(3)]
    seq_arrays = [None, None] if seq is None else [np.asarray(s, dtype=np.int32) for s in seq]
    table_arrays = [None, None] if tables is None else [np.ascontiguousarray(t, dtype=np.int32) for t in tables]
    lo, hi = bh_range if bh_range else (0, b * hq)
    offset_arrays = [None, None] if compact is None else [np.ascontiguousarray(compact[1], dtype=np.int64), np.ascontiguousarray(compact[2], dtype=np.int32)]
    oracle.sdpa_forward(op, rounded + [o_ref] + (rows_ref if stats else [None] * 3) + seq_arrays + table_arrays + [bias, sink_values, block_mask] + offset_arrays, lo, hi, q_step)

    gp = dfgpu.SdpaParams()
    fill(gp, dtype)
    gp.kernel = kernel
    info = dfgpu.query("sdpa_forward", gp)
    dev = [g.to_device(a) for a in host]
    do = g.device_zeros(o_ref.size * dfgpu.DTYPE_BYTES[dtype])
    drows = [g.device_zeros(rows_ref[0].size * 4) for _ in range(3)] if stats else [None] * 3
    dseq = [g.to_device(a) if a is not None else None for a in seq_arrays]
    dtab = [g.to_device(a) if a is not None else None for a in table_arrays]
    scratch = g.device_zeros(info.scratch_bytes) if info.scratch_bytes else None
    dbias = g.to_device(bias) if bias is not None else None
    dsink = g.to_device(sink_values) if sink else None
    dmask = g.to_device(block_mask) if block_mask is not None else None
    doff = [g.to_device(a) if a is not None else None for a in offset_arrays]
    dfgpu.sdpa_forward(gp, [g.ptr(t) for t in dev + [do] + drows + dseq + dtab + [dbias, dsink, dmask] + doff], scratch=g.ptr(scratch))
    if dtype == BF16:
        o = synthetic.bf16_bits_to_f32(g.to_host(do, np.uint16))
    else:
        o = g.to_host(do, np.float32)
    rows = [g.to_host(d, np.float32) for d in drows] if stats else None
    return info, o.reshape(o_dims), o_ref.reshape(o_dims), rows, rows_ref


def test_rowwise_gqa_padding_windows_stats_f32():
    for bottom_right in (0, 1):
        info, o, o_ref, rows, rows_ref = both(F32, [2, 4, 5, 8], [2, 2, 7, 8], [2, 1, 7, 6], 7, 0.3, dfgpu.SDPA_ROWWISE,
                                              seq=([5, 3], [7, 4]), has_right_bound=1, right_bound=1, has_left_bound=1,
                                              left_bound=3, bottom_right=bottom_right)
        close_f32(o, o_ref)
        for a, r in zip(rows, rows_ref):
            close_f32(a, r)
        assert np.all(o[1, :, 3:] == 0.0) and np.all(rows[0].reshape(2, 4, 5)[1, :, 3:] == -INF)


@pytest.mark.parametrize("bias_dims", [None, [2, 6, 5, 7], [1, 1, 5, 7], [1, 6, 1, 7], [2, 1, 5, 1]])
@pytest.mark.parametrize("alibi", [0, 1])
def test_rowwise_bias_and_alibi(bias_dims, alibi):
    """score = attn_scale * dot + bias (extent-1 axes broadcast) + (kv - q) * slope(head); six heads, so the slopes of
    heads 4 and 5 come from the second formula (lib/Compiler/SequenceGraph.cpp:1748-1778)."""
    if bias_dims is None and not alibi:
        pytest.skip("covered by the other tests")
    info, o, o_ref, rows, rows_ref = both(F32, [2, 6, 5, 8], [2, 3, 7, 8], [2, 3, 7, 6], 7, 0.4, dfgpu.SDPA_AUTO, seq=([5, 4], [7, 6]),
                                          bias_dims=bias_dims, alibi_mask=alibi, has_right_bound=1, right_bound=2)
    assert info.kernel == dfgpu.SDPA_ROWWISE
    close_f32(o, o_ref)
    for a, r in zip(rows, rows_ref):
        close_f32(a, r)


@pytest.mark.parametrize("padded", [False, True])
def test_rowwise_sink_token(padded):
    """One extra logit per head: the row maximum starts from it and the row sum from exp(sink - max); it adds nothing to O
    (lib/Compiler/SequenceGraph.cpp:2256-2288). With padding, the rows past SEQ_LEN_Q keep Max = sink, Sum_exp = 1, O = 0."""
    seq = ([5, 3], [7, 4]) if padded else None
    info, o, o_ref, rows, rows_ref = both(F32, [2, 4, 5, 8], [2, 2, 7, 8], [2, 2, 7, 6], 7, 0.5, dfgpu.SDPA_AUTO, seq=seq, sink=True,
                                          has_right_bound=1, right_bound=1, bias_dims=[1, 4, 5, 7])
    assert info.kernel == dfgpu.SDPA_ROWWISE
    close_f32(o, o_ref)
    for a, r in zip(rows, rows_ref):
        close_f32(a, r)
    if padded:
        assert np.all(o[1, :, 3:] == 0.0) and np.all(rows[2].reshape(2, 4, 5)[1, :, 3:] == 1.0)


def test_rowwise_block_mask():
    """One bit per 128 x 128 score tile (lib/Compiler/SequenceGraph.cpp:2059-2088): 2 x 3 tiles per head here; head 1 of batch 0
    has its second query tile switched off entirely, so those rows are fully masked (O = 0, Stats = -inf, Sum_exp = 0)."""
    mask = np.array([[[[0b101], [0b011]], [[0b110], [0b000]]]], dtype=np.uint8)  # [B=1, H=2, 2 query tiles, 1 byte]
    info, o, o_ref, rows, rows_ref = both(F32, [1, 2, 200, 8], [1, 1, 300, 8], [1, 1, 300, 8], 300, 0.4, dfgpu.SDPA_AUTO, block_mask=mask,
                                          has_right_bound=1, right_bound=150)
    assert info.kernel == dfgpu.SDPA_ROWWISE
    close_f32(o, o_ref)
    for a, r in zip(rows, rows_ref):
        close_f32(a, r)
    assert np.all(o[0, 1, 128:] == 0.0) and np.all(rows[0].reshape(1, 2, 200)[0, 1, 128:] == -INF) and np.all(rows[2].reshape(1, 2, 200)[0, 1, 128:] == 0.0)
    assert np.any(o[0, 0, 128:] != 0.0)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("kind", ["probability", "mask", "broadcast_mask"])
def test_rowwise_dropout(kind, dtype):
    """Dropout weights V with (p * mask) * scale and leaves Stats / Max / Sum_exp alone: probability dropout (the Bernoulli stream over the flat
    score index, RNG_DUMP bit for bit the oracle's at every position, masked ones too) and a caller's mask with its scale (full size, and
    broadcast over batch and query rows), with grouped heads, padding and a causal bound; the tensor-core kernels refuse dropout."""
    b, hq, hk, sq, skv, d = 2, 6, 3, 37, 70, 16
    q_dims, k_dims, v_dims, o_dims, row_dims = [b, hq, sq, d], [b, hk, skv, d], [b, hk, skv, d], [b, hq, sq, d], [b, hq, sq, 1]
    raw = [synthetic.normal(21, i + 1, int(np.prod(dims))) for i, dims in enumerate((q_dims, k_dims, v_dims))]
    rounded = [synthetic.round_to_bf16(a) if dtype == BF16 else a for a in raw]
    host = [synthetic.to_bf16_bits(a) if dtype == BF16 else a for a in raw]
    seq_q, seq_kv = np.array([sq, 20], np.int32), np.array([skv - 5, skv], np.int32)
    mask_dims = [b, hq, sq, skv] if kind == "mask" else [1, hq, 1, skv]
    mask = (synthetic.uniform(21, 7, int(np.prod(mask_dims)), 0.0, 1.0) < 0.75).astype(np.float32)
    mask_scale = np.array([1.0 / 0.75], np.float32)
    seed, offset = np.array([-977], np.int64), np.array([1 << 33], np.int64)

    def fill(params, t):
        params.q, params.k, params.v, params.o = (tensor(t, dims) for dims in (q_dims, k_dims, v_dims, o_dims))
        params.stats = params.max = params.sum_exp = tensor(F32, row_dims)
        params.attn_scale, params.s_kv, params.padding_mask, params.has_right_bound, params.right_bound = 0.25, skv, 1, 1, 3
        params.seq_q = params.seq_kv = tensor(I32, [b, 1, 1, 1])
        if kind == "probability":
            params.dropout_kind, params.dropout_probability, params.rng_dump = 1, 0.3, tensor(F32, [b, hq, sq, skv])
        else:
            params.dropout_kind, params.dropout_mask = 2, tensor(F32, mask_dims)

    op = oracle.SdpaParams()
    fill(op, F32)
    o_ref = np.full(int(np.prod(o_dims)), -99.0, np.float32)
    rows_ref = [np.full(int(np.prod(row_dims)), -99.0, np.float32) for _ in range(3)]
    dump_ref = np.full(b * hq * sq * skv, -1.0, np.float32)
    tail = [None, None, seed, offset, dump_ref] if kind == "probability" else [mask, mask_scale, None, None, None]
    oracle.sdpa_forward(op, rounded + [o_ref] + rows_ref + [seq_q, seq_kv] + [None] * 7 + tail)

    gp = dfgpu.SdpaParams()
    fill(gp, dtype)
    if kind != "probability":
        gp.dropout_scale = tensor(F32, [1, 1, 1, 1])
    else:
        gp.seed = gp.offset = tensor(dfgpu.I64, [1, 1, 1, 1])
    gp.kernel = dfgpu.SDPA_AUTO
    info = dfgpu.query("sdpa_forward", gp)
    assert info.kernel == dfgpu.SDPA_ROWWISE
    dev = [g.to_device(a) for a in host]
    do = g.device_zeros(o_ref.size * dfgpu.DTYPE_BYTES[dtype])
    drows = [g.device_zeros(rows_ref[0].size * 4) for _ in range(3)]
    ddump = g.device_zeros(dump_ref.size * 4, 0x3C)
    extra = [None, None, g.to_device(seed), g.to_device(offset), ddump] if kind == "probability" else [g.to_device(mask), g.to_device(mask_scale), None, None, None]
    dfgpu.sdpa_forward(gp, [g.ptr(t) for t in dev + [do] + drows + [g.to_device(seq_q), g.to_device(seq_kv)] + [None] * 7 + extra])
    o = synthetic.bf16_bits_to_f32(g.to_host(do, np.uint16)) if dtype == BF16 else g.to_host(do, np.float32)
    (close_bf16 if dtype == BF16 else close_f32)(o, o_ref)
    for got, want in zip(drows, rows_ref):
        got = g.to_host(got, np.float32)
        live = np.isfinite(want)
        assert np.array_equal(np.isfinite(got), live) and np.allclose(got[live], want[live], rtol=1e-4, atol=1e-5)
    if kind == "probability":
        dump = g.to_host(ddump, np.float32)
        assert np.array_equal(dump, dump_ref) and 0.6 < float(dump.mean()) < 0.8
    # the same attention without dropout differs, and its statistics do not
    gp.dropout_kind = 0
    gp.rng_dump = dfgpu.Tensor()
    do2, drows2 = g.device_zeros(o_ref.size * dfgpu.DTYPE_BYTES[dtype]), [g.device_zeros(rows_ref[0].size * 4) for _ in range(3)]
    dfgpu.sdpa_forward(gp, [g.ptr(t) for t in dev + [do2] + drows2 + [g.to_device(seq_q), g.to_device(seq_kv)] + [None, None]])
    assert not np.array_equal(g.to_host(do2, np.uint8), g.to_host(do, np.uint8))
    assert np.array_equal(g.to_host(drows2[0], np.uint32), g.to_host(drows[0], np.uint32))
    gp.dropout_kind = 1 if kind == "probability" else 2
    for kernel in (dfgpu.SDPA_UMMA, dfgpu.SDPA_PAGED_DECODE):
        gp.kernel = kernel
        with pytest.raises(dfgpu.DfgpuError):
            dfgpu.query("sdpa_forward", gp)


def test_bias_keeps_the_tensor_core_kernels_out():
    params = dfgpu.SdpaParams()
    params.q = params.k = params.v = params.o = tensor(BF16, [1, 2, 256, 128])
    params.attn_scale, params.s_kv = 0.1, 256
    assert dfgpu.query("sdpa_forward", params).kernel == dfgpu.SDPA_UMMA
    params.bias = tensor(F32, [1, 1, 256, 256])
    assert dfgpu.query("sdpa_forward", params).kernel == dfgpu.SDPA_ROWWISE
    params.kernel = dfgpu.SDPA_UMMA
    with pytest.raises(dfgpu.DfgpuError) as error:
        dfgpu.query("sdpa_forward", params)
    assert error.value.code == 20


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_rowwise_causal_medium(dtype):
    info, o, o_ref, rows, rows_ref = both(dtype, [2, 4, 96, 128], [2, 4, 96, 128], [2, 4, 96, 128], 96, 128 ** -0.5,
                                          dfgpu.SDPA_ROWWISE, has_right_bound=1, right_bound=0)
    if dtype == F32:
        close_f32(o, o_ref)
        close_f32(rows[0], rows_ref[0])
    else:
        close_bf16(o, o_ref)
        close_f32(rows[0], rows_ref[0], 2e-3)


def _reference_paged_case():
    q = np.array([0.2, -0.3, -0.5, 0.4], dtype=np.float32)
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


def test_reference_paged_case_and_invalid_pages():
    q, k, v, page_k, page_v, kc, vc = _reference_paged_case()
    p = dfgpu.SdpaParams()
    p.q, p.o = tensor(F32, [2, 1, 1, 2]), tensor(F32, [2, 1, 1, 2])
    p.k = p.v = tensor(F32, [4, 1, 2, 2])
    p.seq_q = p.seq_kv = tensor(I32, [2, 1, 1, 1])
    p.page_table_k = p.page_table_v = tensor(I32, [2, 1, 2, 1])
    p.attn_scale, p.padding_mask, p.s_kv = 0.5, 1, 3
    seq_q, seq_kv = np.array([1, 1], dtype=np.int32), np.array([3, 3], dtype=np.int32)
    # contiguous reference through the oracle
    op = oracle.SdpaParams()
    op.q, op.o = tensor(F32, [2, 1, 1, 2]), tensor(F32, [2, 1, 1, 2])
    op.k = op.v = tensor(F32, [2, 1, 3, 2])
    op.attn_scale, op.s_kv = 0.5, 3
    ref = np.zeros(4, dtype=np.float32)
    oracle.sdpa_forward(op, [q, k, v, ref] + [None] * 7)
    dev = [g.to_device(a) for a in (q, kc, vc)]
    do = g.device_zeros(16)
    dsq, dskv = g.to_device(seq_q), g.to_device(seq_kv)
    for tables, check in (((page_k, page_v), lambda o: close_f32(o, ref)),
                          ((np.array([-1, 99, 3, 1], dtype=np.int32), np.array([-1, 99, 0, 2], dtype=np.int32)),
                           lambda o: (o[0] == 0.0 and o[1] == 0.0) or pytest.fail("invalid pages must read as zero"))):
        dt = [g.to_device(t) for t in tables]
        dfgpu.sdpa_forward(p, [g.ptr(t) for t in dev + [do]] + [0, 0, 0, g.ptr(dsq), g.ptr(dskv), g.ptr(dt[0]), g.ptr(dt[1])])
        check(g.to_host(do, np.float32))


def _paged_inputs(batch, hq, hkv, pages, block, max_len, seed, lengths=None):
    table_len = (max_len + block - 1) // block
    if lengths is None:
        lengths = synthetic.integers(seed, 50, batch, max(1, max_len // 16), max_len)
    tk = np.stack([synthetic.permutation_prefix(seed, 100 + i, pages, table_len) for i in range(batch)])
    tv = np.stack([synthetic.permutation_prefix(seed, 200 + i, pages, table_len) for i in range(batch)])
    return np.asarray(lengths, dtype=np.int32), tk.astype(np.int32), tv.astype(np.int32)


@pytest.mark.parametrize("kernel", [dfgpu.SDPA_PAGED_DECODE, dfgpu.SDPA_PAGED_DECODE_UMMA])
@pytest.mark.parametrize("group,block", [(4, 64), (1, 16), (8, 128), (2, 256)])
def test_paged_decode_matches_oracle(group, block, kernel):
    if kernel == dfgpu.SDPA_PAGED_DECODE_UMMA and block > 128:
        pytest.skip("the TMA kernel takes pages of at most 128 tokens")
    batch, hkv, pages, max_len = 5, 2, 64, 700
    hq = hkv * group
    lengths, tk, tv = _paged_inputs(batch, hq, hkv, pages, block, max_len, seed=31 + group)
    lengths[0] = max_len
    lengths[1] = 1
    tk[2, 1] = -1          # invalid page ids read as zeros
    tv[2, 0] = pages + 7
    info, o, o_ref, rows, rows_ref = both(BF16, [batch, hq, 1, 128], [pages, hkv, block, 128], [pages, hkv, block, 128], max_len,
                                          128 ** -0.5, kernel, seq=([1] * batch, lengths), tables=(tk, tv))
    assert info.kernel == kernel and info.scratch_bytes > 0 and info.launches == 2
    close_bf16(o, o_ref)
    for a, r in zip(rows, rows_ref):
        close_f32(a, r, 1e-3)
    # and the general kernel agrees on the same paged inputs
    info2, o2, _, _, _ = both(BF16, [batch, hq, 1, 128], [pages, hkv, block, 128], [pages, hkv, block, 128], max_len,
                              128 ** -0.5, dfgpu.SDPA_ROWWISE, seq=([1] * batch, lengths), tables=(tk, tv))
    close_bf16(o2, o_ref)


def _compact(lengths, tk, tv, block):
    """The same page assignments stored back to back: each entry keeps the slots its length needs."""
    slots = (np.asarray(lengths, dtype=np.int64) + block - 1) // block
    offsets = np.concatenate([[0], np.cumsum(slots)])
    pack = lambda t: np.concatenate([t[i, :slots[i]] for i in range(len(slots))] + [np.zeros(0, np.int32)]).astype(np.int32)
    return pack(tk), pack(tv), offsets


@pytest.mark.parametrize("kernel", [dfgpu.SDPA_ROWWISE, dfgpu.SDPA_PAGED_DECODE, dfgpu.SDPA_PAGED_DECODE_UMMA])
@pytest.mark.parametrize("group,block", [(4, 64), (1, 16), (8, 128)])
def test_compact_page_tables_match_oracle_and_strided_tables(group, block, kernel):
    """Compact (ragged batch-prefix) page tables, K offsets INT64 and V offsets INT32, exact allocation: every kernel gives
    what it gives for the strided tables of the same pages, and what the oracle gives (lib/Compiler/SequenceGraph.cpp:1811-1864)."""
    batch, hkv, pages, max_len = 5, 2, 64, 700
    hq = hkv * group
    lengths, tk, tv = _paged_inputs(batch, hq, hkv, pages, block, max_len, seed=61 + group)
    lengths[0], lengths[1], lengths[3] = max_len, 1, 0
    tk[2, 1] = -1          # invalid page ids still read as zeros
    ck, cv, offsets = _compact(lengths, tk, tv, block)
    dims = ([batch, hq, 1, 128], [pages, hkv, block, 128], [pages, hkv, block, 128])
    info, o, o_ref, rows, rows_ref = both(BF16, *dims, max_len, 128 ** -0.5, kernel, seq=([1] * batch, lengths), tables=(ck, cv), compact=(tk.shape[1], offsets, offsets))
    assert info.kernel == kernel and info.scratch_bytes >= 256 and info.launches == (2 if kernel == dfgpu.SDPA_ROWWISE else 3)
    close_bf16(o, o_ref)
    _, o_strided, _, rows_strided, _ = both(BF16, *dims, max_len, 128 ** -0.5, kernel, seq=([1] * batch, lengths), tables=(tk, tv))
    assert np.array_equal(o, o_strided)
    for a, r in zip(rows, rows_strided):
        assert np.array_equal(a, r, equal_nan=True)


@pytest.mark.parametrize("kernel", [dfgpu.SDPA_ROWWISE, dfgpu.SDPA_PAGED_DECODE, dfgpu.SDPA_PAGED_DECODE_UMMA])
@pytest.mark.parametrize("which,offsets", [(0, [0, 2, 3, 20, 20, 21]), (1, [1, 11, 12, 23, 23, 34]), (0, [0, 11, 5, 23, 23, 34]), (1, [0, 11, 12, 23, 23, 1 << 20])])
def test_compact_page_table_with_a_bad_prefix_reads_as_invalid_pages(kernel, which, offsets):
    """A prefix that breaks the reference's runtime rule (lib/Runtime/Executable.cpp:619-716: segment shorter than the
    sequence needs, non-zero start, decreasing, past the storage bound) is found on the device: the launch leaves 601 (K)
    or 602 (V) in the device status, the table is never read (so nothing is fetched out of bounds) and its pages read
    as invalid. The context stays usable."""
    batch, hkv, pages, block, max_len = 5, 2, 64, 64, 700
    lengths, tk, tv = _paged_inputs(batch, 8, hkv, pages, block, max_len, seed=71)
    lengths[:] = [700, 1, 700, 0, 650]
    ck, cv, good = _compact(lengths, tk, tv, block)
    assert good.tolist() == [0, 11, 12, 23, 23, 34]
    p = dfgpu.SdpaParams()
    p.q = p.o = tensor(BF16, [batch, 8, 1, 128])
    p.k = p.v = tensor(BF16, [pages, hkv, block, 128])
    p.seq_q = p.seq_kv = tensor(I32, [batch, 1, 1, 1])
    p.page_table_k = p.page_table_v = tensor(I32, [batch, 1, tk.shape[1], 1])
    p.page_offsets_k, p.page_offsets_v = tensor(dfgpu.I64, [batch + 1, 1, 1, 1]), tensor(I32, [batch + 1, 1, 1, 1])
    p.attn_scale, p.padding_mask, p.s_kv, p.kernel = 128 ** -0.5, 1, max_len, kernel
    info = dfgpu.query("sdpa_forward", p)
    host = [synthetic.to_bf16_bits(synthetic.normal(7, i + 1, n)) for i, n in enumerate((batch * 8 * 128, pages * hkv * block * 128, pages * hkv * block * 128))]
    dev = [g.to_device(a) for a in host]
    do = g.device_zeros(batch * 8 * 128 * 2, 0x55)
    ok, ov = (np.array(offsets), good) if which == 0 else (good, np.array(offsets))
    extra = [g.to_device(np.ones(batch, dtype=np.int32)), g.to_device(lengths), g.to_device(ck), g.to_device(cv)]
    doff = [g.to_device(ok.astype(np.int64)), g.to_device(ov.astype(np.int32))]
    scratch = g.device_zeros(info.scratch_bytes)
    dfgpu.sdpa_forward(p, [g.ptr(t) for t in dev + [do]] + [0, 0, 0] + [g.ptr(t) for t in extra] + [0, 0, 0] + [g.ptr(t) for t in doff], scratch=g.ptr(scratch))
    assert dfgpu.device_status() == 601 + which
    o = synthetic.bf16_bits_to_f32(g.to_host(do, np.uint16)).reshape(batch, 8, 128)
    if which == 1:
        assert np.all(o == 0.0)  # every V page reads as zeros
    assert np.all(np.isfinite(o))
    # and the next launch with the good prefix is fine
    doff = [g.to_device(good.astype(np.int64)), g.to_device(good.astype(np.int32))]
    dfgpu.sdpa_forward(p, [g.ptr(t) for t in dev + [do]] + [0, 0, 0] + [g.ptr(t) for t in extra] + [0, 0, 0] + [g.ptr(t) for t in doff], scratch=g.ptr(scratch))
    assert dfgpu.device_status() == 0


def test_paged_decode_zero_length_sequence_gives_zero_output():
    batch, hkv, pages, block, max_len = 3, 2, 16, 64, 256
    lengths, tk, tv = _paged_inputs(batch, 8, hkv, pages, block, max_len, seed=3, lengths=[0, 256, 100])
    info, o, o_ref, rows, rows_ref = both(BF16, [batch, 8, 1, 128], [pages, hkv, block, 128], [pages, hkv, block, 128], max_len,
                                          0.1, dfgpu.SDPA_AUTO, seq=([1] * batch, lengths), tables=(tk, tv))
    assert info.kernel == dfgpu.SDPA_PAGED_DECODE_UMMA
    assert np.all(o[0] == 0.0) and np.all(rows[0].reshape(batch, 8)[0] == -INF)
    close_bf16(o, o_ref)


@pytest.fixture(autouse=True)
def _device_healthy():
    yield
    assert dfgpu.device_status() == 0, "a bounded wait expired inside a kernel"


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("batch,hq,hkv,seq", [(1, 2, 2, 128), (2, 4, 2, 384), (1, 8, 1, 640), (1, 4, 2, 256), (2, 2, 1, 768), (2, 80, 20, 512)])
def test_umma_sdpa_matches_oracle(causal, batch, hq, hkv, seq):
    """Sequence lengths that are a multiple of 256 take the form with two query tiles per CTA
    (probabilities kept in tensor memory), the others one tile per CTA."""
    flags = dict(has_right_bound=1, right_bound=0) if causal else {}
    info, o, o_ref, rows, rows_ref = both(BF16, [batch, hq, seq, 128], [batch, hkv, seq, 128], [batch, hkv, seq, 128], seq,
                                          128 ** -0.5, dfgpu.SDPA_UMMA, stats=False, seed=17, **flags)
    assert info.kernel == dfgpu.SDPA_UMMA
    close_bf16(o, o_ref)


@pytest.mark.parametrize("causal", [True, False])
def test_umma_sdpa_max_and_sum_exp_rows(causal):
    """Stats, Max and Sum_exp from the two-tile tcgen05 kernel: the kernel's running reference maximum is raised
    lazily and exchanged in rounded form, so Max must come from the exact per-thread maxima and Sum_exp must be
    re-expressed against it."""
    flags = dict(has_right_bound=1, right_bound=0) if causal else {}
    info, o, o_ref, rows, rows_ref = both(BF16, [1, 4, 512, 128], [1, 2, 512, 128], [1, 2, 512, 128], 512, 2.5 * 128 ** -0.5,
                                          dfgpu.SDPA_UMMA, stats=True, seed=31, **flags)
    assert info.kernel == dfgpu.SDPA_UMMA
    close_bf16(o, o_ref)
    close_f32(rows[0], rows_ref[0], 2e-3)  # Stats
    close_f32(rows[1], rows_ref[1], 1e-5)  # Max: exact dot-product maximum times the scale
    close_f32(rows[2], rows_ref[2], 2e-3)  # Sum_exp


def test_umma_sdpa_stats_and_large_scores():
    """Stats = max + ln(sum) in natural log; a 4x larger scale makes the running maximum jump between
    tiles, which exercises the in-TMEM rescale of the output accumulator."""
    import gpu_util as g
    batch, heads, seq = 1, 2, 512
    p = dfgpu.SdpaParams()
    dims = [batch, heads, seq, 128]
    p.q = p.k = p.v = p.o = tensor(BF16, dims)
    p.stats = tensor(F32, [batch, heads, seq, 1])
    p.attn_scale, p.s_kv, p.has_right_bound, p.right_bound = 4 * 128 ** -0.5, seq, 1, 0
    raw = [synthetic.normal(23, i + 1, batch * heads * seq * 128) for i in range(3)]
    dev = [g.to_device(synthetic.to_bf16_bits(a)) for a in raw]
    outs = {}
    for kernel in (dfgpu.SDPA_UMMA, dfgpu.SDPA_ROWWISE):
        p.kernel = kernel
        do, ds = g.device_zeros(batch * heads * seq * 128 * 2), g.device_zeros(batch * heads * seq * 4)
        dfgpu.sdpa_forward(p, [g.ptr(dev[0]), g.ptr(dev[1]), g.ptr(dev[2]), g.ptr(do), g.ptr(ds), 0, 0, 0, 0, 0, 0])
        outs[kernel] = (synthetic.bf16_bits_to_f32(g.to_host(do, np.uint16)), g.to_host(ds, np.float32).copy())
    op = oracle.SdpaParams()
    op.q = op.k = op.v = op.o = tensor(F32, dims)
    op.stats = tensor(F32, [batch, heads, seq, 1])
    op.attn_scale, op.s_kv, op.has_right_bound, op.right_bound = p.attn_scale, seq, 1, 0
    rounded = [synthetic.round_to_bf16(a) for a in raw]
    o_ref, s_ref = np.zeros(batch * heads * seq * 128, dtype=np.float32), np.zeros(batch * heads * seq, dtype=np.float32)
    oracle.sdpa_forward(op, rounded + [o_ref, s_ref] + [None] * 6)
    for kernel in outs:
        close_bf16(outs[kernel][0], o_ref)
        close_f32(outs[kernel][1], s_ref, 2e-3)


def test_tma_paged_decode_long_sequences_and_windows():
    """Several CTAs per sequence (chunks of 1024 keys), a left bound that skips whole leading tiles,
    and a bottom-right aligned right bound."""
    batch, hq, hkv, pages, block, max_len = 3, 8, 2, 160, 64, 3000
    lengths, tk, tv = _paged_inputs(batch, hq, hkv, pages, block, max_len, seed=77, lengths=[3000, 1025, 2048])
    for flags in ({}, dict(has_left_bound=1, left_bound=1500, bottom_right=1), dict(has_right_bound=1, right_bound=-10, bottom_right=1)):
        outs = []
        for kernel in (dfgpu.SDPA_PAGED_DECODE_UMMA, dfgpu.SDPA_ROWWISE):
            info, o, o_ref, rows, rows_ref = both(BF16, [batch, hq, 1, 128], [pages, hkv, block, 128], [pages, hkv, block, 128], max_len,
                                                  128 ** -0.5, kernel, seq=([1] * batch, lengths), tables=(tk, tv), **flags)
            close_bf16(o, o_ref)
            close_f32(rows[0], rows_ref[0], 1e-3)
