"""The allocation-free paged-decode entry point (collected last on purpose).

A host that may not allocate device memory around the call -- allocation frozen after
start-up, an allocator lock held above it, a real-time thread -- uses
dfgpu_sdpa_paged_decode_static, which keeps its split-KV partials in an 8 MiB array built
into the library. Its result must equal the regular entry point's (same kernels, different
scratch), on two calls in a row: the array is shared and keeps the first call's contents.
Both are also held to the CPU oracle's answer for the same inputs, so that the pair cannot
agree on something wrong."""
import numpy as np
import pytest

from deepforge_b200 import dfgpu, synthetic
from deepforge_b200.dfgpu import BF16, F32, I32, tensor

pytestmark = pytest.mark.gpu


def _case(batch, hq, hkv, pages, block, max_len, seed):
    import gpu_util as g
    table_len = max_len // block
    lengths = synthetic.integers(seed, 50, batch, max_len // 8, max_len).astype(np.int32)
    lengths[0] = max_len
    tk = np.stack([synthetic.permutation_prefix(seed, 100 + i, pages, table_len) for i in range(batch)]).astype(np.int32)
    tv = np.stack([synthetic.permutation_prefix(seed, 200 + i, pages, table_len) for i in range(batch)]).astype(np.int32)
    p = dfgpu.SdpaParams()
    p.q = p.o = tensor(BF16, [batch, hq, 1, 128])
    p.k = p.v = tensor(BF16, [pages, hkv, block, 128])
    p.stats = tensor(F32, [batch, hq, 1, 1])
    p.seq_q = p.seq_kv = tensor(I32, [batch, 1, 1, 1])
    p.page_table_k = p.page_table_v = tensor(I32, [batch, 1, table_len, 1])
    p.attn_scale, p.padding_mask, p.s_kv = 128 ** -0.5, 1, max_len
    host = [synthetic.to_bf16_bits(synthetic.normal(seed, i + 1, n)) for i, n in enumerate((batch * hq * 128, pages * hkv * block * 128, pages * hkv * block * 128))]
    dev = [g.to_device(a) for a in host]
    extra = [g.to_device(np.ones(batch, dtype=np.int32)), g.to_device(lengths), g.to_device(tk), g.to_device(tv)]
    return p, dev, extra, (host, lengths, tk, tv)


def _oracle(p, host, lengths, tk, tv):
    """The CPU oracle on the same (bf16-rounded) inputs: O and Stats in f32."""
    import oracle
    batch, hq = int(p.q.dim[0]), int(p.q.dim[1])
    op = oracle.SdpaParams()
    for name in ("q", "k", "v", "o"):
        t = getattr(p, name)
        setattr(op, name, tensor(F32, [int(t.dim[i]) for i in range(4)]))
    op.stats = tensor(F32, [batch, hq, 1, 1])
    op.seq_q = op.seq_kv = tensor(I32, [batch, 1, 1, 1])
    op.page_table_k = op.page_table_v = tensor(I32, [batch, 1, tk.shape[1], 1])
    op.attn_scale, op.padding_mask, op.s_kv = p.attn_scale, 1, p.s_kv
    o_ref = np.zeros(batch * hq * 128, dtype=np.float32)
    stats_ref = np.zeros(batch * hq, dtype=np.float32)
    widened = [synthetic.bf16_bits_to_f32(a) for a in host]
    oracle.sdpa_forward(op, widened + [o_ref, stats_ref, None, None, np.ones(batch, dtype=np.int32), lengths,
                                       np.ascontiguousarray(tk), np.ascontiguousarray(tv)])
    return o_ref, stats_ref


def _run(p, dev, extra, static):
    import gpu_util as g
    out = g.device_zeros(p.q.dim[0] * p.q.dim[1] * 128 * 2, 0x7f)
    stats = g.device_zeros(p.q.dim[0] * p.q.dim[1] * 4, 0x7f)
    pointers = [g.ptr(dev[0]), g.ptr(dev[1]), g.ptr(dev[2]), g.ptr(out), g.ptr(stats), 0, 0] + [g.ptr(t) for t in extra]
    if static:
        dfgpu.sdpa_paged_decode_static(p, pointers)
    else:
        p.kernel = dfgpu.SDPA_PAGED_DECODE
        info = dfgpu.query("sdpa_forward", p)
        scratch = g.device_zeros(info.scratch_bytes)
        dfgpu.sdpa_forward(p, pointers, scratch=g.ptr(scratch))
    return g.to_host(out, np.uint16).copy(), g.to_host(stats, np.float32).copy()


def test_static_scratch_decode_matches_the_regular_entry_point_twice_in_a_row():
    # two different problems back to back: the second starts with the first one's partials in the array
    for batch, hq, hkv, pages, block, max_len, seed in ((4, 8, 2, 48, 64, 1024, 3), (3, 32, 8, 40, 64, 768, 4)):
        p, dev, extra, host_side = _case(batch, hq, hkv, pages, block, max_len, seed)
        want_o, want_stats = _run(p, dev, extra, static=False)
        got_o, got_stats = _run(p, dev, extra, static=True)
        # same kernels on the same data: bit-identical, which is inside every tolerance the suite uses
        assert np.array_equal(got_o, want_o)
        assert np.array_equal(got_stats, want_stats)
        # and the answer itself, against the CPU oracle (the suite's bf16 gate; Stats as in the other decode tests)
        o_ref, stats_ref = _oracle(p, *host_side)
        got = synthetic.bf16_bits_to_f32(got_o)
        assert np.all(np.abs(got - o_ref) <= 1e-2 + 2e-2 * np.abs(o_ref))
        assert np.all(np.abs(got_stats - stats_ref) <= 1e-3 * (1 + np.abs(stats_ref)))
    assert dfgpu.device_status() == 0


def test_static_scratch_decode_refuses_requests_beyond_its_limit():
    p, dev, extra, _ = _case(2, 8, 2, 16, 64, 512, 5)
    p.q = p.o = tensor(BF16, [64, 32, 1, 128])  # 64 * 32 * 32 chunks * 520 B = 34 MB > 8 MiB
    p.k = p.v = tensor(BF16, [16, 8, 64, 128])
    p.s_kv = 8192
    p.page_table_k = p.page_table_v = tensor(I32, [64, 1, 128, 1])
    p.seq_q = p.seq_kv = tensor(I32, [64, 1, 1, 1])
    p.stats = tensor(F32, [64, 32, 1, 1])
    with pytest.raises(dfgpu.DfgpuError) as error:
        dfgpu.sdpa_paged_decode_static(p, [0x10000] * 11)
    assert error.value.code == 15 and "8388608" in str(error.value)
