"""The five benchmark graphs end to end: serialized graph -> compile_graph -> Executable.execute
on device buffers, against the CPU oracle evaluating the same document.

Gates: quantized codes and E8M0 scales bit-exact; f32 contractions max|d| <= 1e-4*max|ref|;
bf16 contractions |d| <= 1e-2 + 2e-2*|ref| (f32 accumulation)."""
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "oracle"))
import graph_oracle  # noqa: E402
from deepforge_b200 import dfgpu, harness, runtime, workloads  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _device_healthy():
    yield
    assert dfgpu.device_status() == 0


def oracle_inputs(wl, session, keep_in_storage=()):
    widened, storage = {}, {}
    for uid in list(wl.inputs) + list(wl.device_inputs):
        raw = session.raw(uid)
        data_type = wl.tensor(uid)["data_type"]
        if uid not in keep_in_storage:
            widened[uid] = graph_oracle.widen(raw, data_type)
        storage[uid] = raw.view({"BFLOAT16": np.uint16, "HALF": np.float16, "FLOAT": np.float32, "INT32": np.int32}.get(data_type, np.uint8))
    return widened, storage


def check_f32(actual, reference):
    scale = max(float(np.max(np.abs(reference))), 1e-30)
    assert float(np.max(np.abs(actual - reference))) <= 1e-4 * scale


def check_bf16(actual, reference):
    assert np.all(np.abs(actual - reference) <= 1e-2 + 2e-2 * np.abs(reference))


@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
@pytest.mark.parametrize("shape", [dict(n=1, c=3, h=5, w=5, k=5), dict(n=2, c=17, h=9, w=7, k=33), dict()])
def test_c1_single_conv(layout, shape):
    wl = workloads.c1(layout, **shape)
    s = harness.Session(wl)
    s.run()
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    check_f32(s.output(3), ref[3])
    assert np.all(np.abs(s.output(3) - ref[3]) <= 1e-4 + 1e-3 * np.abs(ref[3]))  # the reference's own acceptance rule


def check_chain(actual, staged, pure):
    """A chain of three bf16 contractions: each contraction is held to the bf16 gate against the
    oracle that feeds it the same bf16-rounded operands (the tensor core reads bf16); against
    the all-f32 twin the rounding of the two intermediates compounds, so that comparison gets
    twice the gate."""
    check_bf16(actual, staged)
    assert np.all(np.abs(actual - pure) <= 2e-2 + 4e-2 * np.abs(pure))


@pytest.mark.parametrize("io,options", [("FLOAT", 0), ("BFLOAT16", 0), ("BFLOAT16", runtime.NO_TENSOR_CORES), ("BFLOAT16", runtime.NO_FUSION)])
def test_c2_bottleneck_small(io, options):
    wl = workloads.c2(n=2, h=14, w=14, io=io)
    s = harness.Session(wl, options=options)
    s.run()
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    if io == "FLOAT":
        check_f32(s.output(7), ref[7])
    elif options == 0:
        # intermediates 13 and 16 live in the workspace as bf16 (they only feed tensor-core convolutions)
        check_chain(s.output(7), graph_oracle.run(wl.document, ins, round_to_bf16=(13, 16))[7], ref[7])
    else:
        check_bf16(s.output(7), ref[7])  # f32 intermediates: the plain gate holds end to end


def test_c2_each_contraction_within_the_gate_given_its_own_inputs():
    """Same DAG with the two intermediates made real bf16 outputs, so every convolution can be
    checked on its own against the oracle fed with the operands the GPU actually read."""
    wl = workloads.c2(n=2, h=14, w=14)
    doc = wl.document
    for uid in ("13", "16"):
        doc["tensors"][uid].update(is_virtual=False, data_type="BFLOAT16")
    s = harness.Session(wl)
    assert s.exe.launch_count == 3
    s.run()
    ins, _ = oracle_inputs(wl, s)
    t1, t2, y = s.output(13), s.output(16), s.output(7)
    stage = lambda nodes, values: graph_oracle.run({**doc, "nodes": nodes}, values)
    check_bf16(t1, stage(doc["nodes"][:3], ins)[13])
    check_bf16(t2, stage(doc["nodes"][3:6], {**ins, 13: t1})[16])
    check_bf16(y, stage(doc["nodes"][6:], {**ins, 16: t2})[7])


def test_c2_bottleneck_full_geometry_two_images():
    wl = workloads.c2(n=2)  # 56x56, 256->64->64->256, the benchmark's per-image geometry
    s = harness.Session(wl)
    assert s.exe.launch_count == 3 and s.exe.plan_text().count("kernel=3") == 3
    s.run()
    ins, _ = oracle_inputs(wl, s)
    check_chain(s.output(7), graph_oracle.run(wl.document, ins, round_to_bf16=(13, 16))[7], graph_oracle.run(wl.document, ins)[7])


@pytest.mark.parametrize("io,c_type,options", [("FLOAT", "FLOAT", 0), ("BFLOAT16", "BFLOAT16", 0), ("BFLOAT16", "FLOAT", runtime.NO_FUSION)])
def test_c3_quantize_matmul_small(io, c_type, options):
    wl = workloads.c3(m=128, k=256, n=192, io=io, c_type=c_type)
    s = harness.Session(wl, options=options)
    s.run()
    ins, storage = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins, storage_inputs=storage)
    for uid in (3, 4, 5, 6):
        assert np.array_equal(s.output(uid), ref[uid]), f"codes/scales of tensor {uid} must be bit-exact"
    (check_f32 if c_type == "FLOAT" else check_bf16)(s.output(9), ref[9])


def test_c3_full_size_codes_exact_and_matmul_rows():
    wl = workloads.c3()
    s = harness.Session(wl)
    s.run()
    ins, storage = oracle_inputs(wl, s)
    # oracle on a slab: 32 rows of A (all of K), and B through its first 64 K-rows
    rows = 32
    sub = workloads.c3(m=rows, k=4096, n=4096)
    a_sub = {1: ins[1][: rows * 4096], 2: ins[2]}
    st_sub = {1: storage[1][: rows * 4096]}
    ref = graph_oracle.run({**sub.document, "nodes": [sub.document["nodes"][0]]}, a_sub, storage_inputs=st_sub)
    assert np.array_equal(s.output(3)[: rows * 4096], ref[3])
    assert np.array_equal(s.output(4)[: rows * 128], ref[4])
    kb = workloads.c3(m=4096, k=64, n=4096)
    ref_b = graph_oracle.run({**kb.document, "nodes": [kb.document["nodes"][1]]}, {2: ins[2][: 64 * 4096]}, storage_inputs={2: storage[2][: 64 * 4096]})
    assert np.array_equal(s.output(5)[: 64 * 4096], ref_b[5])
    assert np.array_equal(s.output(6)[: 2 * 4096], ref_b[6])
    # matmul rows 0..7 from the GPU's own (verified) codes: dequantize + f32 matmul in the oracle
    from oracle import tensor as T
    import oracle
    aq, sa, bq, sb = s.output(3), s.output(4), s.output(5), s.output(6)
    af = np.zeros(8 * 4096, dtype=np.float32)
    oracle.block_scale_dequantize(T(dfgpu.E4M3, [8, 4096]), aq[: 8 * 4096], T(dfgpu.E8M0, [8, 128]), sa[: 8 * 128], T(dfgpu.F32, [8, 4096]), af, [1, 32])
    bf = np.zeros(4096 * 4096, dtype=np.float32)
    oracle.block_scale_dequantize(T(dfgpu.E4M3, [4096, 4096]), bq, T(dfgpu.E8M0, [128, 4096]), sb, T(dfgpu.F32, [4096, 4096]), bf, [32, 1])
    c_ref = (af.reshape(8, 4096).astype(np.float64) @ bf.reshape(4096, 4096).astype(np.float64)).astype(np.float32)
    check_bf16(s.output(9)[: 8 * 4096].reshape(8, 4096), c_ref)


@pytest.mark.parametrize("io", ["FLOAT", "BFLOAT16"])
def test_c4_sdpa_small(io):
    wl = workloads.c4(b=2, h=3, s=160, d=128, io=io)
    s = harness.Session(wl)
    s.run()
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    if io == "FLOAT":
        assert np.all(np.abs(s.output(4) - ref[4]) <= 8e-5 * (1 + np.abs(ref[4])))
        assert np.all(np.abs(s.output(5) - ref[5]) <= 8e-5 * (1 + np.abs(ref[5])))
    else:
        check_bf16(s.output(4), ref[4])
        assert np.all(np.abs(s.output(5) - ref[5]) <= 2e-3 * (1 + np.abs(ref[5])))


def test_c4_sdpa_full_size_sampled_rows():
    wl = workloads.c4()
    s = harness.Session(wl)
    s.run()
    ins, _ = oracle_inputs(wl, s)
    # oracle on (batch 3, head 17) and (batch 7, head 31), every 64th query row
    out = s.output(4).reshape(8, 32, 2048, 128)
    stats = s.output(5).reshape(8, 32, 2048)
    for bh in (3 * 32 + 17, 7 * 32 + 31):
        ref = graph_oracle.run(wl.document, ins, sdpa_bh=(bh, bh + 1), sdpa_q_step=64)
        b, h = divmod(bh, 32)
        check_bf16(out[b, h, ::64], ref[4].reshape(8, 32, 2048, 128)[b, h, ::64])
        r = ref[5].reshape(8, 32, 2048)[b, h, ::64]
        assert np.all(np.abs(stats[b, h, ::64] - r) <= 2e-3 * (1 + np.abs(r)))
    # size-independent property: causal row 0 attends to key 0 only, so O[.., 0, :] == V[.., 0, :]
    v = ins[3].reshape(8, 32, 2048, 128)
    assert np.array_equal(out[:, :, 0], v[:, :, 0])


def test_c5_paged_decode_small_and_generic_agree():
    wl = workloads.c5(batch=6, hq=8, hkv=2, pages=64, block=64, max_len=1024, min_len=64)
    for options in (0,):
        s = harness.Session(wl, options=options)
        assert "kernel=4" in s.exe.plan_text()  # the TMA-streamed paged decode kernel
        s.run()
        ins, _ = oracle_inputs(wl, s)
        ref = graph_oracle.run(wl.document, ins)
        check_bf16(s.output(4), ref[4])


def test_c5_paged_decode_full_size_sampled_sequences():
    wl = workloads.c5()
    s = harness.Session(wl)
    s.run()
    out = s.output(4).reshape(64, 32, 128)
    ins, storage = oracle_inputs(wl, s, keep_in_storage=(2, 3))  # the 2 x 2.1 GB pools stay bf16 on the host
    for b in (0, 41):
        ref = graph_oracle.run(wl.document, ins, sdpa_bh=(b * 32, b * 32 + 8), storage_inputs=storage)
        check_bf16(out[b, :8], ref[4].reshape(64, 32, 128)[b, :8])
    # linearity in V: doubling the V pool doubles the output (bf16 doubling is exact)
    import torch
    s.dev[3].view(torch.bfloat16).mul_(2)
    s.run()
    doubled = s.output(4).reshape(64, 32, 128)
    assert np.array_equal(doubled, out * 2)


@pytest.mark.parametrize("name,size", [("c2", dict(n=2, h=14, w=14)), ("c3", dict(m=128, k=128, n=128)), ("c4", dict(b=1, h=2, s=256)),
                                       ("c5", dict(batch=3, hq=8, hkv=2, pages=32, max_len=512, min_len=100)), ("fp8", dict(m=128, k=128, n=128))])
def test_executable_loaded_from_an_artifact_gives_the_same_bits(name, size):
    """compile -> serialize -> load_artifact_executable: the loaded plan runs the same launches on the same buffers."""
    wl = workloads.BUILDERS[name](**size)
    s = harness.Session(wl)
    s.run()
    compiled = {uid: s.raw(uid).copy() for uid in wl.outputs}
    loaded = runtime.load_artifact(s.exe.serialize())
    assert loaded.plan_text() == s.exe.plan_text()
    for uid in wl.outputs:
        s.dev[uid].zero_()
    s.exe = loaded
    s.run()
    for uid in wl.outputs:
        assert np.array_equal(s.raw(uid), compiled[uid]), f"tensor {uid}"


def test_sdpa_graph_with_bias_and_alibi():
    """The Bias port and alibi_mask through the importer, the lowering and Executable.execute (general kernel)."""
    from deepforge_b200 import graphs, synthetic
    wl = workloads.c4(b=2, h=4, s=48, d=32, io="FLOAT")
    wl.document["tensors"]["9"] = graphs.tensor(9, "Bias", [1, 4, 48, 48])
    wl.document["nodes"][0]["inputs"]["Bias"] = 9
    wl.document["nodes"][0]["alibi_mask"] = True
    wl.inputs[9] = lambda: synthetic.normal(77, 9, 4 * 48 * 48).astype(np.float32)
    s = harness.Session(wl)
    assert "kernel=1" in s.exe.plan_text()
    s.run()
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    check_f32(s.output(4), ref[4])
    check_f32(s.output(5), ref[5])
    loaded = runtime.load_artifact(s.exe.serialize())
    assert loaded.plan_text() == s.exe.plan_text()


def test_sdpa_graph_with_sink_token_and_block_mask():
    """SINK_TOKEN ([1, Hq, 1, 1] FLOAT) and Block_mask (UINT8, one bit per 128 x 128 tile) through Executable.execute."""
    from deepforge_b200 import graphs, synthetic
    wl = workloads.c4(b=1, h=2, s=256, d=32, io="FLOAT", causal=False)
    wl.document["tensors"]["9"] = graphs.tensor(9, "SINK_TOKEN", [1, 2, 1, 1])
    wl.document["tensors"]["10"] = graphs.tensor(10, "Block_mask", [1, 2, 2, 1], "UINT8")
    wl.document["nodes"][0]["inputs"]["SINK_TOKEN"] = 9
    wl.document["nodes"][0]["inputs"]["Block_mask"] = 10
    wl.inputs[9] = lambda: np.array([0.5, -1.0], dtype=np.float32)
    wl.inputs[10] = lambda: np.array([0b01, 0b11, 0b10, 0b00], dtype=np.uint8)
    s = harness.Session(wl)
    assert "kernel=1" in s.exe.plan_text()  # the general kernel, although the shape fits the tcgen05 one
    s.run()
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    check_f32(s.output(4), ref[4])
    check_f32(s.output(5), ref[5])
    stats = s.output(5).reshape(1, 2, 256)
    assert np.allclose(stats[0, 1, 128:], -1.0)  # fully masked rows keep the sink logit: Stats = sink + ln(1)
