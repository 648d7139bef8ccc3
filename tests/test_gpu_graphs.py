"""The five benchmark graphs end to end: serialized graph -> compile_graph -> Executable.execute
on device buffers, against the CPU oracle evaluating the same document.

Gates: quantized codes and E8M0 scales bit-exact; f32 contractions max|d| <= 1e-4*max|ref|;
bf16 contractions |d| <= 1e-2 + 2e-2*|ref| (f32 accumulation)."""
import dataclasses
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "oracle"))
import df_oracle_binding as oracle_binding  # noqa: E402
import graph_oracle  # noqa: E402
from deepforge_b200 import dfgpu, harness, runtime, synthetic, workloads  # noqa: E402

THREADS = oracle_binding.host_threads()  # the oracle's per-element arithmetic does not depend on the thread count

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
        storage[uid] = raw.view({"BFLOAT16": np.uint16, "HALF": np.float16, "FLOAT": np.float32, "INT32": np.int32, "INT64": np.int64}.get(data_type, np.uint8))
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


@pytest.mark.parametrize("io,options", [("FLOAT", 0), ("BFLOAT16", 0), ("BFLOAT16", runtime.NO_CONV_PAIRS), ("BFLOAT16", runtime.NO_TENSOR_CORES), ("BFLOAT16", runtime.NO_FUSION),
                                        ("BFLOAT16", runtime.NO_NARROWING), ("BFLOAT16", runtime.BF16_INTERMEDIATES)])
def test_c2_bottleneck_small(io, options):
    wl = workloads.c2(n=2, h=14, w=14, io=io)
    s = harness.Session(wl, options=options)
    s.run()
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    if io == "FLOAT":
        check_f32(s.output(7), ref[7])
    elif options == runtime.BF16_INTERMEDIATES:
        # the lossy option, off by default: intermediates 13 and 16 are rounded to bf16 in the workspace, so the
        # gate is held against the oracle that rounds at the same two points, not against the all-FLOAT twin
        assert s.exe.plan_text().count("kernel=3") == 3
        check_bf16(s.output(7), graph_oracle.run(wl.document, ins, round_to_bf16=(13, 16))[7])
    else:
        # every other plan holds the plain gate against the all-FLOAT evaluation of the DAG: the default one (conv1, then
        # conv2 > conv3 in the two-convolution kernel, intermediates as (hi, lo) bf16 pairs) and the one with three
        # tcgen05 launches included
        if options == 0:
            assert s.exe.launch_count == 2 and "conv_fprop_pair kernel=1" in s.exe.plan_text()
        if options == runtime.NO_CONV_PAIRS:
            assert s.exe.plan_text().count("conv_fprop kernel=3") == 3
        check_bf16(s.output(7), ref[7])


@pytest.mark.parametrize("layout", ["channels_last", "ncw"])
def test_one_dimensional_convolution_with_bias_and_relu(layout):
    """A rank-3 CONV_FPROP ([N, C, W], filter [K, C, R], stride 2, dilation 2, asymmetric padding) with bias and ReLU behind it: lowered as
    the 2-D convolution over images of a single row, one launch on the tensor cores; a rank-5 one is refused."""
    from deepforge_b200 import graphs
    n, c, width, k, r = 3, 64, 50, 32, 5
    pre, post, stride, dilation = 3, 1, 2, 2
    q = (width + pre + post - (dilation * (r - 1) + 1)) // stride + 1
    strides = (lambda d: [d[1] * d[2], 1, d[1]]) if layout == "channels_last" else (lambda d: [d[1] * d[2], d[2], 1])
    tensors = [graphs.tensor(1, "X", [n, c, width], "FLOAT", strides([n, c, width])), graphs.tensor(2, "W", [k, c, r], "FLOAT", strides([k, c, r])),
               graphs.tensor(3, "B", [1, k, 1], "FLOAT", [k, 1, 1]), graphs.tensor(4, "Y", [n, k, q], "FLOAT", strides([n, k, q])),
               graphs.tensor(11, "conv_out", [n, k, q], "FLOAT", strides([n, k, q]), True), graphs.tensor(12, "bias_out", [n, k, q], "FLOAT", strides([n, k, q]), True)]
    nodes = [graphs.conv_node("conv", 1, 2, 11, (pre,), (post,), (stride,), (dilation,)), graphs.pointwise_node("bias", "ADD", 11, 12, 3),
             graphs.pointwise_node("relu", "RELU_FWD", 12, 4)]
    doc = graphs.document("conv1d", nodes, tensors)
    wl = workloads.Workload(name="conv1d", config=0, document=doc, description={}, metric="conv_fprop_throughput", unit="TFLOP/s", flops=1.0, bytes=1.0,
                            bound="hbm", inputs={1: workloads._uniform(5, 1, n * c * width, "FLOAT", -1.0, 1.0), 2: workloads._uniform(5, 2, k * c * r, "FLOAT", -0.2, 0.2),
                                                 3: workloads._uniform(5, 3, k, "FLOAT", -0.5, 0.5)}, outputs=[4])
    s = harness.Session(wl)
    assert s.exe.launch_count == 1 and "conv_fprop kernel=5 launches=1 [conv+bias+relu]" in s.exe.plan_text()
    s.run()
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    check_f32(s.output(4), ref[4])
    assert np.all(np.abs(s.output(4) - ref[4]) <= 1e-4 + 1e-3 * np.abs(ref[4])) and float(np.min(s.output(4))) == 0.0
    assert dfgpu.device_status() == 0


def test_three_dimensional_convolution_with_bias_and_residual():
    """A rank-5 CONV_FPROP ([N, C, D, H, W], filter [K, C, T, R, S]; stride 2 in depth, dilation 2 in the rows, asymmetric padding) with a
    per-channel bias, ReLU and a full-size addend: one launch of the one-launch tcgen05 kernel, which walks the depth axis too, for the
    channels-last and the NCDHW layout, and for the reversed filter of math_mode CONVOLUTION."""
    from deepforge_b200 import graphs
    n, c, depth, h, w, k = 2, 24, 6, 9, 7, 20
    taps, pre, post, stride, dilation = (3, 3, 2), (1, 2, 0), (1, 2, 1), (2, 1, 1), (1, 2, 1)
    out = [(e + a + b - (d * (f - 1) + 1)) // s + 1 for e, a, b, d, f, s in zip((depth, h, w), pre, post, dilation, taps, stride)]
    for layout in ("channels_last", "ncdhw"):
        for mode in ("CROSS_CORRELATION", "CONVOLUTION"):
            strides = (lambda d: [d[1] * d[2] * d[3] * d[4], 1, d[3] * d[4] * d[1], d[4] * d[1], d[1]]) if layout == "channels_last" else (lambda d: None)
            xd, wd, yd = [n, c, depth, h, w], [k, c, *taps], [n, k, *out]
            tensors = [graphs.tensor(1, "X", xd, "FLOAT", strides(xd)), graphs.tensor(2, "W", wd, "FLOAT", strides(wd)),
                       graphs.tensor(3, "B", [1, k, 1, 1, 1], "FLOAT", [k, 1, 1, 1, 1]), graphs.tensor(4, "Z", yd, "FLOAT", strides(yd)),
                       graphs.tensor(5, "Y", yd, "FLOAT", strides(yd)),
                       graphs.tensor(11, "conv_out", yd, "FLOAT", strides(yd), True), graphs.tensor(12, "bias_out", yd, "FLOAT", strides(yd), True),
                       graphs.tensor(13, "relu_out", yd, "FLOAT", strides(yd), True)]
            nodes = [graphs.conv_node("conv", 1, 2, 11, pre, post, stride, dilation, mode), graphs.pointwise_node("bias", "ADD", 11, 12, 3),
                     graphs.pointwise_node("relu", "RELU_FWD", 12, 13), graphs.pointwise_node("residual", "ADD", 13, 5, 4)]
            doc = graphs.document("conv3d", nodes, tensors)
            count = lambda d: int(np.prod(d))
            wl = workloads.Workload(name="conv3d", config=0, document=doc, description={}, metric="conv_fprop_throughput", unit="TFLOP/s", flops=1.0, bytes=1.0,
                                    bound="hbm", inputs={1: workloads._uniform(6, 1, count(xd), "FLOAT", -1.0, 1.0), 2: workloads._uniform(6, 2, count(wd), "FLOAT", -0.2, 0.2),
                                                         3: workloads._uniform(6, 3, k, "FLOAT", -0.5, 0.5), 4: workloads._uniform(6, 4, count(yd), "FLOAT", -1.0, 1.0)}, outputs=[5])
            s = harness.Session(wl)
            assert s.exe.launch_count == 1 and "conv_fprop kernel=5 launches=1 [conv+bias+relu+residual]" in s.exe.plan_text()
            s.run()
            ins, _ = oracle_inputs(wl, s)
            ref = graph_oracle.run(wl.document, ins)
            check_f32(s.output(5), ref[5])
            assert np.all(np.abs(s.output(5) - ref[5]) <= 1e-4 + 1e-3 * np.abs(ref[5]))
    assert dfgpu.device_status() == 0


@pytest.mark.parametrize("kind", ["probability", "mask"])
def test_sdpa_with_dropout_through_the_executable(kind):
    """SDPA with dropout lowered from the serialized graph: probability dropout (Seed and Offset INT64 scalars, RNG_DUMP output) and custom dropout
    (Dropout_mask broadcast over the batch, Dropout_scale), against the oracle; RNG_DUMP bit for bit."""
    import copy
    wl = workloads.c4(b=2, h=4, s=48, d=32, io="FLOAT")
    doc = copy.deepcopy(wl.document)
    node = doc["nodes"][0]
    inputs = dict(wl.inputs)
    outputs = list(wl.outputs)
    from deepforge_b200 import graphs
    if kind == "probability":
        node["dropout_probability"] = 0.25
        node["inputs"].update(Seed=20, Offset=21)
        node["outputs"]["RNG_DUMP"] = 22
        doc["tensors"]["20"] = graphs.tensor(20, "Seed", [1, 1, 1, 1], "INT64")
        doc["tensors"]["21"] = graphs.tensor(21, "Offset", [1, 1, 1, 1], "INT64")
        doc["tensors"]["22"] = graphs.tensor(22, "RNG_DUMP", [2, 4, 48, 48], "FLOAT")
        inputs[20], inputs[21] = (lambda: np.array([4242], np.int64)), (lambda: np.array([-17], np.int64))
        outputs.append(22)
    else:
        node["inputs"].update(Dropout_mask=20, Dropout_scale=21)
        doc["tensors"]["20"] = graphs.tensor(20, "Dropout_mask", [1, 4, 48, 48], "FLOAT")
        doc["tensors"]["21"] = graphs.tensor(21, "Dropout_scale", [1, 1, 1, 1], "FLOAT")
        inputs[20] = lambda: (synthetic.uniform(3, 20, 4 * 48 * 48, 0.0, 1.0) < 0.8).astype(np.float32)
        inputs[21] = lambda: np.array([1.25], np.float32)
    wl = dataclasses.replace(wl, document=doc, inputs=inputs, outputs=outputs)
    s = harness.Session(wl)
    assert "sdpa_forward kernel=1" in s.exe.plan_text()
    s.run()
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    check_f32(s.output(4), ref[4])
    assert np.allclose(s.output(5), ref[5], rtol=1e-4, atol=1e-5)
    if kind == "probability":
        dump = s.output(22)
        assert np.array_equal(dump, ref[22]) and 0.65 < float(dump.mean()) < 0.85
    plain = harness.Session(workloads.c4(b=2, h=4, s=48, d=32, io="FLOAT"))
    plain.run()
    assert not np.allclose(plain.output(4), s.output(4), atol=1e-3) and np.allclose(plain.output(5), s.output(5), rtol=1e-5, atol=1e-6)
    assert dfgpu.device_status() == 0


def test_c2_bottleneck_float_on_tensor_cores():
    """An all-FLOAT bottleneck big enough for the tensor cores (N = 8, 28 x 28): conv1 and conv2 have 49 output tiles and run as one
    cluster launch each (bias and ReLU in its epilogue), conv3 has 196 and runs as the three-launch split form (residual in the adder);
    the f32 gates hold against the oracle."""
    wl = workloads.c2(n=8, h=28, w=28, io="FLOAT")
    s = harness.Session(wl)
    plan = s.exe.plan_text()
    assert plan.count("conv_fprop kernel=5 launches=1") == 2 and plan.count("conv_fprop kernel=4 launches=3") == 1 and s.exe.launch_count == 5
    s.run()
    ins, _ = oracle_inputs(wl, s)
    check_f32(s.output(7), graph_oracle.run(wl.document, ins, threads=THREADS)[7])
    assert dfgpu.device_status() == 0


@pytest.mark.parametrize("options", [0, runtime.NO_CONV_PAIRS])
@pytest.mark.parametrize("shape", [dict(n=1, h=7, w=7), dict(n=3, h=28, w=28), dict(n=2, h=9, w=11), dict(n=1, h=8, w=120), dict(n=5, h=56, w=56, c_in=128)])
def test_c2_bottleneck_other_geometries(shape, options):
    """Image sizes that give other tile shapes (the 3 x 3 convolution takes 7, 4, 9, 1 or 2 output rows per tile) and a
    128-channel block, through the two-convolution kernel and as three launches."""
    wl = workloads.c2(**shape)
    s = harness.Session(wl, options=options)
    if options == 0 and shape["w"] != 120:  # (two windows of a 122-pixel pitch do not fit beside the filters: three launches there)
        assert s.exe.launch_count == 2 and "conv_fprop_pair kernel=1" in s.exe.plan_text()
    else:
        assert s.exe.plan_text().count("conv_fprop kernel=3") == 3
    s.run()
    ins, _ = oracle_inputs(wl, s)
    check_bf16(s.output(7), graph_oracle.run(wl.document, ins, threads=THREADS)[7])


def test_split_intermediates_carry_f32_grade_values():
    """The (hi, lo) pair storage on its own: with the intermediates made visible through a FLOAT-intermediate run of
    the same graph, hi + lo of what conv1 wrote equals the f32 value to 2^-16 relative, far inside what a single
    bf16 (2^-9) keeps. Read back from the workspace of the default plan."""
    wl = workloads.c2(n=1, h=14, w=14)
    s = harness.Session(wl)
    s.run()
    import torch
    torch.cuda.synchronize()
    plan = s.exe.plan_text()
    assert "ws+0(uid13)" in plan
    pixels, channels = 14 * 14, 64
    raw = s.workspace[: pixels * channels * 4].cpu().numpy().view(np.uint16).reshape(pixels, 2, channels)
    from deepforge_b200 import synthetic
    hi, lo = synthetic.bf16_bits_to_f32(raw[:, 0, :]), synthetic.bf16_bits_to_f32(raw[:, 1, :])
    ins, _ = oracle_inputs(wl, s)
    t1 = graph_oracle.run({**wl.document, "nodes": wl.document["nodes"][:3]}, ins)[13].reshape(pixels, channels)
    assert np.all(np.abs((hi.astype(np.float64) + lo) - t1) <= 2.0 ** -15 * np.abs(t1) + 1e-6)
    assert np.all(np.abs(lo) <= 2.0 ** -8 * np.abs(hi) + 1e-30)  # lo is the rounding remainder of hi


def test_misaligned_argument_is_refused_before_any_launch():
    """Arguments bound to a TMA-fed launch advertise 16-byte alignment: a pointer the reference's rule would accept
    (8-byte aligned bf16) is DFE_INVALID_VARIANT_PACK up front, not a failure part-way through the plan."""
    import torch
    wl = workloads.c2(n=1, h=14, w=14)
    s = harness.Session(wl)
    shifted = torch.zeros(s.dev[1].numel() + 16, dtype=torch.uint8, device=s.device)
    shifted[8:8 + s.dev[1].numel()].copy_(s.dev[1])
    pack = dict(s.pack)
    pack[1] = shifted.data_ptr() + 8
    s.dev[7].zero_()
    with pytest.raises(runtime.DeepForgeError) as error:
        s.exe.execute(pack, s.workspace_ptr)
    assert error.value.code == 17 and "aligned" in str(error.value)
    torch.cuda.synchronize()
    assert not s.dev[7].any()  # nothing ran


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
    assert s.exe.launch_count == 2 and "conv_fprop_pair kernel=1" in s.exe.plan_text()
    s.run()
    ins, _ = oracle_inputs(wl, s)
    check_bf16(s.output(7), graph_oracle.run(wl.document, ins, threads=THREADS)[7])


def test_c2_bottleneck_full_size():
    """The benchmark configuration itself (N = 32): every one of the 25.7 M outputs against the all-FLOAT twin."""
    wl = workloads.c2()
    ins = reference = None
    for options in (0, runtime.NO_CONV_PAIRS):  # the benchmarked plan, and the same graph as three tcgen05 launches
        s = harness.Session(wl, options=options)
        assert ("conv_fprop_pair kernel=1" in s.exe.plan_text()) == (options == 0)
        s.run()
        if reference is None:
            ins, _ = oracle_inputs(wl, s)
            reference = graph_oracle.run(wl.document, ins, threads=THREADS)[7]
        check_bf16(s.output(7), reference)
        del s


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


def test_c3_quantize_matmul_with_e5m2_codes():
    """The same graph with FP8_E5M2 codes for A and B: the quantize nodes run the general kernel (two launches), the dequantize nodes stay
    launches of their own (the block-scaled tensor-core matmul reads E4M3 codes), codes and scales are bit-exact, C holds the bf16 gate."""
    import copy
    wl = workloads.c3(m=128, k=256, n=192)
    wl = dataclasses.replace(wl, document=copy.deepcopy(wl.document))
    for uid in ("3", "5"):
        wl.document["tensors"][uid]["data_type"] = "FP8_E5M2"
    s = harness.Session(wl)
    plan = s.exe.plan_text()
    assert plan.count("block_scale_quantize kernel=1") == 2 and plan.count("block_scale_dequantize") == 2
    s.run()
    ins, storage = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins, storage_inputs=storage)
    for uid in (3, 4, 5, 6):
        assert np.array_equal(s.output(uid), ref[uid]), f"codes/scales of tensor {uid} must be bit-exact"
    check_bf16(s.output(9), ref[9])


def test_packed_four_bit_graphs_reproduce_the_reference_known_answers():
    """The reference's two four-bit cases through the Executable (test/Compiler/SpecializedOpsTest.cpp:736-754 and :661-681): FLOAT ->
    FP4_E2M1 codes with FP8_E4M3 scales (both virtual, in the workspace) -> FLOAT gives 1.03125, 2.0625, -3, 6; INT4 nibbles with HALF
    scales give the BFLOAT16 bits c080 bf00 0000 4160. And a larger FP4 round trip against the oracle, bit for bit."""
    from deepforge_b200 import graphs

    def roundtrip(rows, cols, block):
        t = [graphs.tensor(14, "X", [rows, cols]), graphs.tensor(15, "Q", [rows, cols], "FP4_E2M1", None, True),
             graphs.tensor(16, "S", [rows, cols // block], "FP8_E4M3", None, True), graphs.tensor(17, "Y", [rows, cols])]
        return graphs.document("fp4_roundtrip", [graphs.quantize_node("q", 14, 15, 16, block, 1), graphs.dequantize_node("d", 15, 16, 17, [block])], t)

    def session(doc, inputs, outputs):
        wl = workloads.Workload(name="four_bit", config=0, document=doc, description={}, metric="", unit="GB/s", flops=1.0, bytes=1.0, bound="hbm",
                                inputs=inputs, outputs=outputs)
        s = harness.Session(wl)
        s.run()
        return wl, s

    wl, s = session(roundtrip(1, 4, 2), {14: lambda: np.array([1.0, 2.0, -3.0, 6.0], np.float32)}, [17])
    assert s.output(17).tolist() == [1.03125, 2.0625, -3.0, 6.0] and s.exe.workspace_size == 128
    t = [graphs.tensor(1, "X", [1, 4], "INT4"), graphs.tensor(2, "S", [1, 2], "HALF"), graphs.tensor(3, "Y", [1, 4], "BFLOAT16")]
    wl, s = session(graphs.document("int4", [graphs.dequantize_node("d", 1, 2, 3, [2])], t),
                    {1: lambda: np.array([0xf8, 0x70], np.uint8), 2: lambda: np.array([0x3800, 0x4000], np.uint16)}, [3])
    assert s.raw(3).view(np.uint16).tolist() == [0xc080, 0xbf00, 0x0000, 0x4160]
    wl, s = session(roundtrip(96, 256, 16), {14: workloads._normal(9, 14, 96 * 256, "FLOAT", 3.0)}, [17])
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    assert np.array_equal(s.output(17).view(np.uint32), ref[17].view(np.uint32))
    assert dfgpu.device_status() == 0


def test_every_pointwise_mode_through_the_executable():
    """The reference's all-modes graph (test/Compiler/FoundationalMathOpsTest.cpp:126-167, inputs :617-619): 50 POINTWISE nodes
    over A [2, 3], B [3], T [2, 1], each answer within the reference test's own 3e-4 + 3e-4 |expected| of its f64 formulas
    (:440-556); then the same graph on 64 x 48 seeded values, and in BFLOAT16 against the oracle."""
    import pointwise_reference as reference
    from deepforge_b200 import graphs

    def session(doc, inputs):
        outputs = [1000 + i for i in range(len(graphs.SCHEMA_POINTWISE_MODES))]
        wl = workloads.Workload(name="pointwise_all_modes", config=0, document=doc, description={}, metric="", unit="GB/s", flops=1.0, bytes=1.0,
                                bound="hbm", inputs=inputs, outputs=outputs)
        s = harness.Session(wl)
        s.run()
        return wl, s

    wl, s = session(graphs.pointwise_all_modes(), {101: lambda: reference.A.copy(), 102: lambda: reference.B.copy(), 103: lambda: reference.T.copy()})
    assert s.exe.launch_count == 50
    for position, mode in enumerate(graphs.SCHEMA_POINTWISE_MODES):
        reference.assert_close(mode, s.output(1000 + position), reference.expected(mode, reference.A.reshape(2, 3), reference.B, reference.T))

    rng = np.random.default_rng(4321)
    a = (np.round(rng.uniform(-3.0, 3.0, (64, 48)) * 8) / 8).astype(np.float32)
    b = (np.round(rng.uniform(-3.0, 3.0, 48) * 8) / 8).astype(np.float32)
    t = (rng.integers(0, 2, 64) * rng.uniform(-2.0, 2.0, 64)).astype(np.float32)
    wl, s = session(graphs.pointwise_all_modes((64, 48)), {101: lambda: a.reshape(-1).copy(), 102: lambda: b.copy(), 103: lambda: t.copy()})
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    for position, mode in enumerate(graphs.SCHEMA_POINTWISE_MODES):
        reference.assert_close(mode, s.output(1000 + position), reference.expected(mode, a, b, t))
        reference.assert_close(mode, s.output(1000 + position), ref[1000 + position], 2e-6, 2e-6)

    wl, s = session(graphs.pointwise_all_modes((64, 48), "BFLOAT16"),
                    {101: lambda: synthetic.to_bf16_bits(a.reshape(-1)), 102: lambda: synthetic.to_bf16_bits(b), 103: lambda: synthetic.to_bf16_bits(t)})
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    for position, mode in enumerate(graphs.SCHEMA_POINTWISE_MODES):
        reference.assert_close(mode, s.output(1000 + position), ref[1000 + position], 1e-30, 2.0 ** -7)   # one bf16 step


def test_pass_by_value_scalars_reproduce_the_reference_known_answers():
    """test/Compiler/FoundationalMathOpsTest.cpp:190-221,662-800. A runtime scalar stays an ordinary one-element read
    argument (2.5 added to 1..6 gives 3.5..8.5); an embedded scalar (FLOAT bits 40200000 = 2.5) is owned by the graph:
    absent from the argument table, written into the workspace by the plan's first launch, the same answers, a
    pointer the caller passes for its UID is ignored, and an artifact carries it."""
    from deepforge_b200 import graphs
    x = np.array([1, 2, 3, 4, 5, 6], np.float32)
    expected = [3.5, 4.5, 5.5, 6.5, 7.5, 8.5]

    def session(doc, inputs):
        wl = workloads.Workload(name="scalar", config=0, document=doc, description={}, metric="", unit="GB/s", flops=1.0, bytes=1.0, bound="hbm",
                                inputs=inputs, outputs=[603])
        s = harness.Session(wl)
        s.run()
        return wl, s

    wl, s = session(graphs.scalar_pointwise(), {601: lambda: x.copy(), 602: lambda: np.array([2.5], np.float32)})
    scalar = [a for a in s.exe.arguments() if a["uid"] == 602][0]
    assert scalar["access"] == "read" and scalar["size_bytes"] == 4 and s.exe.workspace_size == 0
    assert s.output(603).tolist() == expected

    embedded = graphs.scalar_pointwise({"index": 3, "value": "40200000"})
    wl, s = session(embedded, {601: lambda: x.copy()})
    assert [a["uid"] for a in s.exe.arguments()] == [601, 603] and s.exe.workspace_size == 64 and s.exe.launch_count == 2
    assert s.output(603).tolist() == expected
    ins, _ = oracle_inputs(wl, s)
    assert graph_oracle.run(wl.document, ins)[603].tolist() == expected
    # the caller cannot override a graph-owned scalar
    wl, s = session(embedded, {601: lambda: x.copy(), 602: lambda: np.array([100.0], np.float32)})
    assert s.output(603).tolist() == expected
    # and the artifact carries it
    loaded = runtime.load_artifact(s.exe.serialize())
    assert loaded.plan_text() == s.exe.plan_text() and [a["uid"] for a in loaded.arguments()] == [601, 603]
    s.dev[603].zero_()
    s.exe = loaded
    s.run()
    assert s.output(603).tolist() == expected
    # HALF and BFLOAT16 payloads are JSON numbers, narrowed to the tensor's type: x * 1.5 and x * -2
    for data_type, payload, factor in (("HALF", {"index": 2, "value": 1.5}, 1.5), ("BFLOAT16", {"index": 5, "value": -2.0}, -2.0)):
        wl, s = session(graphs.scalar_pointwise(payload, mode="MUL", data_type=data_type), {601: lambda: x.copy()})
        assert s.output(603).tolist() == (x * factor).tolist()


def _quantize_slabs(document, node_index, uid, storage, slabs):
    """The oracle's block-scale quantize over independent slabs of one operand (whole 32-element blocks each), on
    host threads; returns (codes, scales) joined in slab order."""
    from concurrent.futures import ThreadPoolExecutor
    node = document["nodes"][node_index]
    y, scale = node["outputs"]["Y"], node["outputs"]["scale"]

    def one(slab):
        sub_document, sub_storage = slab
        out = graph_oracle.run({**sub_document, "nodes": [sub_document["nodes"][node_index]]}, {}, storage_inputs={uid: sub_storage})
        return out[y], out[scale]

    with ThreadPoolExecutor(max_workers=THREADS) as pool:
        parts = list(pool.map(one, slabs))
    return np.concatenate([p[0] for p in parts]), np.concatenate([p[1] for p in parts])


def test_c3_full_size_every_code_and_scale_exact_and_matmul_rows():
    """The benchmark configuration: all 2 x 16.8 M codes and 2 x 524,288 scales byte for byte against the oracle's
    candidate search, and C on 256 rows spread over the matrix (every 16th)."""
    wl = workloads.c3()
    s = harness.Session(wl)
    s.run()
    _, storage = oracle_inputs(wl, s)
    m = k = n = 4096
    # A is quantized along K inside each row: slabs of rows. B along K down each column: slabs of 32 K-rows.
    rows = 128
    a_doc = workloads.c3(m=rows, k=k, n=n).document
    aq, sfa = _quantize_slabs(a_doc, 0, 1, storage[1], [(a_doc, storage[1][r * k:(r + rows) * k]) for r in range(0, m, rows)])
    assert np.array_equal(s.output(3), aq), "Aq"
    assert np.array_equal(s.output(4), sfa), "SFA"
    depth = 128
    b_doc = workloads.c3(m=m, k=depth, n=n).document
    bq, sfb = _quantize_slabs(b_doc, 1, 2, storage[2], [(b_doc, storage[2][r * n:(r + depth) * n]) for r in range(0, k, depth)])
    assert np.array_equal(s.output(5), bq), "Bq"
    assert np.array_equal(s.output(6), sfb), "SFB"
    # C rows 0, 16, 32, ...: dequantize (exact) and multiply in the oracle, f32 with k in order
    picked = np.arange(0, m, 16)
    from oracle import tensor as T
    import oracle
    a_rows = np.ascontiguousarray(aq.reshape(m, k)[picked]).reshape(-1)
    s_rows = np.ascontiguousarray(sfa.reshape(m, k // 32)[picked]).reshape(-1)
    af = np.zeros(picked.size * k, dtype=np.float32)
    oracle.block_scale_dequantize(T(dfgpu.E4M3, [picked.size, k]), a_rows, T(dfgpu.E8M0, [picked.size, k // 32]), s_rows, T(dfgpu.F32, [picked.size, k]), af, [1, 32])
    bf = np.zeros(k * n, dtype=np.float32)
    oracle.block_scale_dequantize(T(dfgpu.E4M3, [k, n]), bq, T(dfgpu.E8M0, [k // 32, n]), sfb, T(dfgpu.F32, [k, n]), bf, [32, 1])
    c_ref = np.zeros(picked.size * n, dtype=np.float32)
    oracle.matmul(T(dfgpu.F32, [picked.size, k]), af, T(dfgpu.F32, [k, n]), bf, T(dfgpu.F32, [picked.size, n]), c_ref, threads=THREADS)
    check_bf16(s.output(9).reshape(m, n)[picked], c_ref.reshape(picked.size, n))


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


def test_c4_sdpa_full_size_whole_heads():
    """The benchmark configuration: every query row of eight (batch, head) pairs, the first and the last among them."""
    wl = workloads.c4()
    s = harness.Session(wl)
    s.run()
    ins, _ = oracle_inputs(wl, s)
    out = s.output(4).reshape(8, 32, 2048, 128)
    stats = s.output(5).reshape(8, 32, 2048)
    pairs = [0, 1, 3 * 32 + 17, 4 * 32, 5 * 32 + 9, 6 * 32 + 30, 7 * 32 + 30, 7 * 32 + 31]
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=THREADS) as pool:
        references = list(pool.map(lambda bh: graph_oracle.run(wl.document, ins, sdpa_bh=(bh, bh + 1)), pairs))
    for bh, ref in zip(pairs, references):
        b, h = divmod(bh, 32)
        check_bf16(out[b, h], ref[4].reshape(8, 32, 2048, 128)[b, h])
        r = ref[5].reshape(8, 32, 2048)[b, h]
        assert np.all(np.abs(stats[b, h] - r) <= 2e-3 * (1 + np.abs(r)))
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


def test_c5_paged_decode_with_compact_page_tables():
    """The same decode with compact page tables (the graph names the offsets in the tables' tensor entries): same plan
    kernel, one launch more, results equal to the oracle's and bit for bit to the strided-table run of the same pages."""
    sizes = dict(batch=6, hq=8, hkv=2, pages=64, block=64, max_len=1024, min_len=1)
    wl = workloads.c5(compact=True, **sizes)
    s = harness.Session(wl)
    assert "kernel=4 launches=3" in s.exe.plan_text() and "uid9 uid10" in s.exe.plan_text()
    s.run()
    ins, _ = oracle_inputs(wl, s)
    ref = graph_oracle.run(wl.document, ins)
    check_bf16(s.output(4), ref[4])
    strided = harness.Session(workloads.c5(**sizes))
    strided.run()
    assert np.array_equal(s.output(4), strided.output(4))
    assert dfgpu.device_status() == 0


def test_c5_paged_decode_full_size_ten_sequences():
    """The benchmark configuration: all 32 heads of ten sequences, the shortest and the longest of the batch among them."""
    wl = workloads.c5()
    s = harness.Session(wl)
    s.run()
    out = s.output(4).reshape(64, 32, 128)
    ins, storage = oracle_inputs(wl, s, keep_in_storage=(2, 3))  # the 2 x 2.1 GB pools stay bf16 on the host
    lengths = ins[6]
    chosen = sorted({int(np.argmin(lengths)), int(np.argmax(lengths)), 0, 7, 19, 28, 41, 50, 57, 63})
    assert len(chosen) >= 8
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=THREADS) as pool:
        references = list(pool.map(lambda b: graph_oracle.run(wl.document, ins, sdpa_bh=(b * 32, b * 32 + 32), storage_inputs=storage), chosen))
    for b, ref in zip(chosen, references):
        check_bf16(out[b], ref[4].reshape(64, 32, 128)[b])
    # linearity in V: doubling the V pool doubles the output (bf16 doubling is exact)
    import torch
    s.dev[3].view(torch.bfloat16).mul_(2)
    s.run()
    doubled = s.output(4).reshape(64, 32, 128)
    assert np.array_equal(doubled, out * 2)


@pytest.mark.parametrize("name,size", [("c2", dict(n=4, h=14, w=14)), ("c3", dict(m=256, k=128, n=128)), ("c4", dict(b=2, h=2, s=256)),
                                       ("c5", dict(batch=4, hq=8, hkv=2, pages=32, max_len=512, min_len=100))])
def test_shards_run_one_after_another_join_into_the_unsharded_result(name, size):
    """What the multi-GPU benchmark runs, on one GPU: the shards workloads.shard cuts for two ranks (their own slices of the
    input streams, kernel selection at the shard's size) executed in turn; their outputs, joined along the gather axis,
    are the unsharded run's outputs bit for bit (which the tests above hold to the oracle)."""
    whole = harness.Session(workloads.BUILDERS[name](**size))
    whole.run()
    parts = []
    for rank in range(2):
        shard = harness.Session(workloads.shard(name, rank, 2, **dict(size)))
        shard.run()
        parts.append({uid: shard.raw(uid).copy() for uid in workloads.GATHER_AXIS[name]})
        del shard
    for uid, axis in workloads.GATHER_AXIS[name].items():
        assert axis == 0  # (every sharded output is split along its slowest axis: joining is concatenation)
        joined = np.concatenate([part[uid].reshape(-1) for part in parts])
        assert np.array_equal(joined.view(np.uint8), whole.raw(uid).reshape(-1).view(np.uint8)), (name, uid)


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


def test_two_threads_execute_one_executable_concurrently():
    """The reference's concurrency case (test/Compiler/CompilerTest.cpp:405-432): two threads call execute on ONE
    executable with the same inputs, separate outputs and separate workspaces; both succeed and agree bit for bit.
    Here once through execute() (shared stream: whole plans are enqueued one after the other) and once through
    execute_on() with a stream per thread (no lock: the plans also overlap on the device), repeated to give the two
    threads many chances to interleave."""
    import threading
    import torch
    wl = workloads.c2(n=2, h=28, w=28)
    s = harness.Session(wl)
    s.run()
    expected = s.raw(7).copy()
    size = s.exe.workspace_size
    outputs = [torch.full_like(s.dev[7], 0x7f) for _ in range(2)]
    spaces = [torch.empty(max(size, 1), dtype=torch.uint8, device=s.device) for _ in range(2)]
    streams = [torch.cuda.Stream(s.device) for _ in range(2)]
    packs = [{**s.pack, 7: out.data_ptr()} for out in outputs]
    for own_stream in (False, True):
        for out in outputs:
            out.fill_(0x7f)
        torch.cuda.synchronize()
        errors = []

        def work(i):
            try:
                for _ in range(50):
                    if own_stream:
                        s.exe.execute_on(streams[i].cuda_stream, packs[i], spaces[i].data_ptr())
                    else:
                        s.exe.execute(packs[i], spaces[i].data_ptr())
            except Exception as error:  # noqa: BLE001 - reported below, in the main thread
                errors.append(error)

        threads = [threading.Thread(target=work, args=(i,)) for i in range(2)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        torch.cuda.synchronize()
        assert not errors, errors
        for out in outputs:
            assert np.array_equal(out.cpu().numpy(), expected)
