"""Host side without a GPU: importer protocol rules and error codes, the workspace planner's
known answers, kernel-selection plans, the argument table and the runtime's variant-pack
checks (all of which fail before any CUDA call).

Reference behaviour being mirrored:
  test/Import/SerializedGraphImporterTest.cpp:393-605,806-848  stable error codes per mutation
  test/Transforms/BufferizationTest.cpp:95-136                placement a@0, c@64, b@0, total 192
  test/Compiler/CompilerTest.cpp:318-403                      runtime negatives (code 17)
"""
import copy
import json

import pytest

from deepforge_b200 import graphs, runtime
from deepforge_b200.runtime import DeepForgeError

OK_DOC = graphs.c1_conv(n=1, c=3, h=5, w=5, k=5)


def code_of(document, fmt=runtime.FORMAT_AUTO):
    try:
        runtime.parse(document, fmt)
    except DeepForgeError as error:
        return error.code
    return 0


def mutated(fn):
    doc = copy.deepcopy(OK_DOC)
    fn(doc)
    return doc


def test_exports_of_the_host_library():
    lib = runtime.load()
    import re
    from pathlib import Path
    header = (Path(__file__).resolve().parent.parent / "include" / "deepforge_b200.h").read_text()
    declared = sorted(set(re.findall(r"\b(df_[a-z0-9_]+)\s*\(", header)))
    assert declared == sorted(runtime.EXPORTS)
    for name in declared:
        assert hasattr(lib, name)


def test_accepts_reference_fixture_shape_and_all_five_configs():
    assert runtime.parse(OK_DOC) == (3, 1)
    assert runtime.parse(json.dumps(OK_DOC), runtime.FORMAT_JSON) == (3, 1)
    for doc in (graphs.c2_bottleneck(n=1, h=8, w=8), graphs.c3_quantize_matmul(128, 128, 128), graphs.c4_sdpa(1, 2, 16, 8), graphs.c5_paged_decode(2, 4, 2, 16, 8, 4, 16)):
        runtime.parse(doc)


@pytest.mark.parametrize("mutation,expected", [
    (lambda d: d.update(json_version="1.1"), 4),
    (lambda d: d.update(cudnn_frontend_version=12300), 5),
    (lambda d: d.pop("context"), 6),
    (lambda d: d["context"].pop("sm_count"), 6),
    (lambda d: d["context"].update(extra=1), 8),
    (lambda d: d.update(unknown_top_level=1), 0),                        # tolerated, as in the reference
    (lambda d: d["tensors"]["1"].update(bogus=1), 8),
    (lambda d: d["tensors"]["1"].pop("stride"), 6),
    (lambda d: d["tensors"]["1"].update(dim="x"), 7),
    (lambda d: d["tensors"]["1"].update(data_type="COMPLEX"), 10),
    (lambda d: d["tensors"]["1"].update(uid=9), 8),                      # key/UID mismatch
    (lambda d: d["tensors"]["1"].update(uid_assigned=False), 8),         # a tensor without a UID is keyed by its name
    (lambda d: (d["tensors"].update(X=d["tensors"].pop("1")), d["tensors"]["X"].update(uid_assigned=False)), 13),
    (lambda d: d["tensors"]["1"].update(dim=[1, 3, 0, 5]), 15),
    (lambda d: d["tensors"]["1"].update(dim=[2 ** 40, 2 ** 40, 5, 5]), 16),
    (lambda d: d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value=1.0), 7),   # a payload is the Frontend's scalar variant object
    (lambda d: d["tensors"]["1"].update(is_pass_by_value=True), 11),                      # the single-node convolution takes no scalars
    (lambda d: d["tensors"]["1"].update(reordering_type="F16x16"), 14),  # a Frontend reordering, not NONE: the single-node graph's layout rule
    (lambda d: d["tensors"]["1"].update(reordering_type="ZIGZAG"), 8),
    (lambda d: d["nodes"][0].update(tag="LAYER_NORM"), 9),
    (lambda d: d["nodes"][0].update(tag="NOT_A_TAG"), 9),
    (lambda d: d["nodes"][0].pop("math_mode"), 6),
    (lambda d: d["nodes"][0].update(surprise=True), 8),
    (lambda d: d["nodes"][0]["inputs"].update(Z=1), 8),
    (lambda d: d["nodes"][0]["inputs"].update(X=42), 13),
    (lambda d: d["nodes"][0]["inputs"].update(X="X"), 13),               # name references are not accepted
    (lambda d: d["nodes"][0]["outputs"].update(Y=1), 0),                 # writes a tensor it reads: parsed, refused by the lowering (20)
    (lambda d: d["context"].update(is_dynamic_shape_enabled=True), 11),
    (lambda d: d.update(fe_workspace_size=64), 11),
    (lambda d: d.update(workspace_modifications={"1": [0, 1, 2]}), 11),
    (lambda d: d.update(variant_pack_replacements=[[1, 2]]), 11),
    (lambda d: d.update(variant_pack_uids=[1, 2]), 11),
    (lambda d: d["tensors"].update({"4": graphs.tensor(4, "Unused", [1])}), 8),
])
def test_importer_error_codes(mutation, expected):
    assert code_of(mutated(mutation)) == expected


def test_importer_rejects_broken_encodings_and_sizes():
    assert code_of(b"") == 1
    assert code_of(b"{not json", runtime.FORMAT_JSON) == 3
    assert code_of(json.dumps(OK_DOC) + " trailing", runtime.FORMAT_JSON) == 3
    assert code_of(b"\x00" * 16, runtime.FORMAT_UBJSON) == 3
    assert code_of(b" " * (16 * 1024 * 1024 + 1)) == 1
    assert code_of(b"\xff\xfe\x00garbage") == 3


def test_virtual_tensor_consumed_before_produced_is_rejected():
    doc = graphs.c2_bottleneck(n=1, h=8, w=8)
    doc["nodes"][0], doc["nodes"][1] = doc["nodes"][1], doc["nodes"][0]
    assert code_of(doc) == 8


def test_workspace_planner_known_answer():
    plan = runtime.plan_workspace([
        {"name": "a", "size_bytes": 64, "alignment": 64, "live_start": 0, "live_end": 3},
        {"name": "b", "size_bytes": 64, "alignment": 64, "live_start": 4, "live_end": 7},
        {"name": "c", "size_bytes": 96, "alignment": 32, "live_start": 2, "live_end": 5},
    ])
    assert plan["order"] == ["a", "c", "b"]
    assert plan["offsets"] == {"a": 0, "c": 64, "b": 0}
    assert plan["total"] == 192
    assert runtime.plan_workspace([{"name": "pad", "size_bytes": 588, "alignment": 64, "live_start": 0, "live_end": 0}])["total"] == 640


@pytest.mark.parametrize("requests,expected", [
    ([{"name": "a", "size_bytes": 8, "alignment": 3, "live_start": 0, "live_end": 1}], 1),
    ([{"name": "a", "size_bytes": 8, "alignment": 128, "live_start": 0, "live_end": 1}], 1),
    ([{"name": "a", "size_bytes": 0, "alignment": 8, "live_start": 0, "live_end": 1}], 1),
    ([{"name": "a", "size_bytes": 8, "alignment": 8, "live_start": 2, "live_end": 1}], 1),
    ([{"name": "a", "size_bytes": 8, "alignment": 8, "live_start": 0, "live_end": 1}] * 2, 8),
    ([{"name": "a", "size_bytes": 2 ** 63 - 1, "alignment": 64, "live_start": 0, "live_end": 1}], 16),
])
def test_workspace_planner_rejections(requests, expected):
    with pytest.raises(DeepForgeError) as error:
        runtime.plan_workspace(requests)
    assert error.value.code == expected


def test_bottleneck_plan_fuses_to_three_launches_and_shares_workspace():
    # default plan: conv1 with its bias and ReLU, then conv2 and conv3 with everything around them in one launch of the
    # two-convolution kernel; the tensor between those two never exists in memory, so the workspace holds one intermediate
    # of 2*8*8*64 elements, stored as (hi, lo) bf16 pairs: FLOAT's 4 bytes per element
    fused = runtime.compile_graph(graphs.c2_bottleneck(n=2, h=8, w=8))
    assert fused.launch_count == 2 and fused.workspace_size == 2 * 8 * 8 * 64 * 4
    assert "conv_fprop kernel=3 launches=1 [conv1+bias1+relu1]" in fused.plan_text()
    assert "conv_fprop_pair kernel=1 launches=1 [conv2+bias2+relu2>conv3+residual]" in fused.plan_text()
    exe = runtime.compile_graph(graphs.c2_bottleneck(n=2, h=8, w=8), options=runtime.NO_CONV_PAIRS)
    text = exe.plan_text()
    assert exe.launch_count == 3
    assert "[conv1+bias1+relu1]" in text and "[conv2+bias2+relu2]" in text and "[conv3+residual]" in text
    assert text.count("kernel=3") == 3  # tcgen05 implicit GEMM for all three
    # two intermediates, alive at the same time
    assert exe.workspace_size == 2 * (2 * 8 * 8 * 64 * 4)
    # the lossy option stores them as single bf16 values
    lossy = runtime.compile_graph(graphs.c2_bottleneck(n=2, h=8, w=8), options=runtime.BF16_INTERMEDIATES)
    assert lossy.plan_text().count("kernel=3") == 3 and lossy.workspace_size == 2 * (2 * 8 * 8 * 64 * 2)
    # without narrowing the intermediates stay FLOAT: the first convolution still runs on tcgen05, its readers on CUDA cores
    plain = runtime.compile_graph(graphs.c2_bottleneck(n=2, h=8, w=8), options=runtime.NO_NARROWING)
    assert plain.plan_text().count("kernel=3") == 1 and plain.workspace_size == 2 * (2 * 8 * 8 * 64 * 4)
    unfused = runtime.compile_graph(graphs.c2_bottleneck(n=2, h=8, w=8), options=runtime.NO_FUSION)
    assert unfused.launch_count == 8
    f32 = runtime.compile_graph(graphs.c2_bottleneck(n=2, h=8, w=8, io="FLOAT"))
    # an all-FLOAT graph: convolutions of at most 148 output tiles with a reduction depth of 128 or more (conv1: 256, conv2: 576) run on
    # tcgen05 in one cluster launch each, conv3 (depth 64) on CUDA cores; no scratch either way
    assert f32.plan_text().count("conv_fprop kernel=5 launches=1") == 2 and f32.plan_text().count("kernel=2") == 1
    assert f32.launch_count == 3 and f32.workspace_size == 2 * (2 * 8 * 8 * 64 * 4)
    # with more than 148 output tiles (128 pixels x 64 channels), from 2^24 multiply-adds on, a convolution is three launches (split,
    # convolution over six-piece operands, the guarded CUDA-core pass) and needs scratch for the split copies
    medium = runtime.compile_graph(graphs.c2_bottleneck(n=8, h=28, w=28, io="FLOAT"))   # 49 pixel tiles: conv3 (256 channels) has 196
    assert medium.plan_text().count("conv_fprop kernel=5 launches=1") == 2 and medium.plan_text().count("conv_fprop kernel=4 launches=3") == 1
    assert medium.launch_count == 5 and medium.plan_text().count("scratch=ws+") == 1
    # (with more tiles the one-launch form stays where all output channels fit one 64-channel tile: conv1 and conv2)
    large = runtime.compile_graph(graphs.c2_bottleneck(n=32, h=28, w=28, io="FLOAT"))
    assert large.plan_text().count("conv_fprop kernel=5 launches=1") == 2 and large.plan_text().count("conv_fprop kernel=4 launches=3") == 1
    assert large.launch_count == 5 and large.plan_text().count("scratch=ws+") == 1 and large.workspace_size > 2 * (32 * 28 * 28 * 64 * 4)
    cores = runtime.compile_graph(graphs.c2_bottleneck(n=8, h=28, w=28, io="FLOAT"), options=runtime.NO_TENSOR_CORES)
    assert cores.plan_text().count("kernel=2") == 3 and cores.workspace_size == 2 * (8 * 28 * 28 * 64 * 4)


def test_quantize_matmul_plans():
    # MXFP8 shape: the block-scaled tensor-core matmul reads codes and scales itself, no dequantize launch, no workspace
    # and the two quantize nodes (bf16, independent of each other) share one launch
    exe = runtime.compile_graph(graphs.c3_quantize_matmul(128, 128, 128))
    assert exe.launch_count == 2 and exe.workspace_size == 0
    assert "block_scale_quantize_pair kernel=1 launches=1 [quantize_a|quantize_b]" in exe.plan_text()
    assert "matmul kernel=3" in exe.plan_text() and "[dequantize_b+dequantize_a+matmul]" in exe.plan_text()
    # only the bf16 tensor-core kernel fits (N is not a multiple of 128): dequantize stays a launch whose
    # output is stored as bf16 (exact), matmul on tcgen05
    exe = runtime.compile_graph(graphs.c3_quantize_matmul(128, 128, 64))
    assert exe.launch_count == 4 and exe.workspace_size == 128 * 128 * 2 + 128 * 64 * 2
    assert "matmul kernel=2" in exe.plan_text()
    # shapes the tcgen05 kernel does not cover: the dequantize nodes are absorbed into the CUDA-core matmul
    for doc, options in ((graphs.c3_quantize_matmul(128, 128, 96), 0), (graphs.c3_quantize_matmul(128, 128, 128), runtime.NO_TENSOR_CORES)):
        absorbed = runtime.compile_graph(doc, options=options)
        assert absorbed.launch_count == 2 and absorbed.workspace_size == 0
        assert "[dequantize_b+dequantize_a+matmul]" in absorbed.plan_text()
    # FLOAT inputs keep one launch per quantize node (the shared launch is the bf16 form)
    assert runtime.compile_graph(graphs.c3_quantize_matmul(128, 128, 128, io="FLOAT")).launch_count == 3
    unfused = runtime.compile_graph(graphs.c3_quantize_matmul(128, 128, 96), options=runtime.NO_FUSION)
    assert unfused.launch_count == 5 and unfused.workspace_size == 128 * 128 * 4 + 128 * 96 * 4


def test_argument_table_is_sorted_with_clamped_alignment():
    # the reference's rule, clamp(element bytes, 1, 8), wherever no TMA-fed kernel reads the argument
    exe = runtime.compile_graph(graphs.c3_quantize_matmul(128, 128, 128), options=runtime.NO_TENSOR_CORES | runtime.NO_FUSION)
    arguments = exe.arguments()
    assert [a["uid"] for a in arguments] == [1, 2, 3, 4, 5, 6, 9]
    by_uid = {a["uid"]: a for a in arguments}
    assert by_uid[1]["alignment"] == 2 and by_uid[3]["alignment"] == 1 and by_uid[9]["alignment"] == 2
    # arguments bound to a tcgen05 / TMA launch advertise the 16 bytes (scales: 4) that launch needs, so that
    # execute() refuses a misaligned variant pack before anything is launched
    exe = runtime.compile_graph(graphs.c3_quantize_matmul(128, 128, 128))
    by_uid = {a["uid"]: a for a in exe.arguments()}
    assert by_uid[1]["alignment"] == 16 and by_uid[3]["alignment"] == 16 and by_uid[5]["alignment"] == 16 and by_uid[9]["alignment"] == 16
    assert by_uid[4]["alignment"] == 8 and by_uid[6]["alignment"] == 8  # 4 for the matmul's scale loads, 8 for the shared quantize launch's stores
    assert by_uid[1]["access"] == "read" and by_uid[3]["access"] == "readwrite" and by_uid[9]["access"] == "write"
    assert by_uid[4]["size_bytes"] == 128 * 4
    decode = runtime.compile_graph(graphs.c5_paged_decode(2, 4, 2, 128, 8, 64, 256))
    assert {a["uid"]: a["alignment"] for a in decode.arguments()}[5] == 4


@pytest.mark.parametrize("doc_fn,expected", [
    (lambda: graphs.c4_sdpa(1, 2, 16, 8, io="HALF"), 0),
    (lambda: _with(graphs.c4_sdpa(1, 2, 16, 8), lambda d: d["nodes"][0].update(alibi_mask=True)), 0),
    (lambda: _with(graphs.c4_sdpa(1, 2, 16, 8), lambda d: d["nodes"][0].update(alibi_mask=True, diagonal_alignment="BOTTOM_RIGHT")), 20),
    (lambda: _with(graphs.c4_sdpa(1, 2, 16, 8), lambda d: d["nodes"][0].update(dropout_probability=0.1)), 8),   # (probability dropout without Seed and Offset)
    (lambda: _with(graphs.c4_sdpa(1, 2, 16, 8), lambda d: d["nodes"][0].update(dropout_probability=1.0)), 8),
    (lambda: _with(graphs.c4_sdpa(1, 2, 16, 8), lambda d: d["nodes"][0].update(generate_stats=False)), 8),
    (lambda: _with(graphs.c2_bottleneck(n=1, h=8, w=8), lambda d: d["nodes"][2].update(mode="GELU_SQUARED_FWD")), 7),   # not a mode of the schema: refused at import
    (lambda: _with(graphs.c2_bottleneck(n=1, h=8, w=8), lambda d: d["nodes"][2].update(mode="GEN_INDEX")), 8),          # no axis
    (lambda: _with(graphs.c2_bottleneck(n=1, h=8, w=8), lambda d: d["nodes"][2].update(mode="SOFTPLUS_FWD", softplus_beta=0.0)), 8),
    (lambda: _with(graphs.c2_bottleneck(n=1, h=8, w=8), lambda d: d["nodes"][2].update(mode="TANH_BWD")), 8),           # two inputs wanted
    (lambda: _with(graphs.c1_conv(n=1, c=3, h=5, w=5, k=5), lambda d: d["tensors"]["3"].update(dim=[1, 5, 4, 5], stride=[100, 1, 25, 5])), 15),
    (lambda: _with(graphs.c3_quantize_matmul(128, 128, 128), lambda d: d["tensors"]["3"].update(data_type="INT8")), 10),
    (lambda: _with(graphs.c3_quantize_matmul(128, 128, 128), lambda d: d["nodes"][0].update(block_size=24)), 15),
])
def test_compile_time_rejections(doc_fn, expected):
    try:
        runtime.compile_graph(doc_fn())
        code = 0
    except DeepForgeError as error:
        code = error.code
    assert code == expected


def _with(doc, fn):
    fn(doc)
    return doc


def test_runtime_rejects_bad_variant_packs_before_any_launch():
    """Missing UID, null, misaligned, write aliasing, workspace problems: all DFE_INVALID_VARIANT_PACK (17)."""
    exe = runtime.compile_graph(graphs.c2_bottleneck(n=1, h=8, w=8))
    sizes = {a["uid"]: a["size_bytes"] for a in exe.arguments()}
    base = 0x10000000
    good, cursor = {}, base
    for uid, size in sizes.items():
        good[uid] = cursor
        cursor += (size + 255) // 256 * 256
    workspace = cursor + 4096

    def code(pack, ws):
        try:
            exe.execute(pack, ws)
        except DeepForgeError as error:
            assert str(error).startswith("DFE_")
            return error.code
        return 0

    missing = dict(good)
    del missing[7]
    assert code(missing, workspace) == 17
    assert code({**good, 1: 0}, workspace) == 17
    assert code({**good, 1: good[1] + 1}, workspace) == 17           # bf16 needs 2-byte alignment
    assert code({**good, 7: good[1]}, workspace) == 17               # output aliases an input
    assert code({**good, 7: good[1] + 64}, workspace) == 17          # partial overlap with a written tensor
    assert code(good, 0) == 17                                       # workspace required but null
    assert code(good, workspace + 8) == 17                           # workspace misaligned
    assert code(good, good[7]) == 17                                 # workspace overlaps an argument


def test_single_convolution_carries_the_conv_adapter_metadata():
    """The reference's single-node path (lib/MLIR/Conv2DImporter.cpp:332-370, checks of lib/Runtime/Executable.cpp:735-768):
    arguments X, W, Y by those names and in that order whatever their UIDs, FLOAT, physical NHWC / KRSC shapes with packed
    strides, alignment 4, read / read / write; UIDs, shapes, the padded input shape and the attributes in the metadata."""
    doc = graphs.c1_conv("nhwc", n=2, c=16, h=9, w=7, k=8)
    # UIDs out of order on purpose: Y has the smallest
    renumber = {"1": 30, "2": 20, "3": 10}
    doc["tensors"] = {str(renumber[k]): {**t, "uid": renumber[k]} for k, t in doc["tensors"].items()}
    node = doc["nodes"][0]
    node["inputs"] = {"X": 30, "W": 20}
    node["outputs"] = {"Y": 10}
    exe = runtime.compile_graph(doc)
    arguments = exe.arguments()
    assert [(a["name"], a["uid"], a["access"], a["alignment"]) for a in arguments] == [("X", 30, "read", 4), ("W", 20, "read", 4), ("Y", 10, "write", 4)]
    assert [a["size_bytes"] for a in arguments] == [2 * 9 * 7 * 16 * 4, 8 * 3 * 3 * 16 * 4, 2 * 9 * 7 * 8 * 4]
    meta = exe.conv2d_metadata()
    assert meta == {"x_uid": 30, "w_uid": 20, "y_uid": 10, "x_shape": [2, 9, 7, 16], "w_shape": [8, 3, 3, 16], "y_shape": [2, 9, 7, 8],
                    "padded_x_shape": [2, 11, 9, 16], "pre_padding": [1, 1], "post_padding": [1, 1], "stride": [1, 1], "dilation": [1, 1]}
    # the artifact describes itself the same way after a round trip
    loaded = runtime.load_artifact(exe.serialize())
    assert loaded.arguments() == arguments and loaded.conv2d_metadata() == meta
    # everything else keeps the generic table: the NCHW-strided extension, a convolution inside a DAG
    assert runtime.compile_graph(graphs.c1_conv("nchw", n=1, c=4, h=5, w=5, k=4)).conv2d_metadata() is None
    generic = runtime.compile_graph(graphs.c2_bottleneck(n=1, h=8, w=8))
    assert generic.conv2d_metadata() is None and [a["uid"] for a in generic.arguments()] == sorted(a["uid"] for a in generic.arguments())


def test_compact_page_tables_plan_metadata_and_rejections(tmp_path):
    """Compact (ragged batch-prefix) page tables: the SDPA launch binds the two offset tensors, gains the validation
    launch and its scratch, the artifact keeps all of it; ragged storage anywhere else is refused, and so are offsets of
    the wrong shape or a dangling reference (lib/Compiler/SequenceGraph.cpp:741-773)."""
    strided = runtime.compile_graph(graphs.c5_paged_decode(batch=4, pages=64, block=64, max_len=1024))
    doc = graphs.c5_paged_decode(batch=4, pages=64, block=64, max_len=1024, compact=True)
    exe = runtime.compile_graph(doc)
    assert "sdpa_forward kernel=4 launches=2" in strided.plan_text() and "sdpa_forward kernel=4 launches=3" in exe.plan_text()
    assert exe.plan_text().rstrip().endswith("uid9 uid10 - - - - - scratch=ws+0") and exe.workspace_size == strided.workspace_size + 256
    assert [a["uid"] for a in exe.arguments()] == list(range(1, 11))
    target = tmp_path / "compact.dfo"
    exe.write_artifact(target)
    assert runtime.load_artifact(target).plan_text() == exe.plan_text()
    for mutate, expected in (
        (lambda d: d["tensors"]["1"].update(ragged_offset_uid=9, ragged_offset_name="Page_table_K_offsets"), 20),   # ragged Q: not executable here
        (lambda d: d["tensors"]["9"].update(dim=[4, 1, 1, 1], stride=[1, 1, 1, 1]), 15),                             # offsets must be [B+1,1,1,1]
        (lambda d: (d["tensors"]["7"].update(ragged_offset_uid=77), d["tensors"].pop("9")), 13),                       # unresolved offsets tensor
        (lambda d: d["tensors"]["7"].pop("ragged_offset_name"), 8),                                                   # UID and name appear together
        (lambda d: d["tensors"]["10"].update(data_type="FLOAT"), 20),                                                  # offsets are INT32 or INT64
    ):
        broken = copy.deepcopy(doc)
        mutate(broken)
        with pytest.raises(DeepForgeError) as error:
            runtime.compile_graph(broken)
        assert error.value.code == expected, error.value


# ---- pass-by-value scalars (test/Compiler/FoundationalMathOpsTest.cpp:190-262,662-800) ---------------------

def test_runtime_scalar_stays_an_ordinary_read_argument():
    exe = runtime.compile_graph(graphs.scalar_pointwise())
    scalar = [a for a in exe.arguments() if a["uid"] == 602][0]
    assert scalar["access"] == "read" and scalar["size_bytes"] == 4
    assert exe.workspace_size == 0 and exe.plan_text().splitlines() == ["0: pointwise kernel=1 launches=1 [runtime_scalar_add] uid601 uid602 uid603 -"]


def test_embedded_scalar_is_graph_owned_and_survives_the_artifact():
    exe = runtime.compile_graph(graphs.scalar_pointwise({"index": 3, "value": "40200000"}))
    assert [a["uid"] for a in exe.arguments()] == [601, 603]          # absent from the public arguments
    assert exe.workspace_size == 64
    assert exe.plan_text().splitlines() == ["0: constants kernel=1 launches=1 [constants] ws+0(uid602)",
                                            "1: pointwise kernel=1 launches=1 [runtime_scalar_add] uid601 ws+0(uid602) uid603 -"]
    loaded = runtime.load_artifact(exe.serialize())
    assert loaded.plan_text() == exe.plan_text() and loaded.arguments() == exe.arguments() and loaded.workspace_size == 64


def test_every_embedded_scalar_type_is_accepted_and_unused_ones_cost_nothing():
    """all_embedded_scalar_types_graph (:223-247): INT64, INT32, HALF, DOUBLE and BFLOAT16 payloads that no node reads."""
    doc = graphs.scalar_pointwise({"index": 3, "value": "40200000"})
    for uid, data_type, payload in ((604, "INT64", {"index": 0, "value": -7}), (605, "INT32", {"index": 1, "value": 7}),
                                    (606, "HALF", {"index": 2, "value": 1.5}), (607, "DOUBLE", {"index": 4, "value": 1.25}),
                                    (608, "BFLOAT16", {"index": 5, "value": -2.0})):
        described = graphs.tensor(uid, "UNUSED_" + data_type, [1], data_type)
        described.update(is_pass_by_value=True, pass_by_value=payload)
        doc["tensors"][str(uid)] = described
        doc["pass_by_values"][str(uid)] = payload
    exe = runtime.compile_graph(doc)
    assert [a["uid"] for a in exe.arguments()] == [601, 603] and exe.workspace_size == 64 and exe.launch_count == 2


@pytest.mark.parametrize("change,expected", [
    (lambda d: d["tensors"]["602"].update(dim=[1, 2], stride=[2, 1]), 20),            # every dimension must equal one
    (lambda d: d["tensors"]["602"].update(data_type="FP8_E4M3"), 10),                 # outside the Frontend's scalar set
    (lambda d: d["tensors"]["602"].update(is_virtual=True), 8),                        # virtual without a producer
    (lambda d: d["tensors"]["603"].update(is_pass_by_value=True, dim=[1, 1], stride=[1, 1]), 20),   # input-only
])
def test_pass_by_value_rejections(change, expected):
    doc = graphs.scalar_pointwise()
    change(doc)
    try:
        runtime.compile_graph(doc)
        code = 0
    except DeepForgeError as error:
        code = error.code
    assert code == expected
