"""Protocol parity of the importer against the REFERENCE importer itself (oracle/_ref, built from
the reference's own lib/Import sources by `make -C oracle ref`). Runs only where that library is
present (the machine that has the reference tree); the GPU box does not need it."""
import copy
import ctypes as C
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from deepforge_b200 import graphs, runtime

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref" / "libdf_ref_import.so"

def _reference_tree() -> Path:
    """Where the reference's source tree lies when this machine has it: oracle/Makefile knows (DEEPFORGE_REFERENCE)."""
    found = subprocess.run(["make", "-s", "-C", str(ROOT / "oracle"), "print-reference"], capture_output=True, text=True)
    return Path(found.stdout.strip() or "/nonexistent")



def _library():
    shim = ROOT / "oracle" / "ref_importer_shim.cpp"
    stale = REF.exists() and REF.stat().st_mtime < shim.stat().st_mtime
    if (not REF.exists() or stale) and (_reference_tree() / "lib" / "Import").exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "ref"], capture_output=True)
    if not REF.exists():
        pytest.skip("reference importer not built on this machine")
    lib = C.CDLL(str(REF))
    lib.ref_parse.restype = C.c_int
    return lib


def _reference_dump(document, fmt=0):
    """The REFERENCE importer's parsed model as canonical text (ref_dump of the shim), or its error code."""
    lib = _library()
    if not hasattr(lib, "ref_dump"):
        pytest.skip("the reference importer library on this machine predates ref_dump")
    data = document if isinstance(document, bytes) else json.dumps(document).encode()
    length = C.c_size_t(0)
    code = lib.ref_dump(data, C.c_size_t(len(data)), C.c_int(fmt), None, C.c_size_t(0), C.byref(length))
    if code != 0:
        return code
    buffer = C.create_string_buffer(length.value + 1)
    lib.ref_dump(data, C.c_size_t(len(data)), C.c_int(fmt), buffer, C.c_size_t(length.value), C.byref(length))
    return buffer.raw[: length.value].decode()


def _reference():
    lib = _library()

    def parse(document, fmt=0):
        data = document if isinstance(document, bytes) else json.dumps(document).encode()
        message = C.create_string_buffer(512)
        tensors, nodes = C.c_int64(0), C.c_int64(0)
        code = lib.ref_parse(data, C.c_size_t(len(data)), C.c_int(fmt), C.byref(tensors), C.byref(nodes), message, C.c_size_t(512))
        return code, tensors.value, nodes.value, message.value.decode(errors="replace")
    return parse


def _ours(document, fmt=0):
    try:
        tensors, nodes = runtime.parse(document if isinstance(document, bytes) else json.dumps(document), fmt)
        return 0, tensors, nodes
    except runtime.DeepForgeError as error:
        return error.code, 0, 0


DOCS = {
    "c1": graphs.c1_conv(n=1, c=3, h=5, w=5, k=5),
    "c2": graphs.c2_bottleneck(n=1, h=8, w=8),
    "c2_f32": graphs.c2_bottleneck(n=1, h=8, w=8, io="FLOAT"),
    "c3": graphs.c3_quantize_matmul(128, 128, 128),
    "c4": graphs.c4_sdpa(1, 2, 16, 8),
    "c5": graphs.c5_paged_decode(2, 4, 2, 16, 8, 4, 16),
    "matmul_fp8": graphs.matmul_fp8(2, 2, 2),
}


@pytest.mark.parametrize("name", sorted(DOCS))
def test_both_importers_accept_the_benchmark_graphs(name):
    reference = _reference()
    code, tensors, nodes, message = reference(DOCS[name])
    assert code == 0, message
    assert _ours(DOCS[name]) == (0, tensors, nodes)


# graphs beyond the benchmark set, for the model comparison: strides, reordering, virtual flags, every attribute type
MODEL_DOCS = {
    **DOCS,
    "c1_wide": graphs.c1_conv("nhwc", n=2, c=4, h=6, w=5, k=3),
    "c3_f32_unaligned": graphs.c3_quantize_matmul(64, 96, 32, io="FLOAT", c_type="FLOAT"),
    "c4_noncausal_f32": graphs.c4_sdpa(2, 3, 40, 16, io="FLOAT", causal=False),
    "fp8_batched": graphs.matmul_fp8(4, 8, 4, c_type="FP8_E4M3", batch=(2, 3), b_k_major=True),
    "scalar_runtime": graphs.scalar_pointwise(),
    "scalar_embedded": graphs.scalar_pointwise({"index": 3, "value": "40200000"}),
    "scalar_embedded_half": graphs.scalar_pointwise({"index": 2, "value": 1.5}, data_type="HALF"),
    "pointwise_all_modes": graphs.pointwise_all_modes(),
}


@pytest.mark.parametrize("name", sorted(MODEL_DOCS))
def test_parsed_models_are_identical(name):
    """Not only accept / reject: the canonical model itself -- context, every tensor (uid, name, type, dims, strides,
    virtual, by-value, reordering) and every node (tag, name, ports, attributes with their value types) -- is the
    same text from both importers (what SerializedGraph::operator== compares, lib/Import/SerializedGraphImporter.cpp
    :1951-2090)."""
    expected = _reference_dump(MODEL_DOCS[name])
    assert isinstance(expected, str), f"the reference rejects this graph with code {expected}"
    assert runtime.dump_graph(MODEL_DOCS[name]) == expected
    # and through the canonical UBJSON encoding of the same document
    ubjson = _to_ubjson(MODEL_DOCS[name])
    if ubjson is not None:
        again = _reference_dump(ubjson, 2)
        if isinstance(again, str):
            assert runtime.dump_graph(ubjson, 2) == again


def _to_ubjson(value) -> bytes:
    """The canonical UBJSON both importers demand (what nlohmann::json::to_ubjson writes without size or type
    optimisation): smallest integer type, 'D' for reals, object keys in sorted order."""
    import struct

    def integer(n: int) -> bytes:
        if 0 <= n <= 127 or -128 <= n < 0:
            return b"i" + struct.pack(">b", n)
        if 0 <= n <= 255:
            return b"U" + struct.pack(">B", n)
        if -32768 <= n <= 32767:
            return b"I" + struct.pack(">h", n)
        if -(2 ** 31) <= n <= 2 ** 31 - 1:
            return b"l" + struct.pack(">i", n)
        return b"L" + struct.pack(">q", n)

    if value is None:
        return b"Z"
    if value is True:
        return b"T"
    if value is False:
        return b"F"
    if isinstance(value, int):
        return integer(value)
    if isinstance(value, float):
        return b"D" + struct.pack(">d", value)
    if isinstance(value, str):
        raw = value.encode()
        return b"S" + integer(len(raw)) + raw
    if isinstance(value, (list, tuple)):
        return b"[" + b"".join(_to_ubjson(item) for item in value) + b"]"
    out = b"{"
    for key in sorted(value):
        raw = key.encode()
        out += integer(len(raw)) + raw + _to_ubjson(value[key])
    return out + b"}"


MUTATIONS = [
    lambda d: d.update(json_version="1.1"),
    lambda d: d.update(cudnn_frontend_version=12300),
    lambda d: d.pop("context"),
    lambda d: d["context"].pop("sm_count"),
    lambda d: d["context"].update(extra=1),
    lambda d: d.update(unknown_top_level=1),
    lambda d: d["tensors"]["1"].update(bogus=1),
    lambda d: d["tensors"]["1"].pop("stride"),
    lambda d: d["tensors"]["1"].update(dim="x"),
    lambda d: d["tensors"]["1"].update(data_type="COMPLEX"),
    lambda d: d["tensors"]["1"].update(uid=9),
    lambda d: d["nodes"][0].update(tag="NOT_A_TAG"),
    lambda d: d["nodes"][0].update(surprise=True),
    lambda d: d["nodes"][0]["inputs"].update(Z=1),
    lambda d: d["nodes"][0]["inputs"].update(X=42),
    lambda d: d["context"].update(is_dynamic_shape_enabled=True),
    lambda d: d.update(fe_workspace_size=64),
    lambda d: d.update(workspace_modifications={"1": [0, 1, 2]}),
    lambda d: d.update(variant_pack_replacements=[[1, 2]]),
    # pass-by-value scalars (lib/Import/SerializedGraphImporter.cpp:190-268,670-686,860-925)
    lambda d: d["tensors"]["1"].update(is_pass_by_value=True),
    lambda d: d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value=1.0),
    lambda d: d["tensors"]["1"].update(pass_by_value={"index": 3, "value": "40200000"}),
    lambda d: d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value={"index": 3, "value": "40200000"}),
    lambda d: (d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value={"index": 3, "value": "40200000"}),
               d.update(pass_by_values={"1": {"index": 3, "value": "40200000"}})),
    lambda d: (d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value={"index": 3, "value": "40200000"}),
               d.update(pass_by_values={"1": {"index": 3, "value": "40200001"}})),
    lambda d: (d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value={"index": 3, "value": "40200000"}),
               d.update(pass_by_values={"01": {"index": 3, "value": "40200000"}})),
    lambda d: d.update(pass_by_values={"77": {"index": 3, "value": "40200000"}}),
    lambda d: d.update(pass_by_values={"1": {"index": 3, "value": "40200000"}}),
    lambda d: d.update(pass_by_values=[1]),
    lambda d: d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value={"index": 2, "value": 1.5}),
    lambda d: d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value={"index": 3, "value": "4020000"}),
    lambda d: d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value={"index": 3, "value": 2.5}),
    lambda d: d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value={"index": 6, "value": 1}),
    lambda d: d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value={"index": 3, "value": "40200000", "more": 1}),
    lambda d: d["tensors"]["1"].update(is_pass_by_value=True, pass_by_value=[3, "40200000"]),
    # tensors no node reads (legal in a DAG unless virtual) and the value types of node attributes (:1096-1192)
    lambda d: d["tensors"].update({"99": graphs.tensor(99, "EXTRA", [4])}),
    lambda d: d["tensors"].update({"99": graphs.tensor(99, "EXTRA", [4], virtual=True)}),
    lambda d: d["nodes"][0].update(math_mode="CORRELATE"),
    lambda d: d["nodes"][0].update(math_mode=None),
    lambda d: d["nodes"][0].update(stride=[1, 1.5]),
    lambda d: d["nodes"][0].update(pre_padding="x"),
    lambda d: d["nodes"][0].update(compute_data_type="WIDE"),
    lambda d: d["nodes"][0].update(compute_data_type=None),
    lambda d: d["nodes"][1].update(mode="NOT_A_MODE"),
    lambda d: d["nodes"][1].update(mode=None),
    lambda d: d["nodes"][1].update(axis=1.5),
    lambda d: d["nodes"][1].update(relu_lower_clip="x"),
    lambda d: d["nodes"][1].update(softplus_beta=True),
    lambda d: d["nodes"][1]["inputs"].update(IN_2=1),
    lambda d: d["nodes"][1]["inputs"].pop("IN_1"),
    lambda d: d["nodes"][1].update(mode="BINARY_SELECT"),
    lambda d: d["nodes"][2].update(mode="TANH_BWD"),
]


def _first(d):
    return d["tensors"][next(iter(d["tensors"]))]


# document, tensor and node structure (every executable benchmark graph x every mutation)
STRUCTURE_MUTATIONS = {
    "tensor dim 0": lambda d: _first(d).update(dim=[0] + _first(d)["dim"][1:]),
    "tensor stride 0": lambda d: _first(d).update(stride=[0] + _first(d)["stride"][1:]),
    "tensor stride negative": lambda d: _first(d).update(stride=[-1] + _first(d)["stride"][1:]),
    "tensor rank mismatch": lambda d: _first(d).update(stride=_first(d)["stride"][1:]),
    "tensor name empty": lambda d: _first(d).update(name=""),
    "tensor names repeat": lambda d: [v.update(name="SAME") for v in d["tensors"].values()],
    "tensor without uid": lambda d: _first(d).update(uid_assigned=False),
    "tensor uid string": lambda d: _first(d).update(uid="1"),
    "tensor is_virtual null": lambda d: _first(d).update(is_virtual=None),
    "tensor reordering unknown": lambda d: _first(d).update(reordering_type="WEIRD"),
    "tensor reordering INT8x32": lambda d: _first(d).update(reordering_type="INT8x32"),
    "tensor reordering F16x16": lambda d: _first(d).update(reordering_type="F16x16"),
    "tensor ragged uid alone": lambda d: _first(d).update(ragged_offset_uid=5),
    "tensor INT8": lambda d: _first(d).update(data_type="INT8"),
    "tensor DOUBLE": lambda d: _first(d).update(data_type="DOUBLE"),
    "tensor BOOLEAN": lambda d: _first(d).update(data_type="BOOLEAN"),
    "tensor type null": lambda d: _first(d).update(data_type=None),
    "tensor rank 9": lambda d: _first(d).update(dim=[1] * 9, stride=[1] * 9),
    "tensor rank 65": lambda d: _first(d).update(dim=[1] * 65, stride=[1] * 65),
    "tensor extents overflow": lambda d: _first(d).update(dim=[1 << 40, 1 << 40], stride=[1 << 40, 1]),
    "node name missing": lambda d: d["nodes"][0].pop("name"),
    "node name empty": lambda d: d["nodes"][0].update(name=""),
    "node inputs list": lambda d: d["nodes"][0].update(inputs=[1]),
    "node outputs empty": lambda d: d["nodes"][0].update(outputs={}),
    "node input by name": lambda d: d["nodes"][0]["inputs"].update({next(iter(d["nodes"][0]["inputs"])): "X"}),
    "node input real": lambda d: d["nodes"][0]["inputs"].update({next(iter(d["nodes"][0]["inputs"])): 1.0}),
    "nodes empty": lambda d: d.update(nodes=[]),
    "tensors empty": lambda d: d.update(tensors={}),
    "graph_uid negative": lambda d: d.update(graph_uid=-1),
    "graph_uid real": lambda d: d.update(graph_uid=1.5),
    "backend version integer": lambda d: d.update(cudnn_backend_version=1),
    "context name integer": lambda d: d["context"].update(name=1),
    "context sm_count string": lambda d: d["context"].update(sm_count="x"),
    "context io null": lambda d: d["context"].update(io_data_type=None),
    "context io unknown": lambda d: d["context"].update(io_data_type="WIDE"),
    "context override enabled": lambda d: d["context"].update(is_override_shape_enabled=True),
    "context dynamic null": lambda d: d["context"].update(is_dynamic_shape_enabled=None),
    "tensors_to_dump": lambda d: d.update(tensors_to_dump=[1]),
    "behavior_notes object": lambda d: d.update(behavior_notes={}),
    "variant_pack_uids strings": lambda d: d.update(variant_pack_uids=["a"]),
    "fe_workspace_size negative": lambda d: d.update(fe_workspace_size=-1),
    "tensor keyed by name": lambda d: d["tensors"].update({_first(d)["name"]: d["tensors"].pop(next(iter(d["tensors"])))}),
    "output is also an input": lambda d: d["nodes"][0]["outputs"].update({next(iter(d["nodes"][0]["outputs"])): next(iter(d["nodes"][0]["inputs"].values()))}),
}
STRUCTURE_DOCS = {**DOCS, "pointwise_all_modes": graphs.pointwise_all_modes(), "scalar": graphs.scalar_pointwise()}


@pytest.mark.parametrize("mutation", sorted(STRUCTURE_MUTATIONS))
@pytest.mark.parametrize("name", sorted(STRUCTURE_DOCS))
def test_structure_error_codes_match_the_reference(name, mutation):
    reference = _reference()
    doc = copy.deepcopy(STRUCTURE_DOCS[name])
    STRUCTURE_MUTATIONS[mutation](doc)
    expected = reference(doc)
    assert _ours(doc)[0] == expected[0], expected[3]


# the same for the attributes of the other executable tags
ATTRIBUTE_MUTATIONS = [
    ("c4", lambda d: d["nodes"][0].update(diagonal_alignment="CENTER")),
    ("c4", lambda d: d["nodes"][0].update(diagonal_alignment=None)),
    ("c4", lambda d: d["nodes"][0].update(padding_mask=None)),
    ("c4", lambda d: d["nodes"][0].update(alibi_mask=1)),
    ("c4", lambda d: d["nodes"][0].update(generate_stats=None)),
    ("c4", lambda d: d["nodes"][0].update(generate_stats="yes")),
    ("c4", lambda d: d["nodes"][0].update(attn_scale_value="1")),
    ("c4", lambda d: d["nodes"][0].update(dropout_probability=True)),
    ("c4", lambda d: d["nodes"][0].update(right_bound=0.5)),
    ("c4", lambda d: d["nodes"][0].update(left_bound="0")),
    ("c4", lambda d: d["nodes"][0].update(max_seq_len_kv=1 << 40)),
    ("c4", lambda d: d["nodes"][0].update(mma_core_mode="FAST")),
    ("c4", lambda d: d["nodes"][0].update(implementation="FUSED")),
    ("c3", lambda d: d["nodes"][0].update(block_size=1 << 40)),
    ("c3", lambda d: d["nodes"][0].update(block_size=[32])),
    ("c3", lambda d: d["nodes"][0].update(axis="1")),
    ("c3", lambda d: d["nodes"][2].update(block_size=32)),
    ("c3", lambda d: d["nodes"][2].update(block_size=[1, 1 << 40])),
    ("c3", lambda d: d["nodes"][2].update(is_negative_scale=None)),
    ("c3", lambda d: d["nodes"][4].update(padding_value="0")),
    ("c3", lambda d: d["nodes"][4].update(padding_value=None)),
]


@pytest.mark.parametrize("index", range(len(ATTRIBUTE_MUTATIONS)))
def test_attribute_value_types_match_the_reference(index):
    reference = _reference()
    name, mutation = ATTRIBUTE_MUTATIONS[index]
    doc = copy.deepcopy(DOCS[name])
    mutation(doc)
    expected = reference(doc)
    assert _ours(doc)[0] == expected[0], expected[3]



@pytest.mark.parametrize("index", range(len(MUTATIONS)))
@pytest.mark.parametrize("name", ["c1", "c2_f32"])
def test_error_codes_match_the_reference(name, index):
    reference = _reference()
    doc = copy.deepcopy(DOCS[name])
    try:
        MUTATIONS[index](doc)
    except (KeyError, IndexError):
        pytest.skip("mutation does not apply to this graph")
    expected = reference(doc)
    assert _ours(doc)[0] == expected[0], expected[3]


def test_encodings_match_the_reference():
    reference = _reference()
    text = json.dumps(DOCS["c1"]).encode()
    for payload, fmt in ((b"{not json", 1), (text + b" trailing", 1), (b"\x00" * 16, 2), (b"\xff\xfegarbage", 0), (text, 2)):
        assert _ours(payload, fmt)[0] == reference(payload, fmt)[0]


@pytest.mark.parametrize("source", ["test/Compiler/RuntimeHeaderTest.cpp", "test/Compiler/SequenceOpsTest.cpp", "test/Compiler/SpecializedOpsTest.cpp",
                                    "test/Compiler/TrainingNormOpsTest.cpp"])
def test_reference_test_sources_compile_against_our_headers(source):
    """The reference's own test sources compiled UNMODIFIED against this repository's include/ tree: the compile-time check
    of the runtime interface (member signatures of Executable::execute and get_workspace_size as static_asserts), and the
    SDPA, block-scale / FP8 and normalisation test programs with everything they use of CompileOptions, CompilationResult,
    the argument metadata, the artifact calls and Executable. A host that builds against the reference's headers builds
    against these. (The other test programs use the x86 schedule / CPU-variant API or the 39-tag schema API, which this
    backend does not have.)"""
    import sysconfig
    path = _reference_tree() / source
    if not path.exists():
        pytest.skip("reference tree not on this machine")
    json_include = sysconfig.get_paths()["purelib"] + "/include"
    built = subprocess.run(["g++", "-std=c++20", "-fsyntax-only", "-I", str(ROOT / "include"), "-isystem", json_include, "-isystem",
                            json_include + "/cudnn_frontend/thirdparty", str(path)], capture_output=True, text=True)
    assert built.returncode == 0, built.stderr[-2000:]


def _reference_attention():
    """The attention oracle of the reference's own SDPA tests, compiled from the test source (oracle/ref_sdpa_shim.cpp)."""
    library = ROOT / "oracle" / "_ref" / "libdf_ref_sdpa.so"
    shim = ROOT / "oracle" / "ref_sdpa_shim.cpp"
    if (not library.exists() or library.stat().st_mtime < shim.stat().st_mtime) and (_reference_tree() / "test" / "Compiler" / "SequenceOpsTest.cpp").exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "ref"], capture_output=True)
    if not library.exists():
        pytest.skip("reference attention oracle not built on this machine")
    import os
    lib = C.CDLL(str(library), mode=os.RTLD_LAZY)  # (the compiler entry points the test's other functions call are never bound)
    lib.ref_attention_forward.restype = C.c_int
    return lib


@pytest.mark.parametrize("case", range(8))
def test_sdpa_restatement_agrees_with_the_references_own_test_oracle(case):
    """oracle/df_oracle.c's SDPA forward against attention_forward of test/Compiler/SequenceOpsTest.cpp:322-509 (the oracle the
    reference's tests hold its compiler to, double-precision scores) on seeded cases: grouped heads, padding with short
    and empty sequences, sliding windows, bottom-right alignment, ALiBi, a bias row, sink tokens, a block mask."""
    import numpy as np
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle
    from deepforge_b200.dfgpu import F32, I32, U8, tensor
    lib = _reference_attention()
    rng = np.random.default_rng(100 + case)
    b, hq, hk, hv = (2, 6, 3, 2) if case % 2 else (3, 4, 1, 4)
    sq, skv, d, dv = (5, 9, 8, 6) if case < 6 else (130, 260, 16, 8)
    q = rng.standard_normal((b, hq, sq, d)).astype(np.float32)
    k = rng.standard_normal((b, hk, skv, d)).astype(np.float32)
    v = rng.standard_normal((b, hv, skv, dv)).astype(np.float32)
    padding = case in (1, 2, 3, 6)
    seq_q = (rng.integers(0, sq + 1, b) if padding else np.full(b, sq)).astype(np.int32)
    seq_kv = (rng.integers(0, skv + 1, b) if padding else np.full(b, skv)).astype(np.int32)
    left, right = (3 if case in (2, 5) else None), (0 if case in (2, 3, 4, 7) else None)
    bottom_right = case in (3, 4)
    alibi = case == 5
    bias = rng.standard_normal((1, hq, 1, skv)).astype(np.float32) if case == 1 else None
    sink = rng.standard_normal(hq).astype(np.float32) if case in (0, 6) else None
    mask = None
    if case == 7:
        mask = rng.integers(1, 256, (b, hq, 2, 1)).astype(np.uint8)  # 2 query tiles x 3 key tiles: one byte per row of tiles
        mask[..., 0] |= 1  # (the first key tile stays on, so that causal rows keep a valid key)
    scale = 0.37
    p = oracle.SdpaParams()
    p.q, p.k, p.v, p.o = tensor(F32, list(q.shape)), tensor(F32, list(k.shape)), tensor(F32, list(v.shape)), tensor(F32, [b, hq, sq, dv])
    p.stats = p.max = p.sum_exp = tensor(F32, [b, hq, sq, 1])
    p.attn_scale, p.s_kv, p.padding_mask, p.bottom_right, p.alibi_mask = scale, skv, int(padding), int(bottom_right), int(alibi)
    if padding:
        p.seq_q = p.seq_kv = tensor(I32, [b, 1, 1, 1])
    if left is not None:
        p.has_left_bound, p.left_bound = 1, left
    if right is not None:
        p.has_right_bound, p.right_bound = 1, right
    if bias is not None:
        p.bias = tensor(F32, list(bias.shape))
    if sink is not None:
        p.sink = tensor(F32, [1, hq, 1, 1])
    if mask is not None:
        p.block_mask = tensor(U8, list(mask.shape))
    rows = b * hq * sq
    o, stats, maximum, sum_exp = (np.zeros(rows * dv, np.float32), np.zeros(rows, np.float32), np.zeros(rows, np.float32), np.zeros(rows, np.float32))
    oracle.sdpa_forward(p, [q, k, v, o, stats, maximum, sum_exp, seq_q if padding else None, seq_kv if padding else None, None, None, bias, sink, mask])
    ro, rs, rm, re = (np.zeros_like(o), np.zeros_like(stats), np.zeros_like(maximum), np.zeros_like(sum_exp))
    i64 = lambda a: (C.c_int64 * 4)(*[int(x) for x in a])
    ptr = lambda a, t: a.ctypes.data_as(C.POINTER(t)) if a is not None else None
    lib.ref_attention_forward(i64(q.shape), i64(k.shape), i64(v.shape), ptr(q, C.c_float), ptr(k, C.c_float), ptr(v, C.c_float), ptr(bias, C.c_float), ptr(sink, C.c_float),
                              ptr(mask, C.c_uint8), C.c_int64(mask.size if mask is not None else 0), ptr(seq_q, C.c_int32), ptr(seq_kv, C.c_int32), C.c_float(scale),
                              int(alibi), int(padding), int(bottom_right), int(left is not None), C.c_int64(left or 0), int(right is not None), C.c_int64(right or 0),
                              ptr(ro, C.c_float), ptr(rs, C.c_float), ptr(rm, C.c_float), ptr(re, C.c_float))
    assert np.allclose(o, ro, rtol=2e-5, atol=2e-6)
    live = re > 0  # rows with at least one valid key (or a sink): the others have no defined statistics
    assert live.any()
    assert np.allclose(maximum[live], rm[live], rtol=1e-6, atol=1e-6) and np.allclose(sum_exp[live], re[live], rtol=2e-5) and np.allclose(stats[live], rs[live], rtol=2e-5, atol=2e-6)


def test_bernoulli_stream_agrees_with_the_references_own():
    """dfo_bernoulli against bernoulli() of test/Compiler/SequenceOpsTest.cpp:199-222 (the stream the reference's RNG and dropout tests hold its
    compiler to): seeds and offsets of either sign, flat indices past 2^32, keep probabilities from 0 to 1."""
    import numpy as np
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle
    lib = _reference_attention()
    lib.ref_bernoulli.restype = C.c_float
    rng = np.random.default_rng(7)
    kept = 0
    for _ in range(4000):
        seed, offset = int(rng.integers(-2 ** 62, 2 ** 62)), int(rng.integers(-2 ** 40, 2 ** 40))
        linear = int(rng.integers(0, 2 ** 40))
        keep = float(rng.choice([0.0, 0.1, 0.375, 0.5, 0.6, 0.9, 0.999999, 1.0]))
        ours = oracle.bernoulli(seed, offset, linear, keep)
        theirs = float(lib.ref_bernoulli(C.c_int64(seed), C.c_int64(offset), C.c_uint64(linear), C.c_double(keep)))
        assert ours == theirs
        kept += int(ours)
    assert 1000 < kept < 3000
    # the cases the reference's tests use: seed -31, offset 19, keep 0.375 (:1149-1165) and seed 123, offset 9, keep 0.6 (:2351-2371)
    for seed, offset, keep in ((-31, 19, 0.375), (123, 9, 0.6), (17, 0, 0.375)):
        assert [oracle.bernoulli(seed, offset, i, keep) for i in range(6)] == [float(lib.ref_bernoulli(C.c_int64(seed), C.c_int64(offset), C.c_uint64(i), C.c_double(keep))) for i in range(6)]


@pytest.mark.parametrize("kind", ["mask", "probability"])
def test_sdpa_dropout_restatement_agrees_with_the_references_own_test_oracle(kind):
    """Dropout in oracle/df_oracle.c's SDPA forward against attention_forward of test/Compiler/SequenceOpsTest.cpp (its dropout_mask and
    dropout_scale, :493-498): a caller's mask with its scale, and probability dropout, whose mask the restatement draws from the Bernoulli stream
    and writes to RNG_DUMP (compared with the reference's stream, then fed to the reference oracle as its mask, as :2351-2390 does)."""
    import numpy as np
    sys.path.insert(0, str(ROOT / "tests"))
    import oracle
    from deepforge_b200.dfgpu import F32, I32, I64, tensor
    lib = _reference_attention()
    lib.ref_bernoulli.restype = C.c_float
    rng = np.random.default_rng(41)
    b, hq, hk, hv, sq, skv, d, dv = 2, 4, 2, 4, 7, 11, 8, 5
    q = rng.standard_normal((b, hq, sq, d)).astype(np.float32)
    k = rng.standard_normal((b, hk, skv, d)).astype(np.float32)
    v = rng.standard_normal((b, hv, skv, dv)).astype(np.float32)
    seq_q, seq_kv = np.array([sq, 4], np.int32), np.array([skv - 2, skv], np.int32)
    scale = 0.29
    p = oracle.SdpaParams()
    p.q, p.k, p.v, p.o = tensor(F32, list(q.shape)), tensor(F32, list(k.shape)), tensor(F32, list(v.shape)), tensor(F32, [b, hq, sq, dv])
    p.stats = p.max = p.sum_exp = tensor(F32, [b, hq, sq, 1])
    p.attn_scale, p.s_kv, p.padding_mask, p.has_right_bound, p.right_bound = scale, skv, 1, 1, 2
    p.seq_q = p.seq_kv = tensor(I32, [b, 1, 1, 1])
    rows = b * hq * sq
    o, stats, maximum, sum_exp = (np.zeros(rows * dv, np.float32), np.zeros(rows, np.float32), np.zeros(rows, np.float32), np.zeros(rows, np.float32))
    if kind == "mask":
        mask = (rng.random((b, hq, sq, skv)) < 0.7).astype(np.float32)
        mask[0, 1] = 0.5  # (the mask is a FLOAT tensor: any value multiplies)
        dropout_scale = np.array([1.0 / 0.7], np.float32)
        p.dropout_kind, p.dropout_mask = 2, tensor(F32, list(mask.shape))
        oracle.sdpa_forward(p, [q, k, v, o, stats, maximum, sum_exp, seq_q, seq_kv, None, None, None, None, None, None, None, mask, dropout_scale])
    else:
        probability, seed, offset = 0.4, np.array([123], np.int64), np.array([9], np.int64)
        dump = np.full(b * hq * sq * skv, -1.0, np.float32)
        p.dropout_kind, p.dropout_probability, p.rng_dump = 1, probability, tensor(F32, [b, hq, sq, skv])
        oracle.sdpa_forward(p, [q, k, v, o, stats, maximum, sum_exp, seq_q, seq_kv, None, None, None, None, None, None, None, None, None, seed, offset, dump])
        expected = np.array([lib.ref_bernoulli(C.c_int64(123), C.c_int64(9), C.c_uint64(i), C.c_double(1.0 - probability)) for i in range(dump.size)], np.float32)
        assert np.array_equal(dump, expected) and 0.5 < dump.mean() < 0.7
        mask, dropout_scale = dump.reshape(b, hq, sq, skv), np.array([1.0 / (1.0 - probability)], np.float32)
    ro, rs, rm, re = (np.zeros_like(o), np.zeros_like(stats), np.zeros_like(maximum), np.zeros_like(sum_exp))
    i64 = lambda a: (C.c_int64 * 4)(*[int(x) for x in a])
    ptr = lambda a, t: a.ctypes.data_as(C.POINTER(t)) if a is not None else None
    lib.ref_attention_forward_dropout.restype = C.c_int
    lib.ref_attention_forward_dropout(i64(q.shape), i64(k.shape), i64(v.shape), ptr(q, C.c_float), ptr(k, C.c_float), ptr(v, C.c_float), ptr(seq_q, C.c_int32),
                                      ptr(seq_kv, C.c_int32), C.c_float(scale), 1, 1, C.c_int64(2), ptr(np.ascontiguousarray(mask), C.c_float),
                                      C.c_float(float(dropout_scale[0])), ptr(ro, C.c_float), ptr(rs, C.c_float), ptr(rm, C.c_float), ptr(re, C.c_float))
    assert np.allclose(o, ro, rtol=2e-5, atol=2e-6) and np.abs(ro).max() > 0.1
    live = re > 0
    assert live.any() and np.allclose(stats[live], rs[live], rtol=2e-5, atol=2e-6)   # (statistics are those without dropout)
