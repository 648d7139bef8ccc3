"""Protocol parity of the importer against the REFERENCE importer itself (oracle/_ref, built from
the reference's own lib/Import sources by `make -C oracle ref`). Runs only where that library is
present (the machine that has the reference tree); the GPU box does not need it."""
import copy
import ctypes as C
import json
import subprocess
from pathlib import Path

import pytest

from deepforge_b200 import graphs, runtime

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref" / "libdf_ref_import.so"


def _reference():
    if not REF.exists() and Path("/root/reference/lib/Import").exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "ref"], capture_output=True)
    if not REF.exists():
        pytest.skip("reference importer not built on this machine")
    lib = C.CDLL(str(REF))
    lib.ref_parse.restype = C.c_int

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
]


@pytest.mark.parametrize("index", range(len(MUTATIONS)))
@pytest.mark.parametrize("name", ["c1", "c2_f32"])
def test_error_codes_match_the_reference(name, index):
    reference = _reference()
    doc = copy.deepcopy(DOCS[name])
    try:
        MUTATIONS[index](doc)
    except KeyError:
        pytest.skip("mutation does not apply to this graph")
    expected = reference(doc)
    assert _ours(doc)[0] == expected[0], expected[3]


def test_encodings_match_the_reference():
    reference = _reference()
    text = json.dumps(DOCS["c1"]).encode()
    for payload, fmt in ((b"{not json", 1), (text + b" trailing", 1), (b"\x00" * 16, 2), (b"\xff\xfegarbage", 0), (text, 2)):
        assert _ours(payload, fmt)[0] == reference(payload, fmt)[0]
