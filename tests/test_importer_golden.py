"""The importer against answers recorded from the REFERENCE importer (tests/golden/importer_reference_results.json,
written by tests/golden/make_importer_golden.py on a machine that has the reference tree): same status code for
every benchmark graph, malformed variant and broken encoding, the same tensor / node counts where it parses, and
the same parsed model (context, tensors, nodes, ports, attributes as canonical text) for every accepted graph."""
import json
from pathlib import Path

import pytest

from deepforge_b200 import runtime

FIXTURE = json.loads((Path(__file__).resolve().parent / "golden" / "importer_reference_results.json").read_text())


@pytest.mark.parametrize("case", FIXTURE["cases"], ids=lambda c: c["case"])
def test_importer_matches_recorded_reference_answer(case):
    payload = case["text"] if "text" in case else bytes.fromhex(case["hex"])
    try:
        tensors, nodes = runtime.parse(payload, case["format"])
        ours = (0, tensors, nodes)
    except runtime.DeepForgeError as error:
        ours = (error.code, 0, 0)
    assert ours[0] == case["code"], case.get("reference_message", "")
    if case["code"] == 0:
        assert ours[1:] == (case["tensors"], case["nodes"])
    if case.get("model") is not None:
        assert runtime.dump_graph(payload, case["format"]) == case["model"]
