"""Writes tests/golden/importer_reference_results.json: what the REFERENCE importer itself (its own lib/Import
sources, compiled into oracle/_ref/libdf_ref_import.so by `make -C oracle ref`) answers for the benchmark graphs, for
malformed variants of them and for broken encodings. Run on a machine that has the reference tree:

    python tests/golden/make_importer_golden.py

The fixture lets tests/test_importer_golden.py hold the importer of this repository to the reference's status
codes, tensor / node counts and parsed models on machines that do not have the reference."""
import copy
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import test_importer_vs_reference as live  # noqa: E402  (the document set and the mutations live there)


def main() -> None:
    reference = live._reference.__wrapped__() if hasattr(live._reference, "__wrapped__") else live._reference()
    cases = []
    for name in sorted(live.MODEL_DOCS):
        code, tensors, nodes, message = reference(live.MODEL_DOCS[name])
        # "model": the reference's parsed model as canonical text (ref_dump of oracle/ref_importer_shim.cpp)
        cases.append({"case": f"accept:{name}", "format": 0, "text": json.dumps(live.MODEL_DOCS[name]), "code": code, "tensors": tensors, "nodes": nodes,
                      "model": live._reference_dump(live.MODEL_DOCS[name])})
        encoded = live._to_ubjson(live.MODEL_DOCS[name])
        code, tensors, nodes, message = reference(encoded, 2)
        cases.append({"case": f"accept_ubjson:{name}", "format": 2, "hex": encoded.hex(), "code": code, "tensors": tensors, "nodes": nodes,
                      "model": live._reference_dump(encoded, 2)})
    for name in ("c1", "c2_f32"):
        for index, mutate in enumerate(live.MUTATIONS):
            document = copy.deepcopy(live.DOCS[name])
            try:
                mutate(document)
            except KeyError:
                continue
            code, tensors, nodes, message = reference(document)
            cases.append({"case": f"mutation:{name}:{index}", "format": 0, "text": json.dumps(document), "code": code, "tensors": tensors, "nodes": nodes,
                          "reference_message": message})
    text = json.dumps(live.DOCS["c1"]).encode()
    for label, payload, fmt in (("not_json", b"{not json", 1), ("trailing", text + b" trailing", 1), ("zeros_as_ubjson", b"\x00" * 16, 2),
                                ("garbage_auto", b"\xff\xfegarbage", 0), ("json_as_ubjson", text, 2)):
        code, tensors, nodes, message = reference(payload, fmt)
        cases.append({"case": f"encoding:{label}", "format": fmt, "hex": payload.hex(), "code": code, "tensors": tensors, "nodes": nodes})
    out = Path(__file__).resolve().parent / "importer_reference_results.json"
    out.write_text(json.dumps({"source": "reference lib/Import compiled by oracle/Makefile target ref", "cases": cases}, indent=1) + "\n")
    print(f"{len(cases)} cases -> {out}")


if __name__ == "__main__":
    main()
