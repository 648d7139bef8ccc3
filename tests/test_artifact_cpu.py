"""Artifacts without a GPU: the container of the reference's format 12 (docs/artifact-format.en.md:55-123) with the
kernel plan as adapter kind 2. Deterministic bytes, round trips, and the negatives of the reference's
test/Compiler/ArtifactTest.cpp: corruption, truncation at every length, checksummed fields that are out of
range, stale formats, writer-side rejections, atomic publication."""
import os
import struct
import threading
from pathlib import Path

import pytest

from deepforge_b200 import graphs, runtime
from deepforge_b200.runtime import DeepForgeError

DOCS = {
    "c1": graphs.c1_conv(n=1, c=3, h=5, w=5, k=5),
    "c2": graphs.c2_bottleneck(n=1, h=8, w=8),
    "c3": graphs.c3_quantize_matmul(128, 128, 128),
    "c3_unfused": graphs.c3_quantize_matmul(128, 128, 96),
    "c4": graphs.c4_sdpa(1, 2, 256, 128),
    "c5": graphs.c5_paged_decode(2, 4, 2, 128, 8, 64, 256),
    "fp8": graphs.matmul_fp8(128, 128, 128, c_type="BFLOAT16"),
}
MAGIC = b"DFOBJ\r\n\x1a"
PARSE_ERROR, INVALID_VALUE, IO_ERROR = 3, 8, 2


def fnv1a(data: bytes) -> int:
    value = 0xcbf29ce484222325
    for byte in data:
        value = ((value ^ byte) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
    return value


def refresh(data: bytearray) -> bytes:
    """Recomputes the trailing checksum, so that what the test changed is what the reader trips over."""
    data[-8:] = struct.pack("<Q", fnv1a(bytes(data[:-8])))
    return bytes(data)


class Layout:
    """Walks the container far enough to know where its fields are."""

    def __init__(self, data: bytes):
        self.data = data
        at = 16
        for _ in range(5):
            at = self._string(at)
        self.flags = at            # u32 dynamic, override, policy, role count, axis count
        at += 20
        self.argument_count = struct.unpack_from("<I", data, at)[0]
        at += 4
        self.arguments = []
        for _ in range(self.argument_count):
            entry = {"uid": at}
            at = self._string(at + 8)
            entry["data_type"], entry["access"], entry["storage_policy"] = at, at + 4, at + 8
            at += 12 + 24
            entry["alignment"], entry["size_bytes"] = at, at + 8
            at += 16
            rank = struct.unpack_from("<I", data, at)[0]
            entry["rank"] = at
            at += 4 + 16 * rank
            self.arguments.append(entry)
        self.adapter_kind = at
        self.adapter_size = struct.unpack_from("<Q", data, at + 4)[0]
        self.plan = at + 12        # u32 abi, u32 step count, then the first step: u32 op
        at = self.plan + self.adapter_size
        self.workspace_size, self.workspace_alignment, self.allocation_count = at, at + 8, at + 16

    def _string(self, at: int) -> int:
        return at + 4 + struct.unpack_from("<I", self.data, at)[0]


def code_of(data: bytes) -> int:
    try:
        runtime.load_artifact(data)
    except DeepForgeError as error:
        return error.code
    return 0


@pytest.mark.parametrize("name", sorted(DOCS))
def test_round_trip_is_deterministic_and_complete(name):
    exe = runtime.compile_graph(DOCS[name])
    first, second = exe.serialize(), runtime.compile_graph(DOCS[name]).serialize()
    assert first == second and exe.serialize() == first
    assert first[:8] == MAGIC and struct.unpack_from("<II", first, 8) == (13, 0x01020304)
    assert struct.unpack_from("<Q", first, len(first) - 8)[0] == fnv1a(first[:-8])
    loaded = runtime.load_artifact(first)
    assert loaded.plan_text() == exe.plan_text()
    assert loaded.workspace_size == exe.workspace_size and loaded.launch_count == exe.launch_count
    assert loaded.arguments() == exe.arguments() and loaded.steps() == exe.steps()
    assert loaded.serialize() == first  # a loaded executable writes the artifact it came from


def test_options_reach_the_artifact():
    plain = runtime.compile_graph(DOCS["c2"]).serialize()
    unfused = runtime.compile_graph(DOCS["c2"], options=runtime.NO_FUSION).serialize()
    assert plain != unfused
    assert runtime.load_artifact(unfused).launch_count == 8 and runtime.load_artifact(plain).launch_count == 2


def test_every_truncation_and_sampled_corruption_is_a_parse_error():
    data = runtime.compile_graph(DOCS["c2"]).serialize()
    for length in range(len(data)):
        assert code_of(data[:length]) == PARSE_ERROR, length
    assert code_of(data + b"\x00") == PARSE_ERROR
    for position in list(range(0, 64)) + list(range(64, len(data), 37)):
        flipped = bytearray(data)
        flipped[position] ^= 0x40
        assert code_of(bytes(flipped)) == PARSE_ERROR, position


def _patched(data: bytes, offset: int, fmt: str, value) -> bytes:
    out = bytearray(data)
    struct.pack_into(fmt, out, offset, value)
    return refresh(out)


def test_checksummed_fields_out_of_range_are_rejected():
    data = runtime.compile_graph(DOCS["c2"]).serialize()
    layout = Layout(data)
    first = layout.arguments[0]
    cases = {
        "stale format 12": _patched(data, 8, "<I", 12),
        "unknown format": _patched(data, 8, "<I", 14),
        "endian marker": _patched(data, 12, "<I", 0x04030201),
        "non-boolean dynamic flag": _patched(data, layout.flags, "<I", 2),
        "override flag set": _patched(data, layout.flags + 4, "<I", 1),
        "unknown override policy": _patched(data, layout.flags + 8, "<I", 0xFFFFFFFF),
        "excessive override roles": _patched(data, layout.flags + 12, "<I", 0xFFFFFFFF),
        "excessive override axes": _patched(data, layout.flags + 16, "<I", 0xFFFFFFFF),
        "argument count": _patched(data, layout.flags + 20, "<I", 0xFFFFFFFF),
        "zero argument alignment": _patched(data, first["alignment"], "<Q", 0),
        "argument size not its span": _patched(data, first["size_bytes"], "<Q", 1),
        "unknown storage policy": _patched(data, first["storage_policy"], "<I", 0xFFFFFFFF),
        "unknown data type": _patched(data, first["data_type"], "<I", 200),
        "unknown access": _patched(data, first["access"], "<I", 3),
        "rank": _patched(data, first["rank"], "<I", 65),
        "duplicate uid": _patched(data, layout.arguments[1]["uid"], "<q", struct.unpack_from("<q", data, first["uid"])[0]),
        "CPU adapter kind": _patched(data, layout.adapter_kind, "<I", 1),
        "adapter size": _patched(data, layout.adapter_kind + 4, "<Q", layout.adapter_size + 8),
        "launch count": _patched(data, layout.plan + 4, "<I", 0),
        "unknown entry point": _patched(data, layout.plan + 8, "<I", 99),
        "zero workspace alignment": _patched(data, layout.workspace_alignment, "<Q", 0),
        "workspace size off its high-water mark": _patched(data, layout.workspace_size, "<Q", struct.unpack_from("<Q", data, layout.workspace_size)[0] + 64),
        "allocation count": _patched(data, layout.allocation_count, "<I", 0xFFFFFFFF),
    }
    for label, mutated in cases.items():
        assert code_of(mutated) == PARSE_ERROR, label
    assert code_of(refresh(bytearray(data))) == 0  # the helper itself leaves a good artifact good


def test_plan_fields_are_validated_against_the_kernel_library():
    data = runtime.compile_graph(DOCS["c3"]).serialize()
    layout = Layout(data)
    # the kernel ABI the plan was built against
    assert code_of(_patched(data, layout.plan, "<I", 999)) == INVALID_VALUE
    # first step: u32 op, string label, u32 node count, u64 nodes[], u32 kernel, u32 launches, u32 params size, params
    at = layout.plan + 8 + 4
    at += 4 + struct.unpack_from("<I", data, at)[0]
    nodes = struct.unpack_from("<I", data, at)[0]
    kernel_at = at + 4 + 8 * nodes
    assert code_of(_patched(data, kernel_at, "<I", 7)) == INVALID_VALUE           # not the kernel the library resolves
    params_at = kernel_at + 12
    assert code_of(_patched(data, kernel_at + 8, "<I", 12)) == PARSE_ERROR         # params block of the wrong size
    assert code_of(_patched(data, params_at + 4, "<i", 9)) == PARSE_ERROR          # first tensor's rank above 8
    assert code_of(_patched(data, params_at, "<i", 77)) == PARSE_ERROR             # first tensor's data type


def test_bindings_must_stay_inside_arguments_and_workspace():
    exe = runtime.compile_graph(DOCS["c2"])
    data = exe.serialize()
    layout = Layout(data)
    # the first launch of the bottleneck writes a workspace tensor: find a binding of kind 2 and push it outside
    needle = struct.pack("<Iq", 2, 13)  # kWorkspace, uid 13 (conv1's fused output)
    at = data.index(needle, layout.plan)
    assert code_of(_patched(data, at + 12, "<Q", exe.workspace_size)) == PARSE_ERROR
    assert code_of(_patched(data, at + 12, "<Q", 8)) == PARSE_ERROR  # inside, but not 16-byte aligned
    assert code_of(_patched(data, at + 12, "<Q", exe.workspace_size - 64)) == PARSE_ERROR  # starts inside, its span runs past the end
    needle = struct.pack("<Iq", 1, 1)   # kArgument, uid 1 (X)
    at = data.index(needle, layout.plan)
    assert code_of(_patched(data, at + 4, "<q", 4242)) == PARSE_ERROR


def test_descriptors_must_fit_the_buffers_they_are_bound_to():
    """A params block whose tensor descriptor spans more bytes than the argument (or workspace range) its slot is
    bound to would make the kernel read or write past the caller's buffer: refused at load, checksum or not."""
    data = runtime.compile_graph(DOCS["c3"]).serialize()
    layout = Layout(data)
    at = layout.plan + 8 + 4
    at += 4 + struct.unpack_from("<I", data, at)[0]
    nodes = struct.unpack_from("<I", data, at)[0]
    params_at = at + 4 + 8 * nodes + 12
    # first launch = quantize A: x is the first descriptor (16 bytes of header, then dim[8], stride[8] as int64)
    assert struct.unpack_from("<q", data, params_at + 16)[0] == 128
    assert code_of(_patched(data, params_at + 16, "<q", 256)) == PARSE_ERROR       # twice the rows of the bound argument
    assert code_of(_patched(data, params_at + 16 + 64, "<q", 1 << 40)) == PARSE_ERROR  # a row stride far beyond it
    assert code_of(_patched(data, params_at + 16, "<q", -1)) == PARSE_ERROR        # no storage span at all
    assert code_of(_patched(data, params_at + 16, "<q", 64)) in (0, INVALID_VALUE)  # a smaller view fits (the kernel re-resolution may still refuse it)


def test_files_are_published_by_rename(tmp_path: Path):
    exe = runtime.compile_graph(DOCS["c4"])
    target = tmp_path / "sdpa.dfo"
    exe.write_artifact(target)
    assert target.read_bytes() == exe.serialize()
    assert [p.name for p in tmp_path.iterdir()] == ["sdpa.dfo"]  # no temporary left behind
    assert runtime.load_artifact(target).plan_text() == exe.plan_text()
    # two writers to one destination: the file is always one complete artifact
    other = runtime.compile_graph(DOCS["c5"])
    threads = [threading.Thread(target=lambda e=e: [e.write_artifact(target) for _ in range(20)]) for e in (exe, other)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert target.read_bytes() in (exe.serialize(), other.serialize())
    assert [p.name for p in tmp_path.iterdir()] == ["sdpa.dfo"]
    with pytest.raises(DeepForgeError) as error:
        runtime.load_artifact(tmp_path / "missing.dfo")
    assert error.value.code == IO_ERROR
    with pytest.raises(DeepForgeError) as error:
        exe.write_artifact(tmp_path / "no_such_directory" / "x.dfo")
    assert error.value.code == IO_ERROR
    (tmp_path / "short.dfo").write_bytes(exe.serialize()[:100])
    with pytest.raises(DeepForgeError) as error:
        runtime.load_artifact(tmp_path / "short.dfo")
    assert error.value.code == PARSE_ERROR
