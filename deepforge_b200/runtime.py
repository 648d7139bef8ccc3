"""ctypes face of the host library (include/deepforge_b200.h): parse, compile, execute.

`Executable.execute` is the Frontend-shaped call: a UID -> device pointer map plus a
workspace pointer. It only enqueues kernels on the stream given to `set_stream` (the
legacy default stream unless told otherwise); synchronisation is the caller's business.
"""
from __future__ import annotations

import ctypes as C
import json
from pathlib import Path
from typing import Dict, Mapping, Optional, Union

FORMAT_AUTO, FORMAT_JSON, FORMAT_UBJSON = 0, 1, 2
NO_FUSION, NO_NARROWING, NO_TENSOR_CORES, BF16_INTERMEDIATES, NO_CONV_PAIRS = 1, 2, 4, 8, 16

EXPORTS = [
    "df_last_error", "df_parse", "df_compile", "df_destroy", "df_workspace_size", "df_launch_count", "df_plan_text",
    "df_argument_count", "df_argument_info", "df_set_stream", "df_execute", "df_plan_workspace",
    "df_step_count", "df_step_info", "df_execute_steps",
    "df_serialize_artifact", "df_write_artifact", "df_load_artifact", "df_load_artifact_file",
    "df_argument_name", "df_conv2d_metadata", "df_dump_graph", "df_execute_on",
]

_LIB: Optional[C.CDLL] = None


class DeepForgeError(RuntimeError):
    """A non-OK DeepForge Status: .code is the numeric ErrorCode, str() the DFE_* message."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


def library_path() -> Path:
    return Path(__file__).resolve().parent / "_build" / "libdeepforge_b200.so"


def load() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = library_path()
        if not path.exists():
            raise RuntimeError(f"{path} is missing: run `python -m deepforge_b200.build` (or __graft_entry__.build())")
        lib = C.CDLL(str(path))
        for name in EXPORTS:
            getattr(lib, name)
        lib.df_last_error.restype = C.c_char_p
        lib.df_workspace_size.restype = C.c_int64
        lib.df_launch_count.restype = C.c_int64
        lib.df_argument_count.restype = C.c_int64
        lib.df_plan_text.restype = C.c_size_t
        lib.df_step_count.restype = C.c_int64
        lib.df_step_count.argtypes = [C.c_void_p]
        for name in ("df_workspace_size", "df_launch_count", "df_argument_count", "df_destroy"):
            getattr(lib, name).argtypes = [C.c_void_p]
        lib.df_plan_text.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t]
        lib.df_argument_name.restype = C.c_size_t
        lib.df_argument_name.argtypes = [C.c_void_p, C.c_int64, C.c_char_p, C.c_size_t]
        lib.df_set_stream.argtypes = [C.c_void_p, C.c_void_p]
        _LIB = lib
    return _LIB


def _check(code: int) -> None:
    if code != 0:
        raise DeepForgeError(code, load().df_last_error().decode(errors="replace"))


def _bytes(document: Union[str, bytes, dict]) -> bytes:
    if isinstance(document, dict):
        document = json.dumps(document)
    if isinstance(document, str):
        document = document.encode()
    return document


def parse(document: Union[str, bytes, dict], fmt: int = FORMAT_AUTO) -> tuple[int, int]:
    """Validate a serialized graph; returns (tensor count, node count)."""
    data = _bytes(document)
    tensors, nodes = C.c_int64(0), C.c_int64(0)
    _check(load().df_parse(data, C.c_size_t(len(data)), C.c_int(fmt), C.byref(tensors), C.byref(nodes)))
    return tensors.value, nodes.value


def dump_graph(document: Union[str, bytes, dict], fmt: int = FORMAT_AUTO) -> str:
    """The parsed model as canonical text (df_dump_graph): context, tensors, nodes with ports and attributes."""
    data = _bytes(document)
    length = C.c_size_t(0)
    _check(load().df_dump_graph(data, C.c_size_t(len(data)), C.c_int(fmt), None, C.c_size_t(0), C.byref(length)))
    buffer = C.create_string_buffer(length.value + 1)
    _check(load().df_dump_graph(data, C.c_size_t(len(data)), C.c_int(fmt), buffer, C.c_size_t(length.value), C.byref(length)))
    return buffer.raw[: length.value].decode()


class Executable:
    def __init__(self, handle: int):
        self._handle = C.c_void_p(handle)

    def __del__(self):
        if getattr(self, "_handle", None) and _LIB is not None:
            _LIB.df_destroy(self._handle)
            self._handle = None

    @property
    def workspace_size(self) -> int:
        return load().df_workspace_size(self._handle)

    @property
    def launch_count(self) -> int:
        return load().df_launch_count(self._handle)

    def plan_text(self) -> str:
        lib = load()
        size = lib.df_plan_text(self._handle, None, 0)
        buffer = C.create_string_buffer(size + 1)
        lib.df_plan_text(self._handle, buffer, size + 1)
        return buffer.value.decode()

    def arguments(self) -> list[dict]:
        lib = load()
        out = []
        for index in range(lib.df_argument_count(self._handle)):
            uid, size, alignment, access = C.c_int64(), C.c_uint64(), C.c_uint64(), C.c_int32()
            _check(lib.df_argument_info(self._handle, C.c_int64(index), C.byref(uid), C.byref(size), C.byref(alignment), C.byref(access)))
            name = C.create_string_buffer(lib.df_argument_name(self._handle, C.c_int64(index), None, 0) + 1)
            lib.df_argument_name(self._handle, C.c_int64(index), name, len(name))
            out.append({"uid": uid.value, "name": name.value.decode(), "size_bytes": size.value, "alignment": alignment.value,
                        "access": ("read", "write", "readwrite")[access.value]})
        return out

    def conv2d_metadata(self) -> Optional[dict]:
        """The single-node CONV_FPROP metadata (physical N, H, W, C shapes), or None under the generic argument table."""
        kind = C.c_int32(1)
        values = (C.c_int64 * 27)()
        _check(load().df_conv2d_metadata(self._handle, C.byref(kind), values))
        if kind.value != 0:
            return None
        v = list(values)
        return {"x_uid": v[0], "w_uid": v[1], "y_uid": v[2], "x_shape": v[3:7], "w_shape": v[7:11], "y_shape": v[11:15], "padded_x_shape": v[15:19],
                "pre_padding": v[19:21], "post_padding": v[21:23], "stride": v[23:25], "dilation": v[25:27]}

    def serialize(self) -> bytes:
        """The artifact bytes of this executable (compiler::serialize_artifact)."""
        size = C.c_size_t(0)
        _check(load().df_serialize_artifact(self._handle, None, C.c_size_t(0), C.byref(size)))
        buffer = (C.c_uint8 * size.value)()
        _check(load().df_serialize_artifact(self._handle, buffer, C.c_size_t(size.value), C.byref(size)))
        return bytes(buffer)

    def write_artifact(self, path: Union[str, Path]) -> None:
        """Publishes the artifact at `path` by writing a temporary file beside it and renaming it."""
        _check(load().df_write_artifact(self._handle, str(path).encode()))

    def set_stream(self, stream: Optional[int]) -> None:
        load().df_set_stream(self._handle, C.c_void_p(stream or None))

    def steps(self) -> list[dict]:
        """One entry per launch group of the kernel plan: label, op, kernel id, launches, bound bytes."""
        lib = load()
        out = []
        for index in range(lib.df_step_count(self._handle)):
            label = C.create_string_buffer(256)
            op, kernel, launches, size = C.c_int32(), C.c_int32(), C.c_int32(), C.c_uint64()
            _check(lib.df_step_info(self._handle, C.c_int64(index), label, C.c_size_t(256), C.byref(op), C.byref(kernel), C.byref(launches), C.byref(size)))
            out.append({"label": label.value.decode(), "op": op.value, "kernel": kernel.value, "launches": launches.value, "bound_bytes": size.value})
        return out

    def execute_steps(self, first: int, last: int, pack: Mapping[int, int], workspace: Optional[int] = None) -> None:
        count = len(pack)
        uids = (C.c_int64 * count)(*pack.keys())
        pointers = (C.c_void_p * count)(*[C.c_void_p(p or None) for p in pack.values()])
        _check(load().df_execute_steps(self._handle, C.c_int64(first), C.c_int64(last), uids, pointers, C.c_size_t(count), C.c_void_p(workspace or None)))

    def execute(self, pack: Mapping[int, int], workspace: Optional[int] = None, handle: Optional[int] = None) -> None:
        count = len(pack)
        uids = (C.c_int64 * count)(*pack.keys())
        pointers = (C.c_void_p * count)(*[C.c_void_p(p or None) for p in pack.values()])
        _check(load().df_execute(self._handle, C.c_void_p(handle or None), uids, pointers, C.c_size_t(count), C.c_void_p(workspace or None)))

    def execute_on(self, stream: int, pack: Mapping[int, int], workspace: Optional[int] = None) -> None:
        """execute() with the launches on `stream` (a cudaStream_t) for this call only; safe to call from several
        threads at once with different streams, workspaces and outputs (ctypes releases the GIL during the call)."""
        count = len(pack)
        uids = (C.c_int64 * count)(*pack.keys())
        pointers = (C.c_void_p * count)(*[C.c_void_p(p or None) for p in pack.values()])
        _check(load().df_execute_on(self._handle, C.c_void_p(stream or None), uids, pointers, C.c_size_t(count), C.c_void_p(workspace or None)))


def compile_graph(document: Union[str, bytes, dict], fmt: int = FORMAT_AUTO, options: int = 0) -> Executable:
    data = _bytes(document)
    handle = C.c_void_p()
    _check(load().df_compile(data, C.c_size_t(len(data)), C.c_int(fmt), C.c_uint32(options), C.byref(handle)))
    return Executable(handle.value)


def load_artifact(source: Union[bytes, str, Path]) -> Executable:
    """An Executable from artifact bytes or from an artifact file, without recompiling (compiler::load_artifact_executable)."""
    handle = C.c_void_p()
    if isinstance(source, (bytes, bytearray)):
        data = bytes(source)
        _check(load().df_load_artifact(data, C.c_size_t(len(data)), C.byref(handle)))
    else:
        _check(load().df_load_artifact_file(str(source).encode(), C.byref(handle)))
    return Executable(handle.value)


def plan_workspace(requests: list[dict]) -> Dict[str, object]:
    """requests: [{name, size_bytes, alignment, live_start, live_end}] -> offsets, placement order, total."""
    count = len(requests)
    names = (C.c_char_p * count)(*[r["name"].encode() for r in requests])
    arrays = {key: (C.c_uint64 * count)(*[r[key] for r in requests]) for key in ("size_bytes", "alignment", "live_start", "live_end")}
    offsets = (C.c_uint64 * count)()
    order = (C.c_int64 * count)()
    total = C.c_uint64()
    _check(load().df_plan_workspace(C.c_size_t(count), names, arrays["size_bytes"], arrays["alignment"], arrays["live_start"],
                                    arrays["live_end"], offsets, order, C.byref(total)))
    return {"offsets": {r["name"]: offsets[i] for i, r in enumerate(requests)},
            "order": [r["name"] for _, r in sorted(zip(order, requests), key=lambda pair: pair[0])], "total": total.value}
