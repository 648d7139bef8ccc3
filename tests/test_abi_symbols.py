"""CPU-side checks of the C ABI: the libraries load without a GPU and export every
symbol the public headers declare; launchers reject bad descriptors before any CUDA call."""
import ctypes as C
import re
from pathlib import Path

from deepforge_b200 import dfgpu

ROOT = Path(__file__).resolve().parent.parent


def _declared(header: Path, prefix: str):
    text = header.read_text()
    return sorted(set(re.findall(r"\b(" + prefix + r"[a-z0-9_]+)\s*\(", text)))


def test_kernel_library_exports_every_declared_symbol():
    lib = dfgpu.load()
    names = _declared(ROOT / "include" / "dfgpu.h", "dfgpu_")
    assert len(names) >= 17
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(dfgpu.EXPORTS) == names
    assert lib.dfgpu_abi_version() == 2


def test_struct_layout_matches_header():
    # sizes computed from include/dfgpu.h by a C compiler (see the build of this repo)
    assert C.sizeof(dfgpu.Tensor) == 144
    assert C.sizeof(dfgpu.PlanInfo) == 16
    assert C.sizeof(dfgpu.EpilogueStep) == 24


def test_query_rejects_bad_descriptors_without_a_gpu():
    p = dfgpu.BsqParams()
    p.x = dfgpu.tensor(dfgpu.F32, [4, 30])
    p.y = dfgpu.tensor(dfgpu.E4M3, [4, 30])
    p.scale = dfgpu.tensor(dfgpu.E8M0, [4, 1])
    p.block_size, p.axis = 32, 1
    try:
        dfgpu.query("block_scale_quantize", p)
        raise AssertionError("expected a shape error")
    except dfgpu.DfgpuError as error:
        assert error.code == 15 and "block size" in str(error)
    p.x = dfgpu.tensor(dfgpu.F32, [4, 64])
    p.y = dfgpu.tensor(dfgpu.E4M3, [4, 64])
    p.scale = dfgpu.tensor(dfgpu.E8M0, [4, 2])
    info = dfgpu.query("block_scale_quantize", p)
    assert info.kernel == dfgpu.BSQ_ROW32 and info.scratch_bytes == 0
    p.axis = 0
    p.scale = dfgpu.tensor(dfgpu.E8M0, [1, 64])
    p.block_size = 4
    assert dfgpu.query("block_scale_quantize", p).kernel == dfgpu.BSQ_GENERIC
