"""CPU-side checks of the C ABI: the libraries load without a GPU and export every
symbol the public headers declare; launchers reject bad descriptors before any CUDA call."""
import ctypes as C
import re
from pathlib import Path

import pytest

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
    assert lib.dfgpu_abi_version() == 11


def test_struct_layout_matches_header():
    # sizes computed from include/dfgpu.h by a C compiler (see the build of this repo)
    assert C.sizeof(dfgpu.Tensor) == 144
    assert C.sizeof(dfgpu.PlanInfo) == 16
    assert C.sizeof(dfgpu.EpilogueStep) == 24
    # every params struct: a host built against another layout must not get past the version check silently
    assert C.sizeof(dfgpu.BsqParams) == 448
    assert C.sizeof(dfgpu.BsdParams) == 504
    assert C.sizeof(dfgpu.BsqPairParams) == 896
    assert C.sizeof(dfgpu.PointwiseParams) == 608
    assert C.sizeof(dfgpu.ConstantsParams) == 200
    assert C.sizeof(dfgpu.ConvParams) == 928
    assert C.sizeof(dfgpu.ConvPairParams) == 1856
    assert C.sizeof(dfgpu.MatmulParams) == 1144
    assert C.sizeof(dfgpu.MatmulFp8Params) == 440
    assert C.sizeof(dfgpu.SdpaParams) == 3096


def test_struct_sizes_agree_with_the_c_compiler(tmp_path):
    """The ctypes mirrors against sizeof() as gcc sees include/dfgpu.h."""
    import shutil
    import subprocess
    if not shutil.which("gcc"):
        import pytest
        pytest.skip("no C compiler")
    names = ["tensor", "plan_info", "epilogue_step", "bsq_params", "bsd_params", "constants_params", "pointwise_params", "conv_params", "matmul_params", "matmul_fp8_params", "sdpa_params", "conv_pair_params", "bsq_pair_params"]
    source = tmp_path / "sizes.c"
    source.write_text('#include <stdio.h>\n#include "dfgpu.h"\nint main(void){' + "".join(f'printf("%zu\\n", sizeof(dfgpu_{n}));' for n in names) + "return 0;}\n")
    binary = tmp_path / "sizes"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(source), "-o", str(binary)], check=True)
    sizes = [int(v) for v in subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout.split()]
    mirrors = [dfgpu.Tensor, dfgpu.PlanInfo, dfgpu.EpilogueStep, dfgpu.BsqParams, dfgpu.BsdParams, dfgpu.ConstantsParams, dfgpu.PointwiseParams, dfgpu.ConvParams,
               dfgpu.MatmulParams, dfgpu.MatmulFp8Params, dfgpu.SdpaParams, dfgpu.ConvPairParams, dfgpu.BsqPairParams]
    assert sizes == [C.sizeof(m) for m in mirrors]


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


def test_pointwise_rejects_what_the_reference_rejects():
    """validate_pointwise (lib/Compiler/FoundationalGraph.cpp:721-775): GEN_INDEX axis, softplus beta, clip order; no launch."""
    d = dfgpu.tensor(dfgpu.F32, [4, 4])
    for mode_name, change in (("GEN_INDEX", dict(axis=2)), ("GEN_INDEX", dict(axis=-1)), ("SOFTPLUS_FWD", dict(softplus_beta=0.0)),
                              ("RELU_BWD", dict(relu_lower=2.0, relu_upper=1.0))):
        p = dfgpu.PointwiseParams()
        p.in0, p.in1, p.out, p.mode = d, d, d, dfgpu.PW_MODES[mode_name]
        p.relu_upper = 3.4028234663852886e38
        for key, value in change.items():
            setattr(p, key, value)
        with pytest.raises(dfgpu.DfgpuError) as error:
            dfgpu.query("pointwise", p)
        assert error.value.code == 8
    p = dfgpu.PointwiseParams()
    p.in0, p.out, p.mode = d, d, 50
    with pytest.raises(dfgpu.DfgpuError) as error:
        dfgpu.query("pointwise", p)
    assert error.value.code == 20
