"""In-tree builds of the two native libraries (no JIT cache, no pip install).

libdfgpu.so         CUDA kernels + the C ABI of include/dfgpu.h, compiled for sm_100a only.
libdeepforge_b200.so  C++20 host side (importer, graph analysis, workspace planner,
                    kernel-selection lowering, runtime) + the flat C API of
                    include/deepforge_b200.h. It links libdfgpu.so.

Both land in deepforge_b200/_build/. nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = Path(__file__).resolve().parent
OUT = PKG / "_build"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-diag-suppress", "177",
]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if candidate and (os.path.sep not in candidate or os.path.exists(candidate)):
            return candidate
    raise RuntimeError("nvcc not found")


def _stamp(sources: list[Path], extra: str) -> str:
    digest = hashlib.sha256(extra.encode())
    for path in sorted(sources):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def _up_to_date(target: Path, stamp: str) -> bool:
    marker = target.with_suffix(target.suffix + ".stamp")
    return target.exists() and marker.exists() and marker.read_text() == stamp


def _run(command: list[str]) -> None:
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        sys.stderr.write(result.stdout + result.stderr)
        raise RuntimeError("build failed: " + " ".join(command[:3]) + " ...")


def nlohmann_include() -> Path:
    """nlohmann/json 3.11.3 as vendored by the image's cudnn-frontend headers (the
    reference takes its JSON library from the same place)."""
    base = Path(sysconfig.get_paths()["purelib"]) / "include" / "cudnn_frontend" / "thirdparty"
    if not (base / "nlohmann" / "json.hpp").exists():
        raise RuntimeError(f"nlohmann/json.hpp not found under {base}")
    return base


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    OUT.mkdir(exist_ok=True)
    sources = sorted((PKG / "csrc").glob("*.cu"))
    headers = sorted((PKG / "csrc").glob("*.cuh")) + [ROOT / "include" / "dfgpu.h"]
    target = OUT / "libdfgpu.so"
    stamp = _stamp(sources + headers, " ".join(NVCC_FLAGS))
    if not force and _up_to_date(target, stamp):
        return target
    objects = []
    jobs = []
    for source in sources:
        obj = OUT / (source.stem + ".o")
        objects.append(obj)
        command = [_nvcc(), *NVCC_FLAGS, "-I", str(ROOT / "include"), "-c", str(source), "-o", str(obj)]
        if verbose:
            command[1:1] = ["-Xptxas", "-v"]
        jobs.append(subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    failed = False
    for job in jobs:
        output, _ = job.communicate()
        if verbose or job.returncode != 0:
            sys.stderr.write(output)
        failed = failed or job.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    _run([_nvcc(), "-shared", "-o", str(target), *map(str, objects)])
    target.with_suffix(".so.stamp").write_text(stamp)
    return target


def build_host(force: bool = False) -> Path:
    OUT.mkdir(exist_ok=True)
    kernels = build_kernels()
    sources = sorted((PKG / "host").glob("*.cpp"))
    headers = sorted((ROOT / "include").rglob("*.h"))
    target = OUT / "libdeepforge_b200.so"
    flags = ["-std=c++20", "-O2", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter"]
    stamp = _stamp(sources + headers, " ".join(flags))
    if not force and _up_to_date(target, stamp):
        return target
    command = ["g++", *flags, "-shared", "-I", str(ROOT / "include"), "-isystem", str(nlohmann_include()),
               *map(str, sources), "-o", str(target), f"-L{OUT}", "-ldfgpu", "-Wl,-rpath,$ORIGIN", "-lpthread"]
    _run(command)
    target.with_suffix(".so.stamp").write_text(stamp)
    assert kernels.exists()
    return target


def build_cli(force: bool = False) -> Path:
    """deepforge-compile (host/cli/deepforge_compile.cpp), linked against the host library beside it."""
    library = build_host()
    source = PKG / "host" / "cli" / "deepforge_compile.cpp"
    headers = sorted((ROOT / "include").rglob("*.h"))
    target = OUT / "deepforge-compile"
    flags = ["-std=c++20", "-O2", "-Wall", "-Wextra"]
    stamp = _stamp([source] + headers, " ".join(flags))
    if not force and _up_to_date(target, stamp):
        return target
    _run(["g++", *flags, "-I", str(ROOT / "include"), str(source), "-o", str(target), f"-L{OUT}", "-ldeepforge_b200", "-ldfgpu",
          "-Wl,-rpath,$ORIGIN", "-lpthread"])
    target.with_suffix(target.suffix + ".stamp").write_text(stamp)
    assert library.exists()
    return target


def cuda_home() -> Path:
    for candidate in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if candidate and (Path(candidate) / "include" / "cuda_runtime_api.h").exists():
            return Path(candidate)
    raise RuntimeError("CUDA toolkit headers not found")


def build_benchmark_tool(force: bool = False) -> Path:
    """deepforge-benchmark (host/cli/deepforge_benchmark.cpp): device buffers and CUDA events through the CUDA runtime."""
    library = build_host()
    source = PKG / "host" / "cli" / "deepforge_benchmark.cpp"
    headers = sorted((ROOT / "include").rglob("*.h"))
    target = OUT / "deepforge-benchmark"
    flags = ["-std=c++20", "-O2", "-Wall", "-Wextra"]
    stamp = _stamp([source] + headers, " ".join(flags))
    if not force and _up_to_date(target, stamp):
        return target
    cuda = cuda_home()
    _run(["g++", *flags, "-I", str(ROOT / "include"), "-isystem", str(cuda / "include"), str(source), "-o", str(target), f"-L{OUT}", "-ldeepforge_b200", "-ldfgpu",
          f"-L{cuda / 'lib64'}", "-lcudart", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{cuda / 'lib64'}", "-lpthread"])
    target.with_suffix(target.suffix + ".stamp").write_text(stamp)
    assert library.exists()
    return target


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_host(force)
    build_cli(force)
    build_benchmark_tool(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built", *sorted(p.name for p in OUT.glob("*.so")))
