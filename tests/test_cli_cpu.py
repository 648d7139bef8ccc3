"""deepforge-compile: the command line, output lines and exit codes of the reference's tool
(tools/deepforge-compile.cpp:50-63, 385-474; docs/user-guide.en.md:313-317): 0 done, 1 the compilation or a
file operation failed, 2 the command line is wrong."""
import json
import subprocess
from pathlib import Path

import pytest

from deepforge_b200 import build, graphs, runtime


@pytest.fixture(scope="module")
def tool() -> Path:
    return build.build_cli()


def run(tool: Path, *arguments, cwd: Path):
    return subprocess.run([str(tool), *map(str, arguments)], cwd=cwd, capture_output=True, text=True, timeout=120)


def test_compile_inspect_and_plan(tool, tmp_path: Path):
    document = graphs.c2_bottleneck(n=1, h=8, w=8)
    (tmp_path / "bottleneck.json").write_text(json.dumps(document))
    done = run(tool, "bottleneck.json", "--dump-plan=plan.txt", cwd=tmp_path)
    assert done.returncode == 0, done.stderr
    exe = runtime.compile_graph(document)
    assert done.stdout.splitlines() == ['output: "bottleneck.dfo"', "target: sm_100a", f"workspace: {exe.workspace_size} bytes"]
    assert (tmp_path / "bottleneck.dfo").read_bytes() == exe.serialize()  # the tool and the library write the same bytes
    assert (tmp_path / "plan.txt").read_text() == exe.plan_text()
    assert sorted(p.name for p in tmp_path.iterdir()) == ["bottleneck.dfo", "bottleneck.json", "plan.txt"]  # no temporaries left
    inspected = run(tool, "--inspect", "bottleneck.dfo", cwd=tmp_path)
    assert inspected.returncode == 0
    lines = inspected.stdout.splitlines()
    assert lines[:8] == ["format: DFOBJ/13", "deepforge: deepforge_b200 1", "llvm: ", "frontend: 1.24.0", "target: sm_100a",
                         "function: deepforge_graph", "uids: 1,2,3,4,5,6,7", f"workspace: {exe.workspace_size} bytes"]
    assert [line.split("]")[0] for line in lines[8:]] == ["launch: [conv1+bias1+relu1", "launch: [conv2+bias2+relu2>conv3+residual"]
    plan = run(tool, "bottleneck.json", "--emit=plan", "-o", "out.plan", "--no-fusion", cwd=tmp_path)
    assert plan.returncode == 0 and plan.stdout.splitlines()[0] == 'output: "out.plan"'
    assert (tmp_path / "out.plan").read_text() == runtime.compile_graph(document, options=runtime.NO_FUSION).plan_text()


def test_exit_codes(tool, tmp_path: Path):
    assert run(tool, "--help", cwd=tmp_path).returncode == 0
    assert "DFOBJ/13" in run(tool, "--version", cwd=tmp_path).stdout
    for arguments in (["--bogus"], [], ["a.json", "b.json"], ["--emit=object", "a.json"], ["--target=x86-64", "a.json"],
                      ["--inspect", "a.dfo", "--emit=plan"], ["a.json", "-o"], ["--input-format=xml", "a.json"]):
        result = run(tool, *arguments, cwd=tmp_path)
        assert result.returncode == 2 and result.stderr.startswith("deepforge-compile: ") and "usage:" in result.stderr, arguments
    missing = run(tool, "missing.json", cwd=tmp_path)
    assert missing.returncode == 1 and missing.stderr.startswith("DFE_IO_ERROR")
    (tmp_path / "bad.json").write_text("{not json")
    assert run(tool, "bad.json", cwd=tmp_path).returncode == 1
    unsupported = graphs.c1_conv(n=1, c=3, h=5, w=5, k=5)
    unsupported["nodes"][0]["tag"] = "RMS_NORM"
    (tmp_path / "norm.json").write_text(json.dumps(unsupported))
    rejected = run(tool, "norm.json", cwd=tmp_path)
    assert rejected.returncode == 1 and rejected.stderr.startswith("DFE_UNSUPPORTED_NODE") and not (tmp_path / "norm.dfo").exists()
    (tmp_path / "short.dfo").write_bytes(b"DFOBJ\r\n\x1a")
    truncated = run(tool, "--inspect", "short.dfo", cwd=tmp_path)
    assert truncated.returncode == 1 and truncated.stderr.startswith("DFE_PARSE_ERROR")
    (tmp_path / "ok.json").write_text(json.dumps(graphs.matmul_fp8(2, 2, 2)))
    nowhere = run(tool, "ok.json", "-o", "no_such_directory/x.dfo", cwd=tmp_path)
    assert nowhere.returncode == 1 and nowhere.stderr.startswith("DFE_IO_ERROR")


def test_benchmark_tool_command_line():
    """deepforge-benchmark keeps the reference tool's command line and exit codes (tools/deepforge-benchmark.cpp:58-103,
    :315-345): --help prints the usage and exits 0, a bad option prints it on stderr and exits 2; without a CUDA device
    the run itself fails with exit code 1 (there is no CPU path to fall back to)."""
    from deepforge_b200 import build
    tool = build.build_benchmark_tool()
    result = subprocess.run([str(tool), "--help"], capture_output=True, text=True)
    assert result.returncode == 0 and result.stdout.startswith("usage: deepforge-benchmark [--profile=small|medium|large|all]")
    for bad in (["--profile=huge"], ["--schedule=fast"], ["--iterations=0"], ["--iterations=1001"], ["--iterations=3x"], ["--surprise"]):
        result = subprocess.run([str(tool), *bad], capture_output=True, text=True)
        assert result.returncode == 2 and "usage:" in result.stderr, bad
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except ImportError:
        has_gpu = False
    if not has_gpu:
        result = subprocess.run([str(tool), "--profile=small"], capture_output=True, text=True)
        assert result.returncode == 1 and "no CUDA device" in result.stderr
