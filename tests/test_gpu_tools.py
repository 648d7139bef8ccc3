"""The native tools on a GPU: deepforge-benchmark runs the reference tool's three single-node convolution profiles
through compile_graph and Executable::execute on device buffers, checks one pass against its own double-precision
host convolution before timing, and prints one CSV row per profile and policy."""
import csv
import io
import subprocess

import pytest

from deepforge_b200 import build

pytestmark = pytest.mark.gpu


def test_benchmark_tool_checks_then_times_every_profile():
    tool = build.build_benchmark_tool()
    result = subprocess.run([str(tool), "--profile=all", "--schedule=both", "--iterations=20"], capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stderr
    rows = list(csv.DictReader(io.StringIO(result.stdout)))
    assert [(r["profile"], r["policy"]) for r in rows] == [(p, s) for p in ("small", "medium", "large") for s in ("baseline", "auto")]
    for row in rows:
        assert row["variant"] == "sm_100a" and row["schedule"] == "kernel-plan" and int(row["iterations"]) == 20
        assert float(row["execute_ms"]) > 0 and float(row["gflops"]) > 0
        # the compared pass held the reference's acceptance rule, so the recorded deviations are small
        assert float(row["max_abs"]) <= 1e-3 and float(row["max_rel"]) < 1.0
    # the large profile runs on tcgen05 in one launch (operands split on their way into shared memory): no scratch either
    assert rows[-1]["shape"] == "1x56x56x64_k64_r3x3" and rows[-1]["workspace_bytes"] == "0"
    assert rows[0]["workspace_bytes"] == "0"  # (the small profile has too few channels for it: CUDA cores)
