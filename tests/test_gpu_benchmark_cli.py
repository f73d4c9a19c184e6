"""The reference-compatible benchmark command line runs on a B200 and prints its correctness line and table."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_benchmark_cli_one_sequence_length():
    r = subprocess.run([sys.executable, "-m", "tinyfa_b200.benchmark", "--head-dim", "128", "--dtype", "bf16", "--causal",
                        "--seqlens", "1024"], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    out = r.stdout
    assert "dtype=bf16 head_dim=128 causal=True batch=2 heads=32" in out
    verdicts = [line for line in out.splitlines() if "tinyfa vs" in line]
    assert len(verdicts) == 1 and "[PASS]" in verdicts[0] and "cos_sim=" in verdicts[0], out
    rows = [line.split() for line in out.splitlines() if line.strip().startswith("1024")]
    assert len(rows) == 1
    ms, tflops = float(rows[0][1]), float(rows[0][2])
    assert ms > 0 and tflops > 50  # far above any CPU or fallback path: the CUDA kernel ran
