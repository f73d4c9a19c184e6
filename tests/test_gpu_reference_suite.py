"""The reference's own C++ test binary and example, compiled UNCHANGED against the drop-in header.

tests/cpp_compat/build.sh compiles reference tests/cpp/test.cpp + test_flash_attn.cu (180 gtest cases, CPU oracle
and tolerances of the reference itself) and examples/basic/main.cu where the reference checkout is present; the
binaries travel with the repository snapshot.  Skipped when they were not built.
"""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu

BUILD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpp_compat", "_build")


@pytest.mark.skipif(not os.path.exists(os.path.join(BUILD, "ref_suite")), reason="reference suite not built")
def test_reference_gtest_suite_passes_unchanged():
    r = subprocess.run([os.path.join(BUILD, "ref_suite")], capture_output=True, text=True, timeout=900)
    tail = r.stdout.strip().splitlines()[-1] if r.stdout.strip() else ""
    m = re.search(r"(\d+) tests: (\d+) passed, (\d+) failed, (\d+) skipped", tail)
    assert r.returncode == 0 and m, (r.stdout[-2000:], r.stderr[-2000:])
    total, passed, failed, skipped = map(int, m.groups())
    assert total == 180 and passed == 180 and failed == 0 and skipped == 0, tail


@pytest.mark.skipif(not os.path.exists(os.path.join(BUILD, "basic_example")), reason="reference example not built")
def test_reference_basic_example_runs_unchanged():
    r = subprocess.run([os.path.join(BUILD, "basic_example")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "completed successfully" in r.stdout, (r.stdout, r.stderr)
