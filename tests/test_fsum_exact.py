"""Builds and runs tests/cpp/fsum_exact_test.cpp: the host libm's expf restated, float sums as scans of
two-state steps, and the sorted walk of the exact top-p procedure against std::sort + sequential sums
(the same header the CUDA kernel is compiled from, plus a sequential model of the kernel's passes)."""
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_fsum_exact_host_checks(tmp_path):
    exe = tmp_path / "fsum_exact_test"
    cmd = ["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-I", str(ROOT / "openvino.genai_b200" / "csrc"), "-I", str(ROOT / "tests" / "cpp"),
           str(ROOT / "tests" / "cpp" / "fsum_exact_test.cpp"), "-o", str(exe)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe), "4099", "160"], capture_output=True, text=True)
    sys.stdout.write(run.stdout)
    assert run.returncode == 0, run.stdout + run.stderr
