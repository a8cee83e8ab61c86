"""Builds and runs tests/cpp/host_layer_test.cpp: the C++ host layer (GenerationConfig, the
ModelRunner marshalling mirror, the host half of the Sampler) over the C-ABI library."""
from __future__ import annotations

import json
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402



def _cuda_home() -> Path:
    entry.load_package()
    """The toolkit the library was built with: CUDA_HOME, else the directory two levels above nvcc."""
    import os
    if os.environ.get("CUDA_HOME"):
        return Path(os.environ["CUDA_HOME"])
    from openvino_genai_b200 import build
    return Path(build._nvcc()).resolve().parent.parent


CUDA_INC = _cuda_home() / "include"
CUDA_LIB = _cuda_home() / "lib64"


def _build(tmp: Path) -> Path:
    pkg = entry.load_package()
    lib = Path(pkg.library_path())
    assert lib.exists(), "the C-ABI library must be built first (python -c 'import __graft_entry__ as g; g.build()')"
    exe = tmp / "host_layer_test"
    cmd = [shutil.which("g++") or "g++", "-std=c++17", "-O1", str(ROOT / "tests" / "cpp" / "host_layer_test.cpp"),
           "-I", str(ROOT / "include"), "-I", str(ROOT / "openvino.genai_b200" / "csrc" / "host"), "-I", str(CUDA_INC),
           "-L", str(lib.parent), "-lgenai_b200", "-L", str(CUDA_LIB), "-lcudart", "-ldl",
           f"-Wl,-rpath,{lib.parent}", f"-Wl,-rpath,{CUDA_LIB}", "-o", str(exe)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    return exe


def _rotation_fixture(tmp: Path) -> Path:
    blocks = json.loads((ROOT / "tests" / "golden" / "rotation_poc_coefficients.json").read_text())["blocks"]
    path = tmp / "rotation_poc.txt"
    path.write_text(str(len(blocks)) + "\n" + "\n".join(" ".join(tokens) for tokens in blocks) + "\n")
    return path


def test_host_layer_cpu(tmp_path):
    exe = _build(tmp_path)
    res = subprocess.run([str(exe), "cpu", str(_rotation_fixture(tmp_path))], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failed" in res.stdout


@pytest.mark.gpu
def test_host_layer_sampler_generations_match_restatement(tmp_path):
    from oracle import build_oracle
    build_oracle.build_restatements()
    exe = _build(tmp_path)
    res = subprocess.run([str(exe), "gpu", str(build_oracle.BUILD / "libsampler_oracle.so")], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failed" in res.stdout
