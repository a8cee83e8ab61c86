"""In-tree build of the sm_100a shared libraries (and of the CPU oracle used by tests).

`build_all()` compiles every `.cu` under `csrc/` for `sm_100a` with nvcc and links them into
`lib/libgenai_b200.so`, the C-ABI library declared in `include/*.h`.  nvcc cross-compiles, so
this works on a machine without a GPU.  Objects are rebuilt only when a source or header is
newer than the object.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = LIB_DIR / "libgenai_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA extension cannot be built")


def _newest_header_mtime() -> float:
    headers = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.hpp")) + list((REPO_ROOT / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def _compile_one(src: Path, obj: Path, log: Path) -> None:
    extra = os.environ.get("GENAI_B200_NVCC_EXTRA", "").split()   # e.g. -DSAMPLER_EXACT_PROF for the kernels' own timers
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-I", str(REPO_ROOT / "include"), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")


def build_all(force: bool = False, verbose: bool = False) -> Path:
    """Builds lib/libgenai_b200.so and returns its path."""
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.rglob("*.cu")) + sorted(CSRC.rglob("*.cpp"))
    hdr_mtime = _newest_header_mtime()
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_mtime)
        if stale:
            jobs.append((src, obj, OBJ_DIR / (src.stem + ".log")))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            futs = [pool.submit(_compile_one, *j) for j in jobs]
            for f in futs:
                f.result()
        if verbose:
            for _, _, log in jobs:
                sys.stderr.write(log.read_text())
    if jobs or not LIB_PATH.exists():
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose=True))
