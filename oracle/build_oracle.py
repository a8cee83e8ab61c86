"""Builds the CPU oracle libraries (test infrastructure, never the product path).

  oracle/_build/libpa_oracle.so       restatement of the PagedAttention contract (pa_oracle.cpp)
  oracle/_build/libsampler_oracle.so  restatement of LogitProcessor ordering + greedy/multinomial
                                      sampling (sampler_oracle.cpp)
  oracle/_ref/libref_sampler.so       the reference's own sampling/logit_transformers.hpp compiled
                                      unmodified behind oracle/ref_shim (only where the reference
                                      tree is present; the prebuilt file travels otherwise)
  oracle/_ref/libref_eviction.so      the reference's own cache_eviction.cpp + kvcrush.cpp compiled
                                      unmodified behind oracle/ref_shim
"""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD = HERE / "_build"
REF_OUT = HERE / "_ref"
# the reference checkout: GENAI_REFERENCE_ROOT, else a directory named "reference" beside this repository
REFERENCE = Path(os.environ.get("GENAI_REFERENCE_ROOT") or HERE.parent.parent / "reference")

# -ffp-contract=off: the oracle's quantiser / rotation spell out every rounding step.
CXXFLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-pthread"]


def _stale(out: Path, deps) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(Path(d).exists() and Path(d).stat().st_mtime > t for d in deps)


def _run(cmd) -> None:
    res = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("oracle build failed: " + " ".join(map(str, cmd)) + "\n" + res.stdout + res.stderr)


def build_restatements() -> None:
    BUILD.mkdir(exist_ok=True)
    inc = HERE.parent / "include"
    for name in ("pa_oracle", "sampler_oracle"):
        src = HERE / f"{name}.cpp"
        if not src.exists():
            continue
        out = BUILD / f"lib{name}.so"
        if _stale(out, [src, inc / "pa_b200.h", inc / "sampler_b200.h"]):
            _run(["g++", *CXXFLAGS, "-I", inc, src, "-o", out])


def build_reference() -> bool:
    """Compiles the reference's own sources where they lie; returns False if the tree is absent."""
    if not (REFERENCE / "src" / "cpp" / "src" / "sampling" / "logit_transformers.hpp").exists():
        return False
    REF_OUT.mkdir(exist_ok=True)
    shim = HERE / "ref_shim"
    ref_src = REFERENCE / "src" / "cpp" / "src"
    ref_inc = REFERENCE / "src" / "cpp" / "include"
    bridge = HERE / "ref_sampler_bridge.cpp"
    if bridge.exists():
        out = REF_OUT / "libref_sampler.so"
        if _stale(out, [bridge, ref_src / "sampling" / "logit_transformers.hpp"]):
            _run(["g++", *CXXFLAGS, "-I", shim / "sampler", "-I", ref_src, bridge, "-o", out])
    bridge = HERE / "ref_eviction_bridge.cpp"
    if bridge.exists():
        out = REF_OUT / "libref_eviction.so"
        srcs = [ref_src / "continuous_batching" / "cache" / "cache_eviction.cpp",
                ref_src / "continuous_batching" / "cache" / "kvcrush.cpp"]
        if _stale(out, [bridge, *srcs]):
            _run(["g++", *CXXFLAGS, "-I", shim / "eviction", "-I", ref_src, "-I", ref_inc, bridge, *srcs, "-o", out])
    return True


def build_all() -> None:
    build_restatements()
    build_reference()


if __name__ == "__main__":
    build_all()
    print("oracle built")
