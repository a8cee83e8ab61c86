"""Regenerates tests/golden/logit_filtering.json and tests/golden/rotation_lut.json from the
reference's own unit tests (run where the reference tree is mounted; the JSON files travel).

Sources, read as text:
  tests/cpp/logit_filtering.cpp            parameterised golden vectors of every logit transform
  tests/cpp/data/cache_rotation_poc_ref_coefficients_per_block_{0..3}.txt   fp16 PoC rotation dumps
Each case is also run through the reference's own logit_transformers.hpp (compiled unmodified
into oracle/_ref/libref_sampler.so) and the observed output is stored beside the expected one,
so the fixture records both what the reference's test expects and what its code produces here.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import re
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
REF = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(os.environ.get("GENAI_REFERENCE_ROOT") or ROOT.parent / "reference")
sys.path.insert(0, str(ROOT))


def _cases(text: str, name: str):
    m = re.search(r"const\s+std::vector<\w+>\s+" + name + r"\s*=\s*\{(.*?)\n\};", text, re.S)
    body = m.group(1)
    body = re.sub(r"//[^\n]*", "", body)
    body = body.replace("-std::numeric_limits<float>::infinity()", '"-inf"')
    body = re.sub(r"\b[A-Z]\w*(?:TestStruct|Ids)\b", "", body)       # type names before braces
    body = re.sub(r"(?<=[0-9.])f\b", "", body)                        # float suffixes
    body = body.replace("{", "[").replace("}", "]")
    body = re.sub(r",\s*\]", "]", body)
    return json.loads("[" + body.strip().rstrip(",") + "]")


def main():
    text = (REF / "tests/cpp/logit_filtering.cpp").read_text()
    out = {"source": "tests/cpp/logit_filtering.cpp", "tolerance": 1e-6, "cases": {}}
    out["cases"]["temperature"] = [{"temperature": c[0], "input": c[1], "expected": c[2]} for c in _cases(text, "TEMPERATURE_TRANSFORM_TEST_CASES")]
    out["cases"]["top_p"] = [{"top_p": c[0], "input": c[1], "expected": [{"p": e[0], "index": e[1]} for e in c[2]]} for c in _cases(text, "TOP_P_TRANSFORM_TEST_CASES")]
    out["cases"]["top_k"] = [{"top_k": c[0], "input": c[1], "expected": [{"p": e[0], "index": e[1]} for e in c[2]]} for c in _cases(text, "TOP_K_TRANSFORM_TEST_CASES")]
    for key, name in (("repetition", "REPETITION_PENALTY_TRANSFORM_TEST_CASES"), ("frequency", "FREQUENCY_PENALTY_TRANSFORM_TEST_CASES"),
                      ("presence", "PRESENCE_PENALTY_TRANSFORM_TEST_CASES")):
        out["cases"][key] = [{"penalty": c[0], "input": c[1], "input_ids": c[2], "expected": c[3]} for c in _cases(text, name)]
    out["cases"]["eos"] = [{"stop_token_ids": c[0], "input": c[1], "expected": c[2]} for c in _cases(text, "EOS_PENALTY_TRANSFORM_TEST_CASES")]
    out["cases"]["min_p"] = [{"min_p": c[0], "input": c[1], "expected": [{"p": e[0], "index": e[1]} for e in c[2]]} for c in _cases(text, "MIN_P_TRANSFORM_TEST_CASES")]
    out["cases"]["out_of_range_ids_throw"] = [{"vocab": 1, "input_ids": [1337]}, {"vocab": 1, "input_ids": [0, -1]}]

    # what the reference's own code produces here
    from oracle import build_oracle
    build_oracle.build_reference()
    ref = C.CDLL(str(build_oracle.REF_OUT / "libref_sampler.so"))

    def run_transform(which, data, param):
        x = np.array(data, np.float32)
        p = np.zeros(len(x), np.float32)
        idx = np.zeros(len(x), np.int64)
        ref.ref_transform.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_double, C.c_void_p, C.c_void_p]
        n = ref.ref_transform(which, x.ctypes.data, len(x), float(param), p.ctypes.data, idx.ctypes.data)
        return [{"p": float(p[i]), "index": int(idx[i])} for i in range(n)]

    for c in out["cases"]["temperature"]:
        c["reference_output"] = [e["p"] for e in run_transform(0, c["input"], c["temperature"])]
    for c in out["cases"]["top_p"]:
        c["reference_output"] = run_transform(1, c["input"], np.float32(c["top_p"]))
    for c in out["cases"]["top_k"]:
        c["reference_output"] = run_transform(2, c["input"], c["top_k"])
    for c in out["cases"]["min_p"]:
        c["reference_output"] = run_transform(3, c["input"], np.float32(c["min_p"]))
    ref.ref_penalty.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_double, C.c_void_p, C.c_int, C.c_void_p, C.c_int]
    for which, key in ((0, "repetition"), (1, "frequency"), (2, "presence")):
        for c in out["cases"][key]:
            x = np.array(c["input"], np.float32)
            ids = np.array(c["input_ids"], np.int64)
            empty = np.zeros(1, np.int64)
            rc = ref.ref_penalty(which, x.ctypes.data, len(x), float(np.float32(c["penalty"])), empty.ctypes.data, 0, ids.ctypes.data, len(ids))
            assert rc == 0
            c["reference_output"] = [float(v) for v in x]
    (HERE / "logit_filtering.json").write_text(json.dumps(out, indent=1))

    # rotation coefficient dumps (fp16 PoC): per block, sin rows then cos rows
    rot = {"source": "tests/cpp/data/cache_rotation_poc_ref_coefficients_per_block_{0..3}.txt",
           "note": "format parsed as tests/cpp/cache_eviction.cpp:1552-1602 does; tolerance 1e-2 there", "blocks": []}
    for i in range(4):
        lines = (REF / f"tests/cpp/data/cache_rotation_poc_ref_coefficients_per_block_{i}.txt").read_text().split("\n")
        rot["blocks"].append([ln for ln in lines if ln.strip()])
    (HERE / "rotation_poc_coefficients.json").write_text(json.dumps(rot))
    print("golden fixtures written")


if __name__ == "__main__":
    main()
