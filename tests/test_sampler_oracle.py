"""CPU tests of the Sampler oracle: the reference's golden vectors (tests/golden/logit_filtering.json,
extracted from tests/cpp/logit_filtering.cpp) and, where the reference's own logit_transformers.hpp
was compiled into oracle/_ref, agreement of the restatement with it on random rows."""
import json
from pathlib import Path

import numpy as np
import pytest

from tests import sampler_harness as H
from oracle import sampler_oracle as SO
from openvino_genai_b200 import _sampler_abi as A

GOLD = json.loads((Path(__file__).parent / "golden" / "logit_filtering.json").read_text())["cases"]
TOL = 1e-6


def _by_index(p, idx):
    order = np.argsort(idx)
    return p[order], idx[order]


@pytest.mark.parametrize("case", GOLD["temperature"])
def test_golden_temperature(case):
    p, _, _ = SO.transform(0, case["input"], case["temperature"])
    assert np.allclose(p, case["expected"], atol=TOL)
    assert np.array_equal(p, np.array(case["reference_output"], np.float32))  # bit-exact with the reference's own code


@pytest.mark.parametrize("case", GOLD["top_p"])
def test_golden_top_p(case):
    p, idx, _ = SO.transform(1, case["input"], np.float32(case["top_p"]))
    assert [int(i) for i in idx] == [e["index"] for e in case["expected"]]
    assert np.allclose(p, [e["p"] for e in case["expected"]], atol=TOL)


@pytest.mark.parametrize("case", GOLD["top_k"])
def test_golden_top_k(case):
    p, idx, _ = SO.transform(2, case["input"], case["top_k"])
    p, idx = _by_index(p, idx)
    exp = sorted(case["expected"], key=lambda e: e["index"])
    assert [int(i) for i in idx] == [e["index"] for e in exp]
    assert np.allclose(p, [e["p"] for e in exp], atol=TOL)
    # heap ORDER must equal the reference's own output here (same libstdc++)
    rp = [e["p"] for e in case["reference_output"]]
    p2, idx2, _ = SO.transform(2, case["input"], case["top_k"])
    assert [int(i) for i in idx2] == [e["index"] for e in case["reference_output"]] and np.allclose(p2, rp, atol=0)


def test_golden_top_k_not_applied_when_k_exceeds_size():
    p, idx, data = SO.transform(2, [0.090031, 0.244728, 0.665241], 5)
    assert len(p) == 3 and np.array_equal(idx, [0, 1, 2])


@pytest.mark.parametrize("case", GOLD["min_p"])
def test_golden_min_p(case):
    p, idx, _ = SO.transform(3, case["input"], np.float32(case["min_p"]))
    p, idx = _by_index(p, idx)
    exp = sorted(case["expected"], key=lambda e: e["index"])
    assert [int(i) for i in idx] == [e["index"] for e in exp]
    assert np.allclose(p, [e["p"] for e in exp], atol=1e-5)


def _penalty_step(kind, case):
    """Runs one penalty through the whole-step oracle: greedy row, history = the case's ids as
    generated tokens (the reference's test feeds them through extract_generated_tokens)."""
    x = np.array([case["input"]], np.float32)
    ids = case["input_ids"]
    uniq = sorted(set(ids))
    hist = (np.array([0, len(uniq)], np.int64), np.array(uniq, np.int32),
            np.array([(ids.count(t) << 3) | A.HIST_GENERATED for t in uniq], np.uint32))
    kw = {"repetition": dict(repetition_penalty=case["penalty"]), "frequency": dict(frequency_penalty=case["penalty"]),
          "presence": dict(presence_penalty=case["penalty"])}[kind]
    rows = H.make_rows(1, do_sample=0, **kw)
    rc, tok, lp, lg = H.run_oracle(x, rows, hist)
    return rc, lg[0]


@pytest.mark.parametrize("kind", ["repetition", "frequency", "presence"])
def test_golden_penalties(kind):
    for case in GOLD[kind]:
        rc, out = _penalty_step(kind, case)
        assert rc == 0
        assert np.allclose(out, case["expected"], atol=TOL), (kind, case)
        assert np.array_equal(out, np.array(case["reference_output"], np.float32)), "differs from the reference's own code"


@pytest.mark.parametrize("case", GOLD["out_of_range_ids_throw"])
def test_out_of_range_history_ids_are_errors(case):
    x = np.array([[43.0]], np.float32)
    ids = case["input_ids"]
    hist = (np.array([0, len(ids)], np.int64), np.array(ids, np.int32), np.array([(1 << 3) | A.HIST_GENERATED] * len(ids), np.uint32))
    rc, *_ = H.run_oracle(x, H.make_rows(1, do_sample=0, repetition_penalty=1.5), hist)
    assert rc == A.SAMPLER_ERR_BAD_TOKEN_ID


@pytest.mark.parametrize("case", GOLD["eos"])
def test_golden_eos_mask(case):
    x = np.array([case["input"]], np.float32)
    ids = sorted(case["stop_token_ids"])
    hist = (np.array([0, len(ids)], np.int64), np.array(ids, np.int32), np.array([A.HIST_STOP_MASK] * len(ids), np.uint32))
    rc, tok, lp, lg = H.run_oracle(x, H.make_rows(1, do_sample=0), hist)
    exp = np.array([float(v) for v in case["expected"]], np.float32)
    assert rc == 0 and np.array_equal(lg[0], exp)


def test_raw_log_probability_rows_report_the_unpenalised_logit():
    """logprobs > 0 (logit_processor.hpp:36-47, sampler.cpp:967-974): same token, log-probability =
    raw logit - log-partition of the raw row."""
    rng = np.random.default_rng(8)
    x = (rng.standard_normal((3, 500)) * 3).astype(np.float32)
    hist = H.make_history(rng, 3, 500, generated_len=40)
    for do_sample, kw in ((0, {}), (1, dict(top_k=10, temperature=0.7)), (1, dict(top_k=10, top_p=0.8))):
        rows = H.make_rows(3, do_sample=do_sample, repetition_penalty=1.5, presence_penalty=0.5, **kw)
        rows["rand_u"] = rng.random(3, dtype=np.float32)
        rc, tok0, _, _ = H.run_oracle(x, rows, hist)
        assert rc == 0
        rows["do_sample"] |= A.ROW_RAW_LOG_PROB
        rc, tok1, lp1, _ = H.run_oracle(x, rows, hist)
        assert rc == 0 and np.array_equal(tok0, tok1)
        x64 = x.astype(np.float64)
        lse = np.log(np.exp(x64 - x64.max(axis=1, keepdims=True)).sum(axis=1)) + x64.max(axis=1)
        np.testing.assert_allclose(lp1, x64[np.arange(3), tok1] - lse, atol=1e-5, rtol=0)


def test_uniform_stream_is_the_mt19937_stream():
    u = SO.uniform_stream(0, 2)
    assert abs(float(u[0]) - 0.548813522) < 1e-7 and abs(float(u[1]) - 0.592844605) < 1e-7


def test_greedy_ties_pick_lowest_index():
    x = np.array([[1.0, 5.0, 5.0, np.nan, 5.0]], np.float32)
    rc, tok, lp, _ = H.run_oracle(x, H.make_rows(1, do_sample=0))
    assert rc == 0 and tok[0] == 1 and lp[0] == 0.0


def test_deferred_expf_path_matches_normalised_path_distribution():
    """top_k active with top_p == 1 defers expf; the chosen token for a given u must be the one
    the explicit softmax CDF over the same heap order gives."""
    rng = np.random.default_rng(5)
    x = H.synthetic_logits(rng, 4, 500)
    rows = H.make_rows(4, top_k=7, temperature=0.7)
    rc, tok, lp, _ = H.run_oracle(x, rows)
    assert rc == 0
    for r in range(4):
        p, idx, _ = SO.transform(2, x[r], 7)
        z = (p * np.float32(1.0 / np.float32(0.7))).astype(np.float32)
        w = np.exp((z - z.max()).astype(np.float64))
        cdf = np.cumsum(w)
        pick = int(np.searchsorted(cdf, cdf[-1] * rows["rand_u"][r], side="right"))
        assert tok[r] == idx[min(pick, 6)]


needs_ref = pytest.mark.skipif(SO.ref_lib() is None, reason="oracle/_ref/libref_sampler.so was not built (no reference tree)")


@needs_ref
@pytest.mark.parametrize("which,param", [(0, 0.7), (0, 1.0), (1, 0.9), (1, 0.3), (2, 50), (2, 1), (3, 0.05)])
def test_restatement_equals_reference_transform(which, param):
    rng = np.random.default_rng(100 + which)
    for trial in range(5):
        n = int(rng.integers(60, 3000))
        x = (rng.standard_normal(n) * 2).astype(np.float32)
        if which in (1, 3):  # these expect probabilities
            e = np.exp(x - x.max())
            x = (e / e.sum()).astype(np.float32)
        pr = np.float32(param) if which in (1, 3) else param
        p1, i1, d1 = SO.transform(which, x, pr)
        p2, i2, d2 = SO.transform(which, x, pr, use_reference=True)
        assert np.array_equal(i1, i2) and np.array_equal(p1, p2) and np.array_equal(d1, d2)


@needs_ref
def test_restatement_equals_reference_chain():
    import ctypes as C
    ref = SO.ref_lib()
    rng = np.random.default_rng(7)
    for top_k, T, top_p, min_p in [(50, 0.7, 0.9, 0.0), (20, 1.0, 1.0, 0.0), (A.TOP_K_OFF, 0.8, 0.95, 0.0), (40, 1.3, 0.8, 0.02),
                                   (A.TOP_K_OFF, 1.0, 1.0, 0.0)]:
        x = H.synthetic_logits(rng, 1, 4000)[0]
        buf = x.copy()
        p = np.zeros(len(x), np.float32)
        idx = np.zeros(len(x), np.int64)
        deferred = C.c_int(0)
        n = ref.ref_filter_chain(buf.ctypes.data, len(x), top_k, T, top_p, min_p, p.ctypes.data, idx.ctypes.data, C.byref(deferred))
        # the oracle's draw must land on the element the reference's candidate list gives for the same u
        rows = H.make_rows(1, top_k=top_k, temperature=T, top_p=top_p, min_p=min_p, seeds=[3])
        rc, tok, lp, _ = H.run_oracle(x[None, :], rows)
        assert rc == 0
        w = p[:n].astype(np.float32)
        if deferred.value:
            w = np.array([np.float32(np.exp(np.float32(v - w.max()))) for v in w], np.float32)
        total = np.float32(0)
        for v in w:
            total = np.float32(total + v)
        r = np.float32(total * rows["rand_u"][0])
        run, pick = np.float32(0), n - 1
        for i, v in enumerate(w):
            run = np.float32(run + v)
            if run > r:
                pick = i
                break
        assert tok[0] == idx[pick], (top_k, T, top_p, min_p)
