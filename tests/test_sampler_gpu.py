"""Parity of the CUDA Sampler step (through the C ABI) with the CPU oracle.

Token ids must be identical for greedy rows and for multinomial rows on the top-k path (the heap
order, every float sum and the draw are reproduced step for step); penalised logits must be
bit-identical.  The full-vocabulary multinomial path sums in a different (deterministic) order
than the reference's index-order float loop, so there the agreement rate is measured and bounded."""
import numpy as np
import pytest
import torch

from tests import sampler_harness as H
from openvino_genai_b200 import _sampler_abi as A

pytestmark = pytest.mark.gpu

VOCAB = 151936


@pytest.fixture(scope="module")
def gpu():
    return H.GpuSampler()


def _both(gpu, x, rows, hist=None):
    rc_o, tok_o, lp_o, lg_o = H.run_oracle(x, rows, hist)
    rc_g, tok_g, lp_g, lg_g = gpu.step_host(x, rows, hist)
    assert rc_o == 0 and rc_g == 0, (rc_o, rc_g, gpu.lib.sampler_b200_last_error())
    return tok_o, lp_o, lg_o, tok_g, lp_g, lg_g


def test_greedy_with_penalties_is_bit_exact(gpu):
    rng = np.random.default_rng(1)
    n = 24
    x = H.synthetic_logits(rng, n, VOCAB)
    hist = H.make_history(rng, n, VOCAB, generated_len=1024, prompt_len=200)
    rows = H.make_rows(n, do_sample=0, repetition_penalty=1.1, presence_penalty=0.2, frequency_penalty=0.1)
    tok_o, lp_o, lg_o, tok_g, lp_g, lg_g = _both(gpu, x, rows, hist)
    assert np.array_equal(tok_o, tok_g)
    assert np.array_equal(lg_o.view(np.uint32), lg_g.view(np.uint32)), "penalised logits differ"
    assert np.all(lp_g == 0)


def test_greedy_ties_nan_and_all_masked(gpu):
    x = np.zeros((3, 1000), np.float32)
    x[0, [10, 500, 999]] = 7.0
    x[1, :] = -np.inf
    x[2, :] = 1.0
    x[2, 3] = np.nan
    x[2, 800] = 2.0
    tok_o, _, _, tok_g, _, _ = _both(gpu, x, H.make_rows(3, do_sample=0))
    assert list(tok_g) == [10, 0, 800] and np.array_equal(tok_o, tok_g)


@pytest.mark.parametrize("top_k,T,top_p,min_p", [(50, 0.7, 0.9, 0.0), (50, 0.7, 1.0, 0.0), (1, 1.0, 1.0, 0.0), (1000, 1.2, 0.5, 0.0),
                                                  (64, 0.9, 0.95, 0.05), (8, 1.0, 0.3, 0.0)])
def test_top_k_path_tokens_are_identical(gpu, top_k, T, top_p, min_p):
    rng = np.random.default_rng(top_k)
    n = 16
    x = H.synthetic_logits(rng, n, VOCAB)
    hist = H.make_history(rng, n, VOCAB, generated_len=1024)
    rows = H.make_rows(n, top_k=top_k, temperature=T, top_p=top_p, min_p=min_p, repetition_penalty=1.1, presence_penalty=0.2,
                       frequency_penalty=0.1, seeds=np.arange(n) + 100 * top_k)
    tok_o, lp_o, lg_o, tok_g, lp_g, lg_g = _both(gpu, x, rows, hist)
    assert np.array_equal(tok_o, tok_g), f"{(tok_o != tok_g).sum()} of {n} tokens differ"
    assert np.array_equal(lg_o.view(np.uint32), lg_g.view(np.uint32))
    assert np.allclose(lp_o, lp_g, atol=2e-6, rtol=1e-6)


def test_top_k_adversarial_orders(gpu):
    """Ascending rows make every element enter the heap; descending rows none after the seed."""
    v = 20000
    x = np.stack([np.linspace(-5, 5, v), np.linspace(5, -5, v), np.zeros(v)]).astype(np.float32)
    rows = H.make_rows(3, top_k=16, temperature=0.8, top_p=0.9, seeds=[5, 6, 7])
    tok_o, lp_o, _, tok_g, lp_g, _ = _both(gpu, x, rows)
    assert np.array_equal(tok_o, tok_g)


@pytest.mark.parametrize("top_k,top_p", [(100, 0.9), (40, 0.99), (600, 0.97), (17, 0.5)])
def test_top_k_path_with_many_equal_logits(gpu, top_k, top_p):
    """Coarsely quantised logits give equal probabilities; the scan order of equal candidates is
    whatever std::partial_sort / std::sort leave, which the kernel restates."""
    rng = np.random.default_rng(top_k + 3)
    n = 12
    x = (np.round(rng.standard_normal((n, 30000)) * 4) / 4).astype(np.float32)
    rows = H.make_rows(n, top_k=top_k, temperature=0.9, top_p=top_p, seeds=np.arange(n) + 77)
    tok_o, lp_o, _, tok_g, lp_g, _ = _both(gpu, x, rows)
    assert np.array_equal(tok_o, tok_g), f"{(tok_o != tok_g).sum()} of {n} tokens differ"


def test_small_vocab_and_k_not_below_vocab(gpu):
    rng = np.random.default_rng(9)
    x = (rng.standard_normal((5, 40)) * 2).astype(np.float32)
    rows = H.make_rows(5, top_k=50, temperature=0.7, top_p=1.0, seeds=[1, 2, 3, 4, 5])  # k >= vocab: full-vocabulary path
    tok_o, _, _, tok_g, _, _ = _both(gpu, x, rows)
    assert np.array_equal(tok_o, tok_g)


def test_row_indirection_and_device_entry(gpu):
    rng = np.random.default_rng(11)
    x = H.synthetic_logits(rng, 6, 32000)
    order = np.array([4, 0, 5], np.int64)
    rows = H.make_rows(3, top_k=50, temperature=0.7, top_p=0.9, logits_rows=order, seeds=[8, 9, 10])
    rc_o, tok_o, lp_o, lg_o = H.run_oracle(x, rows)
    xt = torch.from_numpy(x).cuda()
    rc, tok, lp = gpu.step_device(xt, rows)
    torch.cuda.synchronize()
    assert rc == 0 and np.array_equal(tok.cpu().numpy(), tok_o)


def test_full_vocab_top_p_agreement_rate(gpu):
    """Llama-3 vocabulary, T = 1, top_p = 0.95, no top-k: sums are not taken in the reference's
    order, so agreement is statistical.  The measured rate is printed; the bound is loose."""
    rng = np.random.default_rng(21)
    n, v = 48, 128256
    x = (rng.standard_normal((n, v)) * 2).astype(np.float32)
    rows = H.make_rows(n, top_p=0.95, seeds=np.arange(n) + 1000)
    tok_o, lp_o, _, tok_g, lp_g, _ = _both(gpu, x, rows)
    rate = float((tok_o == tok_g).mean())
    print(f"full-vocab top-p agreement {rate:.3f}")
    assert rate >= 0.6
    same = tok_o == tok_g
    assert np.allclose(lp_o[same], lp_g[same], atol=1e-3)


def test_full_vocab_plain_sampling_agreement_rate(gpu):
    rng = np.random.default_rng(22)
    n, v = 32, 32000
    x = H.synthetic_logits(rng, n, v)
    rows = H.make_rows(n, temperature=0.8, seeds=np.arange(n) + 2000)
    tok_o, _, _, tok_g, _, _ = _both(gpu, x, rows)
    rate = float((tok_o == tok_g).mean())
    print(f"full-vocab index-order agreement {rate:.3f}")
    assert rate >= 0.9


@pytest.mark.parametrize("mode", ["greedy", "top_k", "top_k_deferred", "plain"])
def test_raw_log_probabilities_for_logprobs_rows(gpu, mode):
    """logprobs > 0: the same token as without the flag, and its log-probability is the raw logit
    minus the log-partition of the raw row, also for a token the penalties rewrote."""
    rng = np.random.default_rng(41)
    n, vocab = 12, 32000
    x = H.synthetic_logits(rng, n, vocab)
    hist = H.make_history(rng, n, vocab, generated_len=300, prompt_len=50)
    # make the strongest logit of every row a penalised one, so that greedy rows pick a rewritten token
    for r in range(n):
        x[r, hist[1][hist[0][r]]] = 40.0
    kw = dict(repetition_penalty=1.3, presence_penalty=0.3, frequency_penalty=0.2)
    if mode == "greedy":
        kw.update(do_sample=0)
    elif mode == "top_k":
        kw.update(top_k=40, temperature=0.8, top_p=0.9)
    elif mode == "top_k_deferred":
        kw.update(top_k=40, temperature=0.8)
    else:
        kw.update(temperature=1.3)
    rows = H.make_rows(n, **kw)
    rows["rand_u"] = rng.random(n, dtype=np.float32)
    flagged = rows.copy()
    flagged["do_sample"] |= A.ROW_RAW_LOG_PROB
    tok_plain = _both(gpu, x, rows, hist)[3]
    tok_o, lp_o, _, tok_g, lp_g, _ = _both(gpu, x, flagged, hist)
    assert np.array_equal(tok_g, tok_plain)
    if mode != "plain":   # the full-vocabulary path is compared by agreement rate elsewhere
        assert np.array_equal(tok_g, tok_o)
    x64 = x.astype(np.float64)
    lse = np.log(np.exp(x64 - x64.max(axis=1, keepdims=True)).sum(axis=1)) + x64.max(axis=1)
    want = x64[np.arange(n), tok_g] - lse
    np.testing.assert_allclose(lp_g, want, rtol=0, atol=2e-5)
    same = tok_g == tok_o
    np.testing.assert_allclose(lp_g[same], lp_o[same], rtol=0, atol=2e-5)
    # the device entry point with its scratch gives the same answer
    xt = torch.from_numpy(x).cuda()
    rc, tok_d, lp_d = gpu.step_device(xt, flagged, hist)
    torch.cuda.synchronize()
    assert rc == 0
    assert np.array_equal(tok_d.cpu().numpy(), tok_g)
    np.testing.assert_array_equal(lp_d.cpu().numpy(), lp_g)


def test_raw_log_probabilities_need_the_scratch_on_the_device_entry(gpu):
    rng = np.random.default_rng(42)
    x = H.synthetic_logits(rng, 2, 4096)
    hist = H.make_history(rng, 2, 4096, generated_len=10)
    rows = H.make_rows(2, do_sample=0, repetition_penalty=1.2)
    rows["do_sample"] |= A.ROW_RAW_LOG_PROB
    xt = torch.from_numpy(x).cuda()
    staged = gpu.stage(rows, hist, xt.device)
    staged["hist_raw"] = None
    rc, tok, lp = gpu.step_device(xt, rows, hist, staged=staged)
    torch.cuda.synchronize()
    assert rc == 0
    assert np.isnan(lp.cpu().numpy()).all()
    bits = __import__("ctypes").c_uint32(0)
    assert gpu.lib.sampler_b200_last_device_status(gpu.h, __import__("ctypes").byref(bits)) == 0
    assert bits.value & 4


def test_out_of_range_history_id_is_reported(gpu):
    x = np.zeros((1, 100), np.float32)
    hist = (np.array([0, 1], np.int64), np.array([1337], np.int32), np.array([(1 << 3) | A.HIST_GENERATED], np.uint32))
    rc, *_ = gpu.step_host(x, H.make_rows(1, do_sample=0, repetition_penalty=1.5), hist)
    assert rc == A.SAMPLER_ERR_BAD_TOKEN_ID
    rc, tok, *_ = gpu.step_host(x, H.make_rows(1, do_sample=0))   # the handle is still usable
    assert rc == 0 and tok[0] == 0
