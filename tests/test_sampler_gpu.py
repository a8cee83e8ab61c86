"""Parity of the CUDA Sampler step (through the C ABI) with the CPU oracle.

Token ids must be identical for greedy rows and for multinomial rows on the top-k path (the heap
order, every float sum and the draw are reproduced step for step); penalised logits must be
bit-identical.  The full-vocabulary multinomial path reproduces the host's expf and its sequential
float sums, so its token ids are identical too, except where the draw falls into a run of exactly
equal probabilities (counted and bounded)."""
import numpy as np
import pytest
import torch

import ctypes as C

from tests import sampler_harness as H
from openvino_genai_b200 import _sampler_abi as A
from oracle import sampler_oracle

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


def _assert_same_tokens_up_to_equal_probabilities(tok_o, tok_g, lg_o, rows, max_excluded):
    """Token ids must be identical.  The one exception the reference itself leaves open: several kept
    elements with exactly the same probability, and the draw falls among them (their order after
    std::sort / std::partial_sort is unspecified).  Such rows are counted, reported and bounded."""
    diff = np.flatnonzero(tok_o != tok_g)
    excluded = 0
    for r in diff:
        p, _, _ = sampler_oracle.transform(0, lg_o[rows["logits_row"][r]], float(rows["temperature"][r]))
        assert tok_g[r] >= 0 and p[tok_g[r]] == p[tok_o[r]], f"row {r}: token {tok_g[r]} (p {p[tok_g[r]]}) vs oracle {tok_o[r]} (p {p[tok_o[r]]})"
        excluded += 1
    print(f"{len(tok_o)} rows, {excluded} differ only inside a run of equal probabilities")
    assert excluded <= max_excluded
    return excluded


def test_device_expf_has_the_host_libm_bits(gpu):
    """The full-vocabulary path is exact only if every exponential has the host's bits."""
    rng = np.random.default_rng(5)
    x = np.concatenate([
        -np.abs(rng.standard_normal(1 << 20) * 8).astype(np.float32),
        rng.uniform(-104.5, 0.0, 1 << 20).astype(np.float32),
        np.arange(0x80000000, 0xC2D00000, 4099, dtype=np.uint64).astype(np.uint32).view(np.float32),   # a stride through -0 .. -104
        np.array([-0.0, 0.0, -np.inf, -200.0, -103.98, -103.97, -103.9, -87.4, -1e-30, -1e-45], np.float32),
    ])
    got = np.empty_like(x)
    assert gpu.lib.sampler_b200_selftest_expf(gpu.h, x.ctypes.data, got.ctypes.data, len(x)) == 0
    want = np.empty_like(x)
    lib = C.CDLL("libm.so.6")
    lib.expf.restype = C.c_float
    lib.expf.argtypes = [C.c_float]
    # numpy's exp is not the libm routine: call libm itself on a sample, and the oracle's softmax on all
    idx = rng.choice(len(x), size=20000, replace=False)
    for i in idx:
        want[i] = lib.expf(float(x[i]))
    assert np.array_equal(got[idx].view(np.uint32), want[idx].view(np.uint32))
    # all of them through the oracle: softmax numerators of a row whose maximum is 0
    row = np.concatenate([[np.float32(0.0)], x[np.isfinite(x)]]).astype(np.float32)
    p, _, _ = sampler_oracle.transform(0, row, 1.0)
    got_row = np.empty_like(row)
    assert gpu.lib.sampler_b200_selftest_expf(gpu.h, row.ctypes.data, got_row.ctypes.data, len(row)) == 0
    s = np.float32(0)
    for v in got_row:   # the oracle's own index-order sum
        s = np.float32(s + v)
    assert np.array_equal((got_row / s).astype(np.float32).view(np.uint32), p.view(np.uint32))


@pytest.mark.parametrize("n,v,seed", [(256, 128256, 21), (256, 151936, 23)])
def test_full_vocab_top_p_tokens_are_identical(gpu, n, v, seed):
    """T = 1, top_p = 0.95, no top-k over N(0, 4) logits (the sampler of the sharded engine step):
    46 k elements are kept per row, the reference sorts all of them and adds them one by one."""
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((n, v)) * 2).astype(np.float32)
    rows = H.make_rows(n, top_p=0.95, seeds=np.arange(n) + 1000)
    tok_o, lp_o, lg_o, tok_g, lp_g, lg_g = _both(gpu, x, rows)
    _assert_same_tokens_up_to_equal_probabilities(tok_o, tok_g, lg_o, rows, max_excluded=2)
    same = tok_o == tok_g
    assert np.allclose(lp_o[same], lp_g[same], atol=2e-6, rtol=1e-6)
    assert np.array_equal(lg_o.view(np.uint32), lg_g.view(np.uint32))


@pytest.mark.parametrize("n,v,T,seed", [(256, 151936, 0.7, 22), (256, 128256, 1.0, 24), (64, 32000, 1.3, 25)])
def test_full_vocab_plain_sampling_tokens_are_identical(gpu, n, v, T, seed):
    """Temperature only: softmax over the whole row, the draw walks the probabilities in index order."""
    rng = np.random.default_rng(seed)
    x = H.synthetic_logits(rng, n, v)
    rows = H.make_rows(n, temperature=T, seeds=np.arange(n) + 2000)
    tok_o, lp_o, lg_o, tok_g, lp_g, _ = _both(gpu, x, rows)
    assert np.array_equal(tok_o, tok_g), f"{(tok_o != tok_g).sum()} of {n} tokens differ"
    assert np.allclose(lp_o, lp_g, atol=2e-6, rtol=1e-6)


@pytest.mark.parametrize("case", ["min_p", "min_p_top_p", "penalties_top_p", "bf16_logits", "all_equal", "odd_vocab", "peaked", "flat",
                                  "top_p_tiny", "top_p_almost_one", "masked", "k_above_vocab", "big_equal_runs"])
def test_full_vocab_cases_are_identical(gpu, case):
    rng = np.random.default_rng(sum(map(ord, case)))
    n, v = 24, 50000
    kw = dict(top_p=0.9, temperature=0.9)
    hist = None
    x = (rng.standard_normal((n, v)) * 2).astype(np.float32)
    if case == "min_p":
        kw = dict(min_p=0.02, temperature=1.1)
    elif case == "min_p_top_p":
        kw = dict(min_p=0.001, top_p=0.8)
    elif case == "penalties_top_p":
        hist = H.make_history(rng, n, v, generated_len=500, prompt_len=100)
        kw.update(repetition_penalty=1.2, presence_penalty=0.3, frequency_penalty=0.1)
    elif case == "bf16_logits":   # what a bf16 LM head produces: a few thousand distinct values, long runs of equal probabilities
        x = (x.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
    elif case == "all_equal":
        n = 4
        x = np.full((n, 128256), 1.5, np.float32)
    elif case == "odd_vocab":
        x = np.ascontiguousarray(x[:, :49999])
    elif case == "peaked":
        x *= 4
    elif case == "flat":
        x *= 0.1
    elif case == "top_p_tiny":
        kw = dict(top_p=0.01)
    elif case == "top_p_almost_one":
        kw = dict(top_p=0.9999999)
    elif case == "masked":
        x[:, ::3] = -np.inf
    elif case == "k_above_vocab":
        kw = dict(top_k=60000, top_p=0.9, temperature=0.8)
    elif case == "big_equal_runs":   # quarter-integer logits over a Llama-sized row: single probabilities held by > 4096 elements
        x = (np.round(rng.standard_normal((6, 128256)) * 4) / 4).astype(np.float32); n = 6
        kw = dict(top_p=0.95)
    rows = H.make_rows(n, seeds=np.arange(n) + 500, **kw)
    rows["rand_u"] = rng.random(n, dtype=np.float32)
    tok_o, lp_o, lg_o, tok_g, lp_g, lg_g = _both(gpu, x, rows, hist)
    _assert_same_tokens_up_to_equal_probabilities(tok_o, tok_g, lg_o, rows, max_excluded=n if case in ("bf16_logits", "all_equal", "big_equal_runs") else 1)
    same = tok_o == tok_g
    assert np.allclose(lp_o[same], lp_g[same], atol=2e-6, rtol=1e-6)
    assert np.array_equal(lg_o.view(np.uint32), lg_g.view(np.uint32))


def test_top_k_above_the_heap_capacity_is_refused_loudly(gpu):
    rng = np.random.default_rng(61)
    x = H.synthetic_logits(rng, 2, 32000)
    rows = H.make_rows(2, top_k=2000, temperature=0.8)
    rc, tok, lp, _ = gpu.step_host(x, rows)
    assert rc == A.SAMPLER_ERR_UNSUPPORTED and list(tok) == [-1, -1]
    rc, tok, *_ = gpu.step_host(x, H.make_rows(2, top_k=1024, temperature=0.8))   # the handle is still usable, 1024 is supported
    assert rc == 0 and (tok >= 0).all()


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


@pytest.mark.parametrize("mode", ["top_k", "top_k_deferred", "top_p_full", "plain_full"])
def test_several_draws_from_one_distribution(gpu, mode):
    """num_return_sequences = n: the first sampled token's distribution is drawn from n times with
    consecutive numbers of the request's engine; every draw must equal the oracle's."""
    rng = np.random.default_rng(71)
    n, vocab = 6, 40000
    x = (rng.standard_normal((n, vocab)) * 2).astype(np.float32)   # no spikes: several tokens share the mass
    kw = {"top_k": dict(top_k=40, temperature=0.8, top_p=0.9), "top_k_deferred": dict(top_k=40, temperature=0.8),
          "top_p_full": dict(top_p=0.9, temperature=1.1), "plain_full": dict(temperature=0.9)}[mode]
    rows = H.make_rows(n, seeds=np.arange(n) + 900, **kw)
    counts = np.array([3, 0, 1, 7, 0, 2])
    offs = np.zeros(n + 1, np.int64)
    offs[1:] = np.cumsum(counts)
    us = rng.random(int(offs[-1]), dtype=np.float32)

    def run(step):
        lg = x.copy()
        tok = np.full(n, -7, np.int64); lp = np.zeros(n, np.float32)
        xtok = np.full(len(us), -7, np.int64); xlp = np.zeros(len(us), np.float32)
        a = H.step_args(lg, rows, None, tok, lp)
        a.extra_offsets, a.extra_rand_u = offs.ctypes.data, us.ctypes.data
        a.extra_out_token, a.extra_out_log_prob = xtok.ctypes.data, xlp.ctypes.data
        assert step(a) == 0
        return tok, lp, xtok, xlp

    tok_o, lp_o, xtok_o, xlp_o = run(lambda a: sampler_oracle.step(a, 0))
    tok_g, lp_g, xtok_g, xlp_g = run(lambda a: gpu.lib.sampler_b200_step_host(gpu.h, C.byref(a), 1))
    assert np.array_equal(tok_o, tok_g) and np.array_equal(xtok_o, xtok_g), (xtok_o, xtok_g)
    assert np.allclose(lp_o, lp_g, atol=2e-6, rtol=1e-6) and np.allclose(xlp_o, xlp_g, atol=2e-6, rtol=1e-6)
    # the first draw does not depend on the further ones
    tok_1 = _both(gpu, x, rows)[3]
    assert np.array_equal(tok_1, tok_g)
    assert len(set(xtok_g[offs[3]:offs[4]].tolist())) > 1, "seven draws of one row are not all the same token"


def test_step_args_without_the_extra_draw_members_are_still_accepted(gpu):
    rng = np.random.default_rng(72)
    x = H.synthetic_logits(rng, 3, 5000)
    rows = H.make_rows(3, top_k=20, temperature=0.8)
    lg = x.copy()
    tok = np.full(3, -7, np.int64); lp = np.zeros(3, np.float32)
    a = H.step_args(lg, rows, None, tok, lp)
    a.struct_size = A.sampler_step_args.extra_offsets.offset     # the layout that ends at hist_raw
    a.extra_offsets = 0xdead0000                                   # must not be read
    assert gpu.lib.sampler_b200_step_host(gpu.h, C.byref(a), 0) == 0
    assert np.array_equal(tok, _both(gpu, x, rows)[3])


@pytest.mark.parametrize("mode", ["greedy", "top_k", "top_p_full"])
def test_grammar_bitmask_is_applied_before_the_penalties(gpu, mode):
    """A request's next-token bitmask: disallowed logits become -inf, the logits left behind and the tokens
    equal the oracle's; rows without a mask (index -1) are untouched by it."""
    rng = np.random.default_rng(81)
    n, vocab = 8, 40003    # the last mask word is partial
    x = H.synthetic_logits(rng, n, vocab)
    hist = H.make_history(rng, n, vocab, generated_len=200, prompt_len=40)
    kw = {"greedy": dict(do_sample=0), "top_k": dict(top_k=30, temperature=0.9, top_p=0.95), "top_p_full": dict(top_p=0.9)}[mode]
    rows = H.make_rows(n, repetition_penalty=1.2, presence_penalty=0.1, seeds=np.arange(n) + 300, **kw)
    words = (vocab + 31) // 32
    masks = rng.integers(0, 2 ** 32, size=(3, words), dtype=np.uint64).astype(np.uint32).view(np.int32)
    masks[1] = 0
    masks[1, 7] = 1 << 5            # a single allowed token: 7 * 32 + 5
    masks[2] &= rng.integers(0, 2 ** 32, size=words, dtype=np.uint64).astype(np.uint32).view(np.int32)
    index = np.array([0, 1, -1, 2, 0, -1, 1, 2], np.int32)

    def run(step):
        lg = x.copy()
        tok = np.full(n, -7, np.int64); lp = np.zeros(n, np.float32)
        a = H.step_args(lg, rows, hist, tok, lp)
        a.token_bitmasks, a.bitmask_index, a.bitmask_words = masks.ctypes.data, index.ctypes.data, words
        assert step(a) == 0
        return tok, lp, lg

    tok_o, lp_o, lg_o = run(lambda a: sampler_oracle.step(a, 0))
    tok_g, lp_g, lg_g = run(lambda a: gpu.lib.sampler_b200_step_host(gpu.h, C.byref(a), 1))
    assert np.array_equal(tok_o, tok_g), (tok_o, tok_g)
    assert np.array_equal(lg_o.view(np.uint32), lg_g.view(np.uint32))
    assert tok_g[1] == 7 * 32 + 5 and tok_g[6] == 7 * 32 + 5
    for r in range(n):
        if index[r] >= 0:
            t = int(tok_g[r])
            assert (masks[index[r]].view(np.uint32)[t // 32] >> (t % 32)) & 1, f"row {r} picked a token its grammar does not allow"
    assert np.isinf(lg_g[0]).sum() > vocab // 3 and np.isinf(lg_g[2]).sum() == 0
