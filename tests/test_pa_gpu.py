"""Parity of the CUDA PagedAttention path (through the C ABI) with the CPU oracle.

Tolerances are the ones the operator is specified to: attention output within 2e-3 relative for
f16/bf16 caches and 1e-2 for the u8 cache (relative to the largest reference magnitude);
cache bytes written by the kernels must equal the oracle's bit for bit."""
import numpy as np
import pytest
import torch

from tests import pa_harness as H

pytestmark = pytest.mark.gpu

TOL = {"f16": 2e-3, "bf16": 2e-3, "u8": 1e-2}


def _check(res, cache, act=None):
    assert res["status"] == 0, f"device status {res['status']:#x}"
    assert np.array_equal(res["kc_gpu"], res["kc_ref"]), "key cache bytes differ from the oracle"
    assert np.array_equal(res["vc_gpu"], res["vc_ref"]), "value cache bytes differ from the oracle"
    tol = TOL[cache]
    if act == torch.bfloat16:
        tol = max(tol, 8e-3)  # the output itself is rounded to bf16 (8 significant bits)
    err = H.rel_err(res["out_gpu"], res["out_ref"])
    assert err < tol, f"attention output rel err {err:.3e} >= {tol}"


@pytest.mark.parametrize("cache", ["f16", "bf16", "u8"])
@pytest.mark.parametrize("d,bs", [(64, 32), (128, 32), (128, 16), (64, 16)])
def test_decode_parity(cache, d, bs):
    act = torch.float16 if cache == "f16" else torch.bfloat16
    wl = H.small_workload(hq=8, hkv=2, d=d, bs=bs, act=act, cache=cache, past=[0, 1, 31, 32, 33, 100, 517, 1500],
                          new=[1] * 8, seed=20 + d + bs)
    _check(H.run_both(wl), cache, act)


@pytest.mark.parametrize("hq,hkv", [(4, 4), (28, 4), (32, 4), (16, 1), (40, 2)])
def test_decode_group_sizes(hq, hkv):
    wl = H.small_workload(hq=hq, hkv=hkv, d=128, bs=32, act=torch.float16, cache="u8", past=[77, 300, 1024], new=[1, 1, 1], seed=hq)
    _check(H.run_both(wl), "u8")


def test_decode_config1_tinyllama_shape():
    from openvino_genai_b200 import workloads
    wl = workloads.config_tinyllama_decode()
    _check(H.run_both(wl), "f16")


def test_decode_long_context_many_splits(monkeypatch):
    monkeypatch.setenv("PA_B200_UNUSED", "1")
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=torch.bfloat16, cache="u8", past=[5000, 255, 256, 257], new=[1] * 4, seed=31)
    _check(H.run_both(wl), "u8", torch.bfloat16)


def test_decode_u8_keeps_its_precision_over_a_32k_context():
    """With N(0,1) values the output shrinks like 1/sqrt(context) while the u8 accumulators carry
    1024 + byte per unit of probability: the error must stay at the level of the f16 cache's, far
    inside the 1e-2 bound, and must not grow with the number of accumulated tiles."""
    wl = H.small_workload(hq=16, hkv=2, d=128, bs=16, act=torch.float32, cache="u8", past=[32494, 9000], new=[1, 1], seed=35)
    res = H.run_both(wl)
    _check(res, "u8")
    for s in range(2):
        err = H.rel_err(res["out_gpu"][s], res["out_ref"][s])
        assert err < 2e-3, f"sequence {s}: rel err {err:.3e}"


def test_decode_f32_activations():
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=torch.float32, cache="u8", past=[200, 64], new=[1, 1], seed=33)
    _check(H.run_both(wl), "u8")


@pytest.mark.parametrize("cache", ["f16", "bf16", "u8"])
@pytest.mark.parametrize("d,bs", [(128, 32), (64, 32), (64, 16)])
def test_prefill_and_mixed_parity(cache, d, bs):
    act = torch.float16 if cache == "f16" else torch.bfloat16
    wl = H.small_workload(hq=8, hkv=2, d=d, bs=bs, act=act, cache=cache, past=[0, 40, 300, 0, 65], new=[37, 1, 64, 1, 130], seed=41)
    res = H.run_both(wl)
    _check(res, cache, act)
    assert res["prefill_kernel"] == "tcgen05"   # every cache type, both head sizes


@pytest.mark.parametrize("hq,hkv,bs,past,new", [
    (28, 4, 32, [0, 700, 63, 4000], [256, 256, 130, 64]),     # Qwen2.5-7B group of 7: q tiles straddle tokens
    (32, 8, 16, [1000, 5], [200, 33]),                        # block size 16
    (8, 8, 32, [300], [129]),                                 # no grouping: one head per q-tile row
    (64, 8, 32, [0, 90], [40, 17]),                           # group of 8
])
def test_prefill_tensor_core_shapes(hq, hkv, bs, past, new):
    """u8 cache, head size 128: the tcgen05 / TMEM chunk kernel."""
    wl = H.small_workload(hq=hq, hkv=hkv, d=128, bs=bs, act=torch.bfloat16, cache="u8", past=past, new=new, seed=hq + bs)
    _check(H.run_both(wl), "u8", torch.bfloat16)


@pytest.mark.parametrize("cache,d,bs,hq,hkv,act", [
    ("u8", 128, 32, 28, 4, torch.float16), ("f16", 128, 32, 28, 4, torch.float16), ("f16", 128, 16, 32, 8, torch.float16),
    ("f16", 64, 16, 12, 4, torch.float16), ("f16", 64, 32, 32, 4, torch.float32), ("u8", 64, 32, 32, 4, torch.bfloat16), ("u8", 64, 16, 12, 4, torch.float16),
    ("bf16", 128, 32, 28, 4, torch.bfloat16), ("bf16", 128, 16, 8, 2, torch.bfloat16), ("bf16", 64, 32, 40, 2, torch.bfloat16), ("bf16", 64, 16, 8, 8, torch.bfloat16),
    ("bf16", 128, 16, 8, 2, torch.float16), ("bf16", 64, 32, 40, 2, torch.float32)])
def test_prefill_tensor_core_matches_generic_kernel(monkeypatch, cache, d, bs, hq, hkv, act):
    """The tensor-core chunk kernels (tcgen05 for the u8 and f16 caches and for the bf16 cache under bf16 activations, mma.sync for
    the bf16 cache under other activations) against the CUDA-core one."""
    wl = H.small_workload(hq=hq, hkv=hkv, d=d, bs=bs, act=act, cache=cache, past=[500, 0, 33], new=[256, 100, 2], seed=71)
    data = H.make_host_data(wl)
    tc = H.run_gpu(wl, data)
    monkeypatch.setenv("PA_B200_GENERIC_PREFILL", "1")
    gen = H.run_gpu(wl, data)
    assert tc["status"] == 0 and gen["status"] == 0
    assert gen["prefill_kernel"] == "generic"
    assert tc["prefill_kernel"] == ("mma_sync" if cache == "bf16" and act != torch.bfloat16 else "tcgen05")
    # both kernels round their output to the activation type: bf16 outputs differ by an ulp where the f32 values straddle a tie
    assert H.rel_err(tc["out_gpu"], gen["out_gpu"]) < (8e-3 if act == torch.bfloat16 else 2e-3)


@pytest.mark.parametrize("seed", range(12))
def test_random_mixed_steps_against_the_oracle(seed):
    """Seeded random geometry (cache type, head size, block size, GQA group) and ragged sequences (past 0 ... 1500, 1 ... 300 new
    tokens, decode rows mixed in): every kernel choice the dispatcher makes is compared with the oracle."""
    rng = np.random.default_rng(1000 + seed)
    cache = ["u8", "f16", "bf16"][seed % 3]
    d = int(rng.choice([64, 128]))
    bs = int(rng.choice([16, 32]))
    hkv = int(rng.choice([1, 2, 4]))
    g = int(rng.choice([1, 2, 3, 4, 7, 8]))
    act = {"u8": [torch.float16, torch.bfloat16, torch.float32], "f16": [torch.float16, torch.float32], "bf16": [torch.bfloat16, torch.float16]}[cache][seed // 3 % 2]
    nseq = int(rng.integers(2, 7))
    past = [int(x) for x in rng.integers(0, 1500, nseq)]
    new = [int(x) if rng.random() < 0.7 else 1 for x in rng.integers(1, 300, nseq)]
    past[0] = 0                                   # a first chunk without context
    wl = H.small_workload(hq=hkv * g, hkv=hkv, d=d, bs=bs, act=act, cache=cache, past=past, new=new, seed=500 + seed)
    res = H.run_both(wl)
    assert res["status"] == 0
    assert np.array_equal(res["kc_gpu"], res["kc_ref"]) and np.array_equal(res["vc_gpu"], res["vc_ref"])
    tol = 1e-2 if cache == "u8" else 2e-3
    if act == torch.bfloat16:
        tol = max(tol, 8e-3)                      # one bf16 ulp of the largest output
    elif act == torch.float16:
        tol = max(tol, 2.5e-3)
    assert H.rel_err(res["out_gpu"], res["out_ref"]) < tol, (cache, d, bs, hkv, g, act, past, new)


def test_host_entry_point_matches():
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=torch.bfloat16, cache="u8", past=[0, 40, 300], new=[20, 1, 1], seed=43)
    _check(H.run_both(wl, host_entry=True), "u8", torch.bfloat16)


@pytest.mark.parametrize("cache", ["f16", "u8"])
def test_scores_parity(cache):
    act = torch.float16
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=act, cache=cache, past=[0, 40, 300, 90], new=[37, 1, 1, 16], seed=47)
    wl.score_aggregation_window = np.array([8, 1, 0, 40], np.int32)
    res = H.run_both(wl)
    _check(res, cache, act)
    ref, got = res["scores_ref"], res["scores_gpu"]
    assert not np.isnan(got).any()
    assert np.abs(got - ref).max() <= 2e-3 * max(1.0, np.abs(ref).max())
    off = int(wl.past_lens[0] + wl.new_lens[0] + wl.past_lens[1] + wl.new_lens[1])
    assert np.all(got[off:off + 301] == 0), "window 0 must write zeros"


def test_scores_qwen_shape_windows_and_block16():
    """Group of 7 heads, window larger than 16 rows / G (several row tiles), block size 16."""
    wl = H.small_workload(hq=28, hkv=4, d=128, bs=16, act=torch.bfloat16, cache="u8", past=[0, 700, 64, 2000, 31],
                          new=[256, 1, 40, 1, 3], seed=91)
    wl.score_aggregation_window = np.array([8, 1, 16, 1, 5], np.int32)
    res = H.run_both(wl)
    _check(res, "u8", torch.bfloat16)
    ref, got = res["scores_ref"], res["scores_gpu"]
    assert not np.isnan(got).any()
    assert np.abs(got - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max())
    assert abs(got.sum() - ref.sum()) <= 1e-2 * ref.sum()


@pytest.mark.parametrize("hq,hkv,cache", [(32, 2, "u8"), (40, 2, "u8"), (24, 2, "f16"), (8, 8, "u8")])
def test_scores_of_decode_rows_come_from_the_decode_kernel(hq, hkv, cache):
    """Rows with one new token take their scores from the logits the decode kernel leaves behind:
    GQA groups above 8 and above 16 heads (two head tiles), a group of one, a context long enough
    to be split over many workers, a window of 0 among them."""
    wl = H.small_workload(hq=hq, hkv=hkv, d=128, bs=32, act=torch.float16, cache=cache, past=[6000, 33, 0, 250, 1023],
                          new=[1, 1, 1, 1, 1], seed=hq + hkv)
    wl.score_aggregation_window = np.array([1, 1, 1, 0, 1], np.int32)
    res = H.run_both(wl)
    _check(res, cache, torch.float16)
    ref, got = res["scores_ref"], res["scores_gpu"]
    assert not np.isnan(got).any()
    assert np.abs(got - ref).max() <= 2e-3 * max(1.0, np.abs(ref).max())
    off = 6001 + 34 + 1
    assert np.all(got[off:off + 251] == 0), "window 0 must write zeros"
    # every sequence's scores add up to the number of q heads (one softmax row per head)
    assert abs(got[:6001].sum() - hq) < 1e-2 * hq


@pytest.mark.parametrize("cache", ["f16", "bf16", "u8"])
def test_rotation_is_bit_exact(cache):
    from openvino_genai_b200 import workloads
    act = torch.float16 if cache == "f16" else torch.bfloat16
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=act, cache=cache, past=[200, 96], new=[1, 1], seed=53)
    wl.rotated_block_indices = np.concatenate([wl.block_indices[1:4], wl.block_indices[8:9]]).astype(np.int32)
    wl.rotation_deltas = np.array([1, 7, 2, 5], np.int32)
    wl.rotation_trig_lut = workloads.rotation_trig_lut(9, 32, 128, 1e6)
    _check(H.run_both(wl), cache, act)


def test_bad_block_index_sets_status_and_does_not_fault():
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=torch.bfloat16, cache="u8", past=[100, 50], new=[1, 1], seed=59)
    data = H.make_host_data(wl)
    good = wl.block_indices.copy()
    op = H.make_op(wl)
    res = H.run_gpu(wl, data, op=op)
    assert res["status"] == 0
    wl.block_indices = good.copy()
    wl.block_indices[1] = wl.num_blocks + 7
    res = H.run_gpu(wl, data, op=op)
    from openvino_genai_b200 import _abi
    assert res["status"] & _abi.PA_DEV_BAD_BLOCK_INDEX
    wl.block_indices = good
    assert H.run_gpu(wl, data, op=op)["status"] == 0  # the context is still usable


def test_unsupported_inputs_are_rejected(pkg):
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=torch.bfloat16, cache="u8", past=[10], new=[1], seed=61)
    op = H.make_op(wl)
    dev = torch.device("cuda", 0)
    q, k, v = (x.to(dev) for x in H.workloads.random_activations(wl))
    kc, vc = op.allocate_cache(wl.num_blocks)
    t = lambda a: torch.from_numpy(a).to(dev)
    common = dict(query=q, key=k, value=v, key_cache=kc, value_cache=vc, past_lens=t(wl.past_lens),
                  subsequence_begins=t(wl.subsequence_begins), block_indices=t(wl.block_indices),
                  block_indices_begins=t(wl.block_indices_begins), max_context_len=wl.max_context_len)
    with pytest.raises(pkg.GenaiB200Error):
        op.evaluate(dict(common, sliding_window=128), {"output": torch.empty_like(q)})
    with pytest.raises(pkg.GenaiB200Error):
        op.evaluate(dict(common, alibi_slopes=torch.zeros(8, device=dev)), {"output": torch.empty_like(q)})


def test_copy_blocks():
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=torch.bfloat16, cache="u8", past=[100], new=[1], seed=67, pool=12)
    res = H.run_both(wl)
    op = res["op"]
    dev = torch.device("cuda", 0)
    kc = torch.from_numpy(res["kc_gpu"]).to(dev)
    vc = torch.from_numpy(res["vc_gpu"]).to(dev)
    src = int(wl.block_indices[0])
    free = [b for b in range(wl.num_blocks) if b not in set(wl.block_indices.tolist())][:2]
    pairs = torch.tensor([[src, free[0]], [src, free[1]]], dtype=torch.int32, device=dev)
    op.copy_blocks(kc, vc, pairs)
    torch.cuda.synchronize()
    bb = H.block_bytes(wl)
    k = kc.cpu().numpy()
    for f in free:
        assert np.array_equal(k[f * bb:(f + 1) * bb], k[src * bb:(src + 1) * bb])


@pytest.mark.parametrize("cache,bs", [("u8", 32), ("u8", 16), ("f16", 32)])
def test_contexts_on_block_and_tile_boundaries(cache, bs):
    """Decode rows whose context ends exactly on, one before and one after a block / tile boundary
    (the first token of a sequence included), and chunks that start or end on one."""
    act = torch.float16 if cache == "f16" else torch.bfloat16
    past = [0, 15, 16, 31, 32, 63, 64, 127, 128, 255, 0, 0, 63, 64, 33]
    new = [1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 2, 128, 65, 64, 31]
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=bs, act=act, cache=cache, past=past, new=new, seed=97)
    _check(H.run_both(wl), cache, act)


def test_score_window_longer_than_the_chunk_is_clamped():
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=torch.bfloat16, cache="u8", past=[100, 0, 40], new=[1, 5, 3], seed=101)
    wl.score_aggregation_window = np.array([7, 64, 3], np.int32)   # 7 > 1 and 64 > 5: clamped to the chunk
    res = H.run_both(wl)
    _check(res, "u8", torch.bfloat16)
    ref, got = res["scores_ref"], res["scores_gpu"]
    assert np.abs(got - ref).max() <= 1e-2 * max(1.0, np.abs(ref).max())
    # one decode row with 8 q heads: its scores are one probability distribution per head
    assert abs(got[:101].sum() - 8.0) < 1e-2


def test_empty_step_is_a_no_op():
    import ctypes as C
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=torch.bfloat16, cache="u8", past=[10], new=[1], seed=3)
    op = H.make_op(wl)
    kc, vc = op.allocate_cache(wl.num_blocks, fill=0)
    dev = kc.device
    z = torch.zeros((0, 8 * 128), dtype=torch.bfloat16, device=dev)
    zk = torch.zeros((0, 2 * 128), dtype=torch.bfloat16, device=dev)
    zi = torch.zeros(1, dtype=torch.int32, device=dev)
    before = op.launch_count()
    args = op.make_args(z, zk, zk, z, kc, vc, zi[:0], zi, zi[:0], zi, wl.scale, 0)
    assert op.lib.pa_b200_forward(op._h, C.byref(args)) == 0
    assert op.launch_count() == before and op.device_status() == 0


def test_a_copy_that_never_arrives_ends_with_a_status_bit_not_a_hang(monkeypatch):
    """Every wait of the decode kernel on a staged record is bounded.  The test hook makes worker 0 arm the
    barrier of its first tile without issuing the copy (nothing is in flight) and poll 2^10 times only: the
    step must return with PA_DEV_WAIT_TIMEOUT_DECODE set, and the next step on the same context must be clean."""
    from openvino_genai_b200 import _abi
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=torch.bfloat16, cache="u8", past=[900, 300, 64], new=[1, 1, 1], seed=113)
    data = H.make_host_data(wl)
    good = H.run_gpu(wl, data)
    assert good["status"] == 0
    monkeypatch.setenv("PA_B200_TEST_DROP_FIRST_COPY", "1")
    hooked = H.run_gpu(wl, data)            # a new handle reads the hook
    assert hooked["status"] & _abi.PA_DEV_WAIT_TIMEOUT_DECODE
    monkeypatch.delenv("PA_B200_TEST_DROP_FIRST_COPY")
    again = H.run_gpu(wl, data)
    assert again["status"] == 0 and np.allclose(again["out_gpu"], good["out_gpu"], rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("act,cache", [(torch.float32, "u8"), (torch.bfloat16, "u8"), (torch.float32, "f16"), (torch.bfloat16, "f16"), (torch.bfloat16, "bf16")])
def test_queries_beyond_the_f16_range(act, cache):
    """|q| around 1e5 (with a softmax scale that brings the logits back to order one): prefill chunks and decode
    rows rescale such rows by an exact power of two before packing them for the tensor cores."""
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=act, cache=cache, past=[300, 40, 0], new=[64, 1, 33], seed=127, scale=1.0 / (1.0e5 * 128 ** 0.5))
    q, k, v, fill, pk, pv = H.make_host_data(wl)
    data = ((q.float() * 1.0e5).to(act), k, v, fill, pk, pv)
    res = H.run_oracle(wl, data)
    res.update(H.run_gpu(wl, data))
    assert res["status"] == 0
    assert np.isfinite(res["out_gpu"]).all()
    assert H.rel_err(res["out_gpu"], res["out_ref"]) < (1e-2 if act == torch.float32 else 1.2e-2)
