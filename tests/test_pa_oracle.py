"""CPU tests of the PagedAttention oracle: the restatement against an independent second opinion
(torch scaled_dot_product_attention over the gathered dense K/V) and its own invariants.
Parity of this oracle with the reference operator is unpinned (the operator lives in the
un-vendored OpenVINO runtime); these tests pin the oracle to the tensor contract instead."""
import numpy as np
import pytest
import torch

from tests import pa_harness as H
from oracle import pa_oracle


def _second_opinion(wl, data, res):
    q = data[0].float()
    desc = H.desc_of(wl)
    G = wl.num_q_heads // wl.num_kv_heads
    out = torch.zeros_like(q)
    for s in range(wl.num_sequences):
        t0, n, past = int(wl.subsequence_begins[s]), int(wl.new_lens[s]), int(wl.past_lens[s])
        ctx = past + n
        table = wl.block_indices[wl.block_indices_begins[s]:wl.block_indices_begins[s + 1]]
        for hk in range(wl.num_kv_heads):
            k, v = pa_oracle.gather_dense(desc, res["kc_ref"], res["vc_ref"], table, ctx, hk, wl.head_size)
            k, v = torch.from_numpy(k), torch.from_numpy(v)
            qs = q[t0:t0 + n].view(n, wl.num_q_heads, wl.head_size)[:, hk * G:(hk + 1) * G].permute(1, 0, 2)  # [G, n, D]
            mask = torch.ones(n, ctx, dtype=torch.bool).tril(diagonal=past)
            o = torch.nn.functional.scaled_dot_product_attention(qs, k[None], v[None], attn_mask=mask, scale=wl.scale)
            out[t0:t0 + n].view(n, wl.num_q_heads, wl.head_size)[:, hk * G:(hk + 1) * G] = o.permute(1, 0, 2)
    return out.numpy()


@pytest.mark.parametrize("cache,act,tol", [("f16", torch.float16, 2e-3), ("bf16", torch.bfloat16, 8e-3), ("u8", torch.float32, 1e-5)])
def test_oracle_matches_dense_sdpa(cache, act, tol):
    wl = H.small_workload(hq=8, hkv=2, d=64, bs=16, act=act, cache=cache, past=[0, 5, 40, 17], new=[3, 1, 9, 1], seed=3)
    data = H.make_host_data(wl)
    res = H.run_oracle(wl, data)
    ref = _second_opinion(wl, data, res)
    # the output is rounded to the activation dtype; compare at that precision
    assert H.rel_err(res["out_ref"], ref) < tol


def test_u8_quantisation_round_trip():
    wl = H.small_workload(hq=4, hkv=4, d=128, bs=32, act=torch.float32, cache="u8", past=[64], new=[1], seed=11)
    data = H.make_host_data(wl)
    res = H.run_oracle(wl, data)
    desc = H.desc_of(wl)
    table = wl.block_indices[:wl.block_indices_begins[1]]
    pk = data[4].view(64, 4, 128)
    for hk in range(4):
        k, _ = pa_oracle.gather_dense(desc, res["kc_ref"], res["vc_ref"], table, 64, hk, 128)
        x = pk[:, hk].numpy()
        step = (x.max(axis=1) - x.min(axis=1)) / 255.0
        assert np.all(np.abs(k - x) <= 0.5 * step[:, None] * 1.001 + 1e-6)


def test_scores_are_probability_mass():
    """Each window row of each head contributes a distribution that sums to 1."""
    wl = H.small_workload(hq=6, hkv=2, d=64, bs=16, act=torch.float16, cache="f16", past=[20, 0, 7], new=[1, 12, 5], seed=5)
    wl.score_aggregation_window = np.array([1, 4, 9], np.int32)  # last one is clamped to the chunk length
    res = H.run_oracle(wl)
    off = 0
    for s in range(wl.num_sequences):
        ln = int(wl.past_lens[s] + wl.new_lens[s])
        w = min(int(wl.score_aggregation_window[s]), int(wl.new_lens[s]))
        assert abs(res["scores_ref"][off:off + ln].sum() - w * wl.num_q_heads) < 1e-3
        off += ln


def test_zero_window_writes_zeros():
    wl = H.small_workload(hq=2, hkv=1, d=64, bs=16, act=torch.float16, cache="f16", past=[9], new=[4], seed=6)
    wl.score_aggregation_window = np.array([0], np.int32)
    res = H.run_oracle(wl)
    assert np.all(res["scores_ref"] == 0)


def test_rotation_by_row_zero_is_identity_for_f16():
    from openvino_genai_b200 import workloads
    wl = H.small_workload(hq=2, hkv=2, d=64, bs=16, act=torch.float16, cache="f16", past=[48], new=[1], seed=8)
    base = H.run_oracle(wl)
    wl.rotated_block_indices = wl.block_indices[:2].copy()
    wl.rotation_deltas = np.zeros(2, np.int32)
    wl.rotation_trig_lut = workloads.rotation_trig_lut(4, 16, 64, 10000.0)
    rot = H.run_oracle(wl)
    assert np.array_equal(base["kc_ref"], rot["kc_ref"])


def test_rotation_preserves_norm():
    from openvino_genai_b200 import workloads
    wl = H.small_workload(hq=2, hkv=2, d=64, bs=16, act=torch.float32, cache="bf16", past=[32], new=[1], seed=9)
    base = H.run_oracle(wl)
    wl.rotated_block_indices = wl.block_indices[:1].copy()
    wl.rotation_deltas = np.array([3], np.int32)
    wl.rotation_trig_lut = workloads.rotation_trig_lut(4, 16, 64, 10000.0)
    rot = H.run_oracle(wl)
    desc = H.desc_of(wl)
    table = wl.block_indices[:1]
    for hk in range(2):
        k0, _ = pa_oracle.gather_dense(desc, base["kc_ref"], base["vc_ref"], table, 16, hk, 64)
        k1, _ = pa_oracle.gather_dense(desc, rot["kc_ref"], rot["vc_ref"], table, 16, hk, 64)
        assert not np.allclose(k0, k1)
        assert np.allclose(np.linalg.norm(k0, axis=1), np.linalg.norm(k1, axis=1), rtol=1e-2)


def test_bad_block_index_is_reported():
    wl = H.small_workload(hq=2, hkv=1, d=64, bs=16, act=torch.float16, cache="f16", past=[3], new=[1], seed=10)
    wl.block_indices = wl.block_indices.copy()
    wl.block_indices[0] = wl.num_blocks + 5
    desc = H.desc_of(wl)
    q, k, v, *_ = H.make_host_data(wl)
    n = wl.num_blocks * H.block_bytes(wl)
    kc, vc = np.zeros(n, np.uint8), np.zeros(n, np.uint8)
    out = torch.zeros_like(q)
    from openvino_genai_b200 import _abi
    assert pa_oracle.forward(desc, H.host_args(wl, q, k, v, out, kc, vc)) == _abi.PA_ERR_BAD_INDEX
