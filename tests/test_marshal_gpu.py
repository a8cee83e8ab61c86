"""Device-side marshalling of the operator's scheduler inputs (pa_b200_marshal_inputs) against the host rules of
ModelRunner::forward (src/cpp/src/continuous_batching/model_runner.hpp:802-856, 1420-1481): bit-exact
tensors on random schedules with skipped blocks and evicted tokens, and the layouts the reference's own
tests pin (tests/cpp/model_runner.cpp:90-225: flattened per-sequence block ids, their prefix sums, past lengths)."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests import pa_harness as H
from openvino_genai_b200 import _abi

pytestmark = pytest.mark.gpu


def host_rules(tables, processed, evicted, scheduled, skipped, block_size):
    """The host construction, sequence by sequence in scheduled order."""
    past, sub, bi, bib, mcl = [], [0], [], [0], 0
    for s, table in enumerate(tables):
        used = [b for j, b in enumerate(table) if j not in skipped[s]]
        past.append(processed[s] - evicted[s] - len(skipped[s]) * block_size)
        sub.append(sub[-1] + scheduled[s])
        bi.extend(used)
        bib.append(bib[-1] + len(used))
        mcl = max(mcl, processed[s] + scheduled[s])
    return np.array(past, np.int32), np.array(sub, np.int32), np.array(bi, np.int32), np.array(bib, np.int32), mcl


def run_device(op, tables, slots, processed, evicted, scheduled, skipped, stride, num_slots, capacity=None):
    dev = torch.device("cuda", 0)
    B = len(slots)
    table = np.full((num_slots, stride), -1, np.int32)
    lens = np.zeros(num_slots, np.int32)
    for s, sl in enumerate(slots):
        if 0 <= sl < num_slots:   # a test may name a row that does not exist
            table[sl, :len(tables[s])] = tables[s]
            lens[sl] = len(tables[s])
    words = (stride + 31) // 32
    mask = np.zeros((B, words), np.uint32)
    for s in range(B):
        for j in skipped[s]:
            mask[s, j // 32] |= np.uint32(1 << (j % 32))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    d = {"table": t(table), "lens": t(lens), "slot": t(np.array(slots, np.int32)), "proc": t(np.array(processed, np.int32)),
         "evi": t(np.array(evicted, np.int32)), "sched": t(np.array(scheduled, np.int32)), "mask": t(mask.view(np.int32))}
    total_blocks = int(sum(len(x) for x in tables))
    cap = total_blocks if capacity is None else capacity
    out = {"past": torch.full((B,), -9, dtype=torch.int32, device=dev), "sub": torch.full((B + 1,), -9, dtype=torch.int32, device=dev),
           "bi": torch.full((max(cap, 1),), -9, dtype=torch.int32, device=dev), "bib": torch.full((B + 1,), -9, dtype=torch.int32, device=dev),
           "tot": torch.full((3,), -9, dtype=torch.int32, device=dev)}
    a = _abi.pa_marshal_args()
    a.struct_size = C.sizeof(_abi.pa_marshal_args)
    a.block_table, a.block_table_len, a.table_stride, a.num_slots = d["table"].data_ptr(), d["lens"].data_ptr(), stride, num_slots
    a.slot, a.num_processed_tokens, a.num_evicted_tokens = d["slot"].data_ptr(), d["proc"].data_ptr(), d["evi"].data_ptr()
    a.num_scheduled_tokens, a.skip_mask, a.skip_words, a.num_sequences = d["sched"].data_ptr(), d["mask"].data_ptr(), words, B
    a.past_lens, a.subsequence_begins, a.block_indices = out["past"].data_ptr(), out["sub"].data_ptr(), out["bi"].data_ptr()
    a.block_indices_begins, a.totals, a.block_indices_capacity = out["bib"].data_ptr(), out["tot"].data_ptr(), cap
    a.stream = torch.cuda.current_stream(dev).cuda_stream or 1
    op._check(op.lib.pa_b200_marshal_inputs(op._h, C.byref(a)))
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in out.items()}, op.device_status()


@pytest.fixture(scope="module")
def op():
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=16, act=torch.bfloat16, cache="u8", past=[10], new=[1], seed=1)
    return H.make_op(wl)


@pytest.mark.parametrize("B,max_blocks,seed", [(1, 5, 1), (7, 70, 2), (300, 40, 3), (1024, 2100, 4), (1500, 9, 5)])
def test_random_schedules_are_bit_exact(op, B, max_blocks, seed):
    rng = np.random.default_rng(seed)
    bs = 16
    num_slots = B + 13
    slots = rng.permutation(num_slots)[:B].tolist()
    tables, processed, evicted, scheduled, skipped = [], [], [], [], []
    next_id = 0
    for s in range(B):
        nb = int(rng.integers(1, max_blocks + 1))
        tables.append(rng.permutation(10 * max_blocks * 4)[:nb].astype(np.int32) + next_id)
        sk = set(rng.choice(nb, size=int(rng.integers(0, max(1, nb // 4) + 1)), replace=False).tolist()) if s % 3 == 0 and nb > 3 else set()
        skipped.append(sk)
        sched = int(rng.integers(1, bs + 1)) if s % 5 else int(rng.integers(1, min(nb * bs, 300) + 1))
        ev = int(rng.integers(0, 3)) * bs if s % 4 == 1 else 0
        cache_tokens = max(nb * bs - sched, len(sk) * bs)        # what the table can hold before this step
        processed.append(cache_tokens + ev)
        evicted.append(ev)
        scheduled.append(sched)
    want = host_rules(tables, processed, evicted, scheduled, skipped, bs)
    got, status = run_device(op, tables, slots, processed, evicted, scheduled, skipped, stride=max_blocks + 3, num_slots=num_slots)
    assert status == 0
    assert np.array_equal(got["past"], want[0]) and np.array_equal(got["sub"], want[1]) and np.array_equal(got["bib"], want[3])
    n_bi = int(want[3][-1])
    assert np.array_equal(got["bi"][:n_bi], want[2])
    assert (got["bi"][n_bi:] == -9).all(), "stores beyond the used blocks"
    assert got["tot"].tolist() == [int(want[1][-1]), n_bi, want[4]]


def test_layouts_pinned_by_the_reference_tests(op):
    """tests/cpp/model_runner.cpp:90-225: {10,10,11,12} / begins {0,4} / past {0};  {20,20} / {0,2} / {4};
    two sequences {30,30},{40,40} / {0,2,4} / {4,4}."""
    got, st = run_device(op, [[10, 10, 11, 12]], [0], [0], [0], [260], [set()], stride=8, num_slots=2)
    assert st == 0 and got["bi"].tolist() == [10, 10, 11, 12] and got["bib"].tolist() == [0, 4] and got["past"].tolist() == [0]
    got, st = run_device(op, [[20, 20]], [1], [4], [0], [1], [set()], stride=8, num_slots=2)
    assert st == 0 and got["bi"].tolist() == [20, 20] and got["bib"].tolist() == [0, 2] and got["past"].tolist() == [4]
    got, st = run_device(op, [[30, 30], [40, 40]], [0, 1], [4, 4], [0, 0], [1, 1], [set(), set()], stride=8, num_slots=2)
    assert st == 0 and got["bi"].tolist() == [30, 30, 40, 40] and got["bib"].tolist() == [0, 2, 4] and got["past"].tolist() == [4, 4]
    assert got["sub"].tolist() == [0, 1, 2] and got["tot"].tolist() == [2, 4, 5]


def test_numbers_that_do_not_hold_together_are_flagged(op):
    tables = [[1, 2, 3], [4, 5], [6, 7, 8, 9]]
    ok = dict(slots=[0, 1, 2], processed=[40, 20, 50], evicted=[0, 0, 0], scheduled=[1, 1, 1], skipped=[set(), set(), set()])
    bad = [dict(ok, evicted=[0, 30, 0]),                       # more evicted than processed
           dict(ok, skipped=[set(), {0, 1}, set()], processed=[40, 20, 50]),   # skipped blocks exceed the occupancy (2 * 16 > 20)
           dict(ok, slots=[0, 7, 2]),                          # no such table row
           dict(ok, scheduled=[1, -1, 1])]
    for case in bad:
        got, st = run_device(op, tables, case["slots"], case["processed"], case["evicted"], case["scheduled"], case["skipped"], stride=6, num_slots=4)
        assert st & _abi.PA_DEV_BAD_BEGINS
        assert got["bib"].tolist() == [0, 3, 3, 7] and got["sub"].tolist() == [0, 1, 1, 2], "the flagged sequence gets no tokens and no blocks"
    got, st = run_device(op, tables, **ok, stride=6, num_slots=4, capacity=5)   # output too small for the ids
    assert st & _abi.PA_DEV_BAD_BEGINS and (got["bi"][:5] >= 1).all()
    got, st = run_device(op, tables, **ok, stride=6, num_slots=4)
    assert st == 0
