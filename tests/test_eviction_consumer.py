"""The consumers of the operator's outputs, run from the reference's own sources: the eviction
algorithm that reads the score vector, the SnapKV window rule that produces
score_aggregation_window, and the rotation LUT the operator is handed.  The reference's
cache_eviction.cpp / kvcrush.cpp are compiled unmodified into oracle/_ref/libref_eviction.so."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import ref_eviction  # noqa: E402

pytestmark = pytest.mark.skipif(ref_eviction.lib() is None, reason="oracle/_ref/libref_eviction.so was not built")


def test_rotation_lut_equals_reference_calculator():
    from tests import pa_harness as H
    for bs, rows, head, theta in ((32, 65, 128, 1e4), (32, 513, 128, 1e6), (16, 33, 64, 1e4), (2, 8, 4, 2.0)):
        ref = ref_eviction.rotation_lut(bs, rows, head, theta)
        ours = H.workloads.rotation_trig_lut(rows, bs, head, theta)
        assert np.array_equal(ref, ours), (bs, rows, head, theta)
    # tests/cpp/cache_eviction.cpp:1421-1437: block size 2, head 4, theta 2, a block that moves two blocks
    row = ref_eviction.rotation_lut(2, 8, 4, 2.0)[2]
    assert np.allclose(row, [-0.65364362, -0.95136312, 0.75680249, -0.30807174], atol=1e-7)


def test_snapkv_window_rule_matches_reference_cases():
    # tests/cpp/cache_eviction.cpp:648-665
    assert ref_eviction.snapkv_window(8, 100, 30, 45) == 0
    assert ref_eviction.snapkv_window(16, 30, 13, 4) == 3
    assert ref_eviction.snapkv_window(16, 30, 16, 8) == 8


def test_eviction_picks_the_lowest_scored_blocks():
    """Sanity of the bridge itself: NORM_SUM over one registered vector evicts the blocks with the
    smallest block sums from the evictable area only."""
    bs = 4
    scores = np.ones(12 * bs, np.float32)
    scores[3 * bs:4 * bs] = 0.01      # block 3
    scores[6 * bs:7 * bs] = 0.02      # block 6
    scores[0:bs] = 0.0                # start area: never evicted
    got = ref_eviction.select_blocks([scores], [0], start_size=bs, recent_size=2 * bs, max_cache_size=10 * bs, block_size=bs, snapkv_window=0)
    assert got == [3, 6]


@pytest.mark.gpu
@pytest.mark.parametrize("aggregation", ["SUM", "NORM_SUM"])
def test_block_selection_from_gpu_scores_equals_selection_from_restatement(aggregation):
    """Decode steps of long sequences: the reference's eviction algorithm must choose the same
    blocks whether it reads the CUDA operator's scores or the CPU restatement's."""
    from tests import pa_harness as H
    bs = 32
    past = [1500, 2047, 900, 3100]
    wl = H.small_workload(hq=28, hkv=4, d=128, bs=bs, act=torch.bfloat16, cache="u8", past=past, new=[1, 1, 1, 1], seed=314)
    wl.score_aggregation_window = np.ones(4, np.int32)
    res = H.run_both(wl)
    off = 0
    for s, p in enumerate(past):
        n = p + 1
        ref, got = res["scores_ref"][off:off + n], res["scores_gpu"][off:off + n]
        off += n
        assert np.abs(got - ref).max() <= 1e-2 * max(1.0, np.abs(ref).max())
        kw = dict(start_size=bs, recent_size=4 * bs, max_cache_size=(n // bs - 6) * bs, block_size=bs, aggregation=aggregation, snapkv_window=0,
                  max_pool_window=7)
        # the algorithm tracks whole blocks: hand it the scores of the full blocks
        full = (n // bs) * bs
        want_blocks = ref_eviction.select_blocks([ref[:full]], [0], **kw)
        got_blocks = ref_eviction.select_blocks([got[:full]], [0], **kw)
        assert len(want_blocks) >= 5
        assert got_blocks == want_blocks, (s, want_blocks, got_blocks)
