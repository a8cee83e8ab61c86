"""Eviction scoring on the device (include/eviction_b200.h) against the reference's own CacheEvictionAlgorithm
(cache/cache_eviction.cpp compiled unmodified, oracle/ref_eviction_bridge.cpp): the same score vectors are
registered step by step on both sides; the evicted block lists must be identical at every step, for SUM and
NORM_SUM, with and without a SnapKV window, on random scores and on scores with many equal block sums."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests import pa_harness as H    # loads the package
from openvino_genai_b200 import _eviction_abi as E
from oracle import ref_eviction

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(ref_eviction.lib() is None or not hasattr(ref_eviction.lib(), "ref_eviction_new"),
                                                  reason="oracle/_ref/libref_eviction.so was not built with the step-by-step entry points")]


class DeviceEviction:
    def __init__(self, *, start_size, recent_size, max_cache_size, block_size, aggregation, snapkv_window, num_slots, max_tokens, layers=1):
        self.lib = H.pkg.load_library()
        cfg = E.eviction_config_b200(C.sizeof(E.eviction_config_b200), start_size, recent_size, max_cache_size, block_size,
                                     E.AGG_SUM if aggregation == "SUM" else E.AGG_NORM_SUM, snapkv_window, 7, layers, num_slots, max_tokens, 512)
        self.h = C.c_void_p()
        rc = self.lib.eviction_b200_create(C.byref(cfg), 0, C.byref(self.h))
        assert rc == 0, self.lib.eviction_b200_last_error()
        self.max_evicted = 512

    def step(self, scores_per_seq, slots, snapkv, do_evict=True, layer=0):
        dev = torch.device("cuda", 0)
        flat = np.concatenate([np.asarray(s, np.float32) for s in scores_per_seq]) if scores_per_seq else np.zeros(0, np.float32)
        lens = np.array([len(s) for s in scores_per_seq], np.int32)
        begins = np.zeros(len(lens), np.int64)
        begins[1:] = np.cumsum(lens)[:-1]
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        d = [t(flat if len(flat) else np.zeros(1, np.float32)), t(begins), t(lens), t(np.array(slots, np.int32)), t(np.array(snapkv, np.int32))]
        cnt = torch.full((len(lens),), -1, dtype=torch.int32, device=dev)
        blocks = torch.full((len(lens), self.max_evicted), -1, dtype=torch.int32, device=dev)
        a = E.eviction_step_args(C.sizeof(E.eviction_step_args), layer, len(lens), d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(),
                                 d[4].data_ptr(), 1 if do_evict else 0, cnt.data_ptr(), blocks.data_ptr(), torch.cuda.current_stream(dev).cuda_stream or 1)
        rc = self.lib.eviction_b200_step(self.h, C.byref(a))
        assert rc == 0, self.lib.eviction_b200_last_error()
        torch.cuda.synchronize()
        bits = C.c_uint32(0)
        assert self.lib.eviction_b200_last_device_status(self.h, C.byref(bits)) == 0 and bits.value == 0, hex(bits.value)
        c, b = cnt.cpu().numpy(), blocks.cpu().numpy()
        return [b[i, :c[i]].tolist() for i in range(len(lens))]

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.eviction_b200_destroy(self.h)
            self.h = None


@pytest.mark.parametrize("aggregation", ["SUM", "NORM_SUM"])
@pytest.mark.parametrize("snapkv_window", [0, 8])
@pytest.mark.parametrize("kind", ["random", "many_equal_block_sums"])
def test_block_lists_equal_the_reference_over_a_generation(aggregation, snapkv_window, kind):
    bs, start, recent, max_cache = 16, 32, 64, 256
    rng = np.random.default_rng(len(aggregation) * 100 + snapkv_window * 10 + len(kind))
    n_seq = 5
    prompt = [40, 300, 130, 257, 1000]
    dev = DeviceEviction(start_size=start, recent_size=recent, max_cache_size=max_cache, block_size=bs, aggregation=aggregation,
                         snapkv_window=snapkv_window, num_slots=9, max_tokens=1400)
    ref = [ref_eviction.Algorithm(start_size=start, recent_size=recent, max_cache_size=max_cache, block_size=bs, aggregation=aggregation,
                                  snapkv_window=snapkv_window, max_pool_window=7) for _ in range(n_seq)]
    slots = [3, 0, 8, 5, 1]
    ctx = [0] * n_seq          # tokens in the cache as the eviction algorithm sees them (context - evicted)

    def scores_of(length):
        if kind == "random":
            return rng.random(length).astype(np.float32) * rng.choice([1e-3, 1.0, 50.0])
        return (rng.integers(0, 3, size=length) * 0.25).astype(np.float32)   # few distinct values: equal block sums, index tie-breaks

    total_evicted = 0
    for step in range(60):
        per_seq, snap = [], []
        for s in range(n_seq):
            if step == 0:
                ctx[s] = prompt[s]
                snap.append(min(snapkv_window, prompt[s]) if snapkv_window else 0)
            else:
                ctx[s] += 1
                snap.append(0)
            per_seq.append(scores_of(ctx[s]))
        want = []
        for s in range(n_seq):
            ref[s].register(per_seq[s], snap[s])
            want.append(ref[s].evict())
        got = dev.step(per_seq, slots, snap)
        assert got == want, (step, got, want)
        for s in range(n_seq):
            ctx[s] -= len(want[s]) * bs
            total_evicted += len(want[s])
    assert total_evicted > 40, "the test must actually evict"


def test_slots_are_independent_and_can_be_reused():
    bs = 16
    kw = dict(start_size=16, recent_size=32, max_cache_size=128, block_size=bs, aggregation="NORM_SUM", snapkv_window=0)
    dev = DeviceEviction(num_slots=4, max_tokens=600, **kw)
    rng = np.random.default_rng(5)
    a = ref_eviction.Algorithm(max_pool_window=7, **kw)
    s1 = rng.random(400).astype(np.float32)
    a.register(s1)
    assert dev.step([s1], [2], [0]) == [a.evict()]
    # the slot is handed to a new sequence
    assert dev.lib.eviction_b200_reset_slot(dev.h, 2, None) == 0
    b = ref_eviction.Algorithm(max_pool_window=7, **kw)
    s2 = rng.random(200).astype(np.float32)
    b.register(s2)
    assert dev.step([s2], [2], [0]) == [b.evict()]
