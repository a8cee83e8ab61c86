"""The KV cache pool that grows in place (pa_b200_cache_pool_*): what KVCacheManager::allocate_cache_if_needed
(src/cpp/src/continuous_batching/cache/kv_cache_manager.hpp:159-262) achieves by allocate-new-and-copy-all.
After a growth the cache addresses are the same, the blocks written before keep their bytes, the new blocks
read as zeros, and the operator over the grown pool equals the oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests import pa_harness as H
from openvino_genai_b200 import _abi

pytestmark = pytest.mark.gpu


class Pool:
    def __init__(self, wl, max_blocks, initial):
        self.lib = H.pkg.load_library()
        self.desc = H.desc_of(wl)
        self.block_bytes = H.block_bytes(wl)
        self.h = C.c_void_p()
        rc = self.lib.pa_b200_cache_pool_create(C.byref(self.desc), 0, max_blocks, initial, C.byref(self.h))
        assert rc == 0, self.lib.pa_b200_cache_pool_last_error()

    def get(self):
        k, v, n = C.c_void_p(), C.c_void_p(), C.c_int64()
        assert self.lib.pa_b200_cache_pool_get(self.h, C.byref(k), C.byref(v), C.byref(n)) == 0
        return k.value, v.value, n.value

    def tensors(self):
        k, v, n = self.get()
        return H.wrap_device_bytes(k, n * self.block_bytes), H.wrap_device_bytes(v, n * self.block_bytes)

    def grow(self, n):
        return self.lib.pa_b200_cache_pool_grow(self.h, n)

    def close(self):
        if self.h:
            self.lib.pa_b200_cache_pool_destroy(self.h)
            self.h = None


@pytest.mark.parametrize("cache,act", [("u8", torch.bfloat16), ("f16", torch.float16)])
def test_pool_grows_without_moving_or_copying(cache, act):
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=act, cache=cache, past=[700, 90, 1500, 33], new=[1, 1, 1, 40], seed=131, pool=120)
    pool = Pool(wl, max_blocks=4096, initial=8)
    try:
        k0, v0, n0 = pool.get()
        assert n0 == 8 and k0 and v0 and k0 != v0
        kc, vc = pool.tensors()
        assert int(kc.sum().item()) == 0, "a fresh pool reads as zeros"
        pattern = torch.arange(kc.numel(), device=kc.device, dtype=torch.int64).remainder(251).to(torch.uint8)
        kc.copy_(pattern); vc.copy_(pattern + 1)
        torch.cuda.synchronize()
        assert pool.grow(4) == 0 and pool.get()[2] == 8, "a smaller request changes nothing"
        assert pool.grow(wl.num_blocks) == 0
        k1, v1, n1 = pool.get()
        assert (k1, v1) == (k0, v0) and n1 == wl.num_blocks, "the cache addresses never move"
        kc2, vc2 = pool.tensors()
        assert torch.equal(kc2[:kc.numel()], pattern) and torch.equal(vc2[:vc.numel()], pattern + 1), "blocks written before the growth keep their bytes"
        assert int(kc2[kc.numel():].sum().item()) == 0 and int(vc2[vc.numel():].sum().item()) == 0, "new blocks read as zeros"
        assert pool.grow(4097) == _abi.PA_ERR_TOO_LARGE
        # the operator over the grown pool (block ids on both sides of the old end) against the oracle
        kc2.zero_(); vc2.zero_()
        data = H.make_host_data(wl)
        res = H.run_oracle(wl, data)
        res.update(H.run_gpu(wl, data, caches=(kc2, vc2)))
        assert res["status"] == 0
        assert np.array_equal(res["kc_gpu"], res["kc_ref"]) and np.array_equal(res["vc_gpu"], res["vc_ref"])
        assert H.rel_err(res["out_gpu"], res["out_ref"]) < (1e-2 if cache == "u8" else 8e-3)
        assert pool.grow(3000) == 0 and pool.get()[:2] == (k0, v0)
        assert np.array_equal(pool.tensors()[0][: wl.num_blocks * pool.block_bytes].cpu().numpy(), res["kc_gpu"])
    finally:
        pool.close()


def test_pool_argument_errors():
    wl = H.small_workload(hq=8, hkv=2, d=128, bs=32, act=torch.bfloat16, cache="u8", past=[10], new=[1], seed=1)
    lib = H.pkg.load_library()
    desc = H.desc_of(wl)
    h = C.c_void_p()
    assert lib.pa_b200_cache_pool_create(C.byref(desc), 0, 0, 0, C.byref(h)) == _abi.PA_ERR_INVALID_ARG
    assert lib.pa_b200_cache_pool_create(C.byref(desc), 0, 16, 32, C.byref(h)) == _abi.PA_ERR_INVALID_ARG
    assert lib.pa_b200_cache_pool_grow(None, 4) == _abi.PA_ERR_INVALID_ARG
