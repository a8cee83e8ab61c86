"""Host logic of the multi-GPU extension on two gloo ranks (CPU): balanced sequence sharding and
the all-gather of sampled ids into global sequence order."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, lens, result_dir):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(root))
    import __graft_entry__ as entry
    entry.load_package()
    from openvino_genai_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shards = sharding.shard_sequences(lens, world)
        mine = torch.from_numpy(shards[rank])
        ids = mine * 10 + rank                                   # a recognisable "sampled id" per sequence
        out = sharding.all_gather_token_ids(ids, mine, len(lens))
        same = sharding.all_gather_token_ids(ids, mine, len(lens), counts=[len(p) for p in shards])
        assert torch.equal(out, same), "known partition sizes must give the same result as the size exchange"
        mx = sharding.max_over_ranks(float(rank + 1), "cpu")
        np.save(os.path.join(result_dir, f"out{rank}.npy"), out.numpy())
        np.save(os.path.join(result_dir, f"mx{rank}.npy"), np.array([mx]))
    finally:
        dist.destroy_process_group()


def test_shards_are_balanced_and_cover_everything():
    import __graft_entry__ as entry
    entry.load_package()
    from openvino_genai_b200 import sharding
    rng = np.random.default_rng(5)
    lens = np.exp(rng.uniform(np.log(1024), np.log(32768), size=1024)).astype(np.int64)   # log-uniform like the 70B config
    for world in (1, 2, 4, 8):
        shards = sharding.shard_sequences(lens, world)
        assert sorted(np.concatenate(shards).tolist()) == list(range(len(lens)))
        loads = np.array([lens[s].sum() for s in shards])
        assert loads.max() <= loads.mean() * 1.01 + lens.max()


def test_all_gather_of_sampled_ids_on_two_gloo_ranks(tmp_path):
    lens = [5000, 100, 2500, 2400, 90, 80, 70]                   # uneven shares: 3 vs 4 sequences
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, lens, str(tmp_path)), nprocs=2, join=True)
    out0 = np.load(tmp_path / "out0.npy")
    out1 = np.load(tmp_path / "out1.npy")
    assert np.array_equal(out0, out1)
    assert np.all(out0 >= 0)
    import __graft_entry__ as entry
    entry.load_package()
    from openvino_genai_b200 import sharding
    shards = sharding.shard_sequences(lens, 2)
    for r in range(2):
        assert np.array_equal(out0[shards[r]], shards[r] * 10 + r)
    assert np.load(tmp_path / "mx0.npy")[0] == 2.0 and np.load(tmp_path / "mx1.npy")[0] == 2.0
