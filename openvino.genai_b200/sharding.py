"""Request-level sharding across ranks: sequences (and their KV block pools) are partitioned by
rank, so the attention step needs no collective; the only exchange of an engine step is the
all-gather of the sampled token ids (and of a status word) so that every rank's scheduler sees
all of them.  The reference is single-process (its only multi-device notion is "all execution
devices are GPU", src/cpp/src/continuous_batching/pipeline_impl.cpp:183-190); this module is the
host logic of the multi-GPU extension and runs equally on the gloo backend for CPU tests."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist


def shard_sequences(context_lens: Sequence[int], world_size: int) -> List[np.ndarray]:
    """Assigns sequences to ranks so that the summed context length (the KV bytes a decode step
    reads) is balanced: longest first, each to the currently lightest rank.  Returns, per rank,
    the ascending indices of its sequences."""
    lens = np.asarray(context_lens, np.int64)
    order = np.argsort(-lens, kind="stable")
    load = np.zeros(world_size, np.int64)
    owner = np.empty(len(lens), np.int64)
    for i in order:
        r = int(np.argmin(load))
        owner[i] = r
        load[r] += lens[i]
    return [np.sort(np.nonzero(owner == r)[0]) for r in range(world_size)]


def all_gather_token_ids(local_ids: torch.Tensor, local_index: torch.Tensor, total: int,
                         group: Optional[dist.ProcessGroup] = None, counts: Optional[Sequence[int]] = None) -> torch.Tensor:
    """All-gathers this rank's sampled ids (int64 [n_local], for the global sequence indices
    `local_index`) into an int64 [total] tensor in global sequence order on every rank.
    Ranks may own different numbers of sequences: shares are padded to the largest one.
    `counts` (sequences per rank) saves the size exchange and its host synchronisation when the
    partition is known on every rank, as it is after shard_sequences()."""
    world = dist.get_world_size(group)
    if counts is not None:
        counts = [torch.tensor([int(c)], dtype=torch.int64) for c in counts]
    else:
        n_local = torch.tensor([local_ids.numel()], dtype=torch.int64, device=local_ids.device)
        counts = [torch.zeros_like(n_local) for _ in range(world)]
        dist.all_gather(counts, n_local, group=group)
    cap = int(max(int(c.item()) for c in counts))
    packed = torch.full((2, cap), -1, dtype=torch.int64, device=local_ids.device)
    packed[0, : local_ids.numel()] = local_ids
    packed[1, : local_ids.numel()] = local_index
    gathered = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(gathered, packed, group=group)   # list form: available on both nccl and gloo
    out = torch.full((total,), -1, dtype=torch.int64, device=local_ids.device)
    for r in range(world):
        n = int(counts[r].item())
        out[gathered[r][1, :n]] = gathered[r][0, :n]
    return out


class TokenExchange:
    """The exchange step on GPUs: one in-place ncclAllGather of a fixed [world, cap] int64 buffer, issued by
    the C++ host layer (include/exchange_b200.h) on the sampler's stream.  The sampler writes this
    rank's ids straight into `local_row`; after `all_gather(n_local, stream)` every rank holds all
    rows in `all_rows` (rank-contiguous; slot k of row r is the k-th sequence rank r owns; unused
    slots are -1).  The communicator id travels through torch.distributed (any backend)."""

    def __init__(self, device: torch.device, cap: int, group: Optional[dist.ProcessGroup] = None):
        import ctypes as C
        from . import _exchange_abi as X, load_library
        self.lib = load_library()
        self.rank, self.world, self.cap = dist.get_rank(group), dist.get_world_size(group), int(cap)
        ident = torch.zeros(X.ID_BYTES, dtype=torch.uint8)
        if self.rank == 0:
            buf = (C.c_uint8 * X.ID_BYTES)()
            self._check(self.lib.exchange_b200_unique_id(buf))
            ident = torch.frombuffer(bytearray(buf), dtype=torch.uint8).clone()
        ident = ident.to(device) if dist.get_backend(group) == "nccl" else ident
        dist.broadcast(ident, src=0, group=group)
        raw = bytes(ident.cpu().numpy().tobytes())
        self._h = C.c_void_p()
        self._check(self.lib.exchange_b200_create(C.c_char_p(raw), self.rank, self.world, device.index or 0, self.cap, C.byref(self._h)))
        n = self.world * self.cap
        base = self.lib.exchange_b200_all_rows(self._h)
        self.all_rows = _wrap_device_int64(base, n, device).view(self.world, self.cap)
        self.local_row = self.all_rows[self.rank]

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise RuntimeError(f"exchange_b200 error {rc}: {self.lib.exchange_b200_last_error().decode()}")

    def all_gather(self, n_local: int, stream: int) -> torch.Tensor:
        self._check(self.lib.exchange_b200_all_gather_ids(self._h, int(n_local), stream or None))
        return self.all_rows

    def close(self) -> None:
        if getattr(self, "_h", None):
            self.lib.exchange_b200_destroy(self._h)
            self._h = None


def _wrap_device_int64(ptr: int, n: int, device: torch.device) -> torch.Tensor:
    """A torch view of device memory the C++ layer owns (no copy, no ownership)."""
    class _Mem:
        pass
    holder = _Mem()
    holder.__cuda_array_interface__ = {"shape": (n,), "typestr": "<i8", "data": (int(ptr), False), "version": 3, "strides": None}
    return torch.as_tensor(holder, device=device)


def max_over_ranks(value: float, device, group: Optional[dist.ProcessGroup] = None) -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
