"""ctypes mirror of the Sampler step (include/sampler_b200.h) for device tensors: the numeric half
of ov::genai::Sampler::sample (src/cpp/src/sampling/sampler.cpp:1708-1810) as one kernel launch.
The request bookkeeping (per-request std::mt19937, token maps, stop checks) lives in the C++ class
genai_b200::Sampler (csrc/host/sampler_host.hpp); this wrapper is what bench.py and Python callers
use when they already hold packed row parameters."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import numpy as np
import torch

from . import GenaiB200Error, _sampler_abi as A, load_library


class SamplerStep:
    def __init__(self, device: int = 0):
        self.lib = load_library()
        self.device = device
        self._h = C.c_void_p()
        rc = self.lib.sampler_b200_create(device, 0, 0, C.byref(self._h))
        if rc != 0:
            raise GenaiB200Error(f"sampler_b200_create: {self.lib.sampler_b200_last_error().decode()}")

    def close(self) -> None:
        if getattr(self, "_h", None):
            self.lib.sampler_b200_destroy(self._h)
            self._h = None

    __del__ = close

    def launch_count(self) -> int:
        return int(self.lib.sampler_b200_launch_count(self._h)) if self._h else 0

    def stage(self, rows: np.ndarray, hist: Optional[Tuple[np.ndarray, np.ndarray, np.ndarray]] = None):
        """Copies packed row parameters (dtype _sampler_abi.ROW_DTYPE) and the CSR history to the device."""
        dev = torch.device("cuda", self.device)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.uint8) if a.dtype.fields else np.ascontiguousarray(a)).to(dev)
        n = len(rows)
        raw = torch.empty(len(hist[1]), dtype=torch.float32, device=dev) if hist is not None else None
        return {"n": n, "rows": t(rows), "hist": tuple(t(x) for x in hist) if hist is not None else None, "hist_raw": raw,
                "tokens": torch.full((n,), -1, dtype=torch.int64, device=dev), "log_probs": torch.zeros(n, dtype=torch.float32, device=dev)}

    def step(self, logits: torch.Tensor, staged: dict, stream: int = 0, out_tokens: Optional[torch.Tensor] = None):
        """One step over device logits [rows, vocab] f32 (mutated in place); asynchronous on `stream`
        (a cudaStream_t handle; 0 = the legacy default stream).  Returns the output tensors: the staged
        ones, or `out_tokens` (int64, at least `rows` long - e.g. this rank's row of the exchange buffer)."""
        a = A.sampler_step_args()
        a.struct_size = C.sizeof(A.sampler_step_args)
        a.logits = logits.data_ptr()
        a.num_logit_rows, a.vocab = logits.shape
        a.num_rows = staged["n"]
        a.rows = staged["rows"].data_ptr()
        if staged["hist"] is not None:
            a.hist_offsets, a.hist_ids, a.hist_meta = (x.data_ptr() for x in staged["hist"])
            a.hist_raw = staged["hist_raw"].data_ptr()   # scratch for rows that report raw log-probabilities
        tokens = staged["tokens"] if out_tokens is None else out_tokens
        a.out_token = tokens.data_ptr()
        a.out_log_prob = staged["log_probs"].data_ptr()
        a.stream = stream if stream else 1   # 1 = cudaStreamLegacy: a null handle would select the handle's own stream
        rc = self.lib.sampler_b200_step(self._h, C.byref(a))
        if rc != 0:
            raise GenaiB200Error(f"sampler_b200_step: {self.lib.sampler_b200_last_error().decode()}")
        return tokens, staged["log_probs"]
