"""Shared plumbing of the Sampler parity tests: builds one set of seeded host inputs (logits,
per-row parameters, CSR history, uniform draws) and runs it through the CPU oracle and through
the CUDA kernel (C ABI)."""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402

pkg = entry.load_package()
from openvino_genai_b200 import _sampler_abi as A  # noqa: E402
from oracle import sampler_oracle  # noqa: E402


def make_rows(n, *, do_sample=1, temperature=1.0, top_k=A.TOP_K_OFF, top_p=1.0, min_p=0.0, repetition_penalty=1.0,
              presence_penalty=0.0, frequency_penalty=0.0, seeds=None, logits_rows=None):
    rows = np.zeros(n, dtype=np.dtype(A.ROW_DTYPE))
    rows["logits_row"] = np.arange(n) if logits_rows is None else logits_rows
    rows["top_k"] = top_k
    rows["do_sample"] = do_sample
    rows["temperature"] = temperature
    rows["top_p"] = top_p
    rows["min_p"] = min_p
    rows["repetition_penalty"] = repetition_penalty
    rows["presence_penalty"] = presence_penalty
    rows["frequency_penalty"] = frequency_penalty
    seeds = seeds if seeds is not None else np.arange(n) + 1
    rows["rand_u"] = [sampler_oracle.uniform_stream(int(s), 1)[0] for s in seeds]
    return rows


def make_history(rng, n, vocab, generated_len, prompt_len=0, stop_ids=None):
    """CSR history of distinct ids per row: prompt ids (flag 1), generated ids with counts (flag 2)."""
    offs, ids, meta = [0], [], []
    for _ in range(n):
        gen = rng.integers(0, vocab, size=generated_len)
        prompt = rng.integers(0, vocab, size=prompt_len)
        uniq = {}
        for t in prompt:
            uniq.setdefault(int(t), [0, 0])[0] = 1
        for t in gen:
            e = uniq.setdefault(int(t), [0, 0])
            e[1] += 1
        for t in (stop_ids or []):
            uniq.setdefault(int(t), [0, 0])
        for t in sorted(uniq):
            flag = (A.HIST_IN_PROMPT if uniq[t][0] else 0) | (A.HIST_GENERATED if uniq[t][1] else 0)
            if stop_ids and t in stop_ids:
                flag |= A.HIST_STOP_MASK
            ids.append(t)
            meta.append((uniq[t][1] << 3) | flag)
        offs.append(len(ids))
    return np.array(offs, np.int64), np.array(ids, np.int32), np.array(meta, np.uint32)


def step_args(logits, rows, hist, out_tok, out_lp, ptr=lambda x: x.ctypes.data):
    a = A.sampler_step_args()
    a.struct_size = C.sizeof(A.sampler_step_args)
    a.logits = ptr(logits)
    a.num_logit_rows, a.vocab = logits.shape
    a.num_rows = len(rows) if isinstance(rows, np.ndarray) else rows.shape[0] // 48
    a.rows = ptr(rows)
    if hist is not None:
        a.hist_offsets, a.hist_ids, a.hist_meta = ptr(hist[0]), ptr(hist[1]), ptr(hist[2])
    a.out_token, a.out_log_prob = ptr(out_tok), ptr(out_lp)
    return a


def run_oracle(logits, rows, hist=None, threads=0):
    lg = logits.copy()
    tok = np.full(len(rows), -7, np.int64)
    lp = np.zeros(len(rows), np.float32)
    rc = sampler_oracle.step(step_args(lg, rows, hist, tok, lp), threads)
    return rc, tok, lp, lg


class GpuSampler:
    def __init__(self, device=0):
        self.lib = pkg.load_library()
        self.h = C.c_void_p()
        rc = self.lib.sampler_b200_create(device, 0, 0, C.byref(self.h))
        assert rc == 0, self.lib.sampler_b200_last_error()

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.sampler_b200_destroy(self.h)
            self.h = None

    def step_host(self, logits, rows, hist=None, copy_back=True):
        lg = logits.copy()
        tok = np.full(len(rows), -7, np.int64)
        lp = np.zeros(len(rows), np.float32)
        args = step_args(lg, rows, hist, tok, lp)
        rc = self.lib.sampler_b200_step_host(self.h, C.byref(args), 1 if copy_back else 0)
        return rc, tok, lp, lg

    def stage(self, rows, hist, dev):
        """Copies the row parameters and the CSR history to the device once."""
        import torch
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.uint8) if a.dtype.fields else a).to(dev)
        return {"rows": t(rows), "hist": tuple(t(x) for x in hist) if hist is not None else None,
                "hist_raw": torch.empty(len(hist[1]), dtype=torch.float32, device=dev) if hist is not None else None,
                "tok": torch.full((len(rows),), -7, dtype=torch.int64, device=dev),
                "lp": torch.zeros(len(rows), dtype=torch.float32, device=dev)}

    def step_device(self, logits_t, rows, hist=None, stream=None, staged=None):
        """logits_t: CUDA torch tensor [rows, vocab] f32 (mutated in place)."""
        import torch
        dev = logits_t.device
        staged = staged or self.stage(rows, hist, dev)
        rows_t, hist_t, tok, lp = staged["rows"], staged["hist"], staged["tok"], staged["lp"]
        a = step_args(logits_t, rows_t, hist_t, tok, lp, ptr=lambda x: x.data_ptr())
        a.num_rows = len(rows)
        a.num_logit_rows, a.vocab = logits_t.shape
        s = torch.cuda.current_stream(dev).cuda_stream if stream is None else stream
        a.stream = s if s else 1
        if staged.get("hist_raw") is not None:
            a.hist_raw = staged["hist_raw"].data_ptr()
        rc = self.lib.sampler_b200_step(self.h, C.byref(a))
        self._keep = (rows_t, hist_t, staged.get("hist_raw"))
        return rc, tok, lp


def synthetic_logits(rng, n, vocab, spikes=8, sigma=2.0, spike=15.0):
    x = (rng.standard_normal((n, vocab)) * sigma).astype(np.float32)
    for r in range(n):
        x[r, rng.choice(vocab, size=spikes, replace=False)] += np.float32(spike)
    return x
