"""Shared plumbing of the PagedAttention parity tests: builds one set of seeded host inputs and
runs it through the CPU oracle and through the CUDA path (C ABI), filling the past of every
sequence through each side's own cache-write path first."""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as entry  # noqa: E402

pkg = entry.load_package()
from openvino_genai_b200 import _abi, workloads  # noqa: E402
from oracle import pa_oracle  # noqa: E402

_ACT = {torch.float32: _abi.PA_DTYPE_F32, torch.float16: _abi.PA_DTYPE_F16, torch.bfloat16: _abi.PA_DTYPE_BF16}
_CACHE = {"f16": _abi.PA_DTYPE_F16, "bf16": _abi.PA_DTYPE_BF16, "u8": _abi.PA_DTYPE_U8}


def small_workload(*, hq, hkv, d, bs, act, cache, past, new, seed, pool=None, scale=None):
    past = np.asarray(past, np.int64)
    new = np.asarray(new, np.int64)
    need = int(((past + new + bs - 1) // bs).sum())
    return workloads.make_workload("small", hq=hq, hkv=hkv, d=d, bs=bs, act=act, cache=cache, past=past, new=new,
                                   num_blocks=pool or need + 3, seed=seed, scale=scale)


def desc_of(wl) -> _abi.pa_model_desc:
    return _abi.pa_model_desc(C.sizeof(_abi.pa_model_desc), wl.num_q_heads, wl.num_kv_heads, wl.head_size, wl.block_size,
                              _ACT[wl.act_dtype], _CACHE[wl.cache_dtype])


def block_bytes(wl) -> int:
    per = wl.block_size * (wl.head_size + 8) if wl.cache_dtype == "u8" else wl.block_size * wl.head_size * 2
    return per * wl.num_kv_heads


def _p(x):
    if x is None:
        return None
    return x.ctypes.data if isinstance(x, np.ndarray) else x.data_ptr()


def host_args(wl, q, k, v, out, kc, vc, scores=None, with_eviction=True) -> _abi.pa_forward_args:
    """pa_forward_args over HOST buffers (numpy / CPU torch)."""
    a = _abi.pa_forward_args()
    a.struct_size = C.sizeof(_abi.pa_forward_args)
    a.query, a.key, a.value, a.output = _p(q), _p(k), _p(v), _p(out)
    a.num_tokens = wl.num_tokens
    a.key_cache, a.value_cache, a.num_blocks = _p(kc), _p(vc), wl.num_blocks
    a.past_lens, a.subsequence_begins = _p(wl.past_lens), _p(wl.subsequence_begins)
    a.block_indices, a.block_indices_begins = _p(wl.block_indices), _p(wl.block_indices_begins)
    a.num_sequences, a.num_block_indices = wl.num_sequences, int(wl.block_indices.shape[0])
    a.max_context_len = wl.max_context_len
    a.scale = wl.scale
    if with_eviction:
        if scores is not None and wl.score_aggregation_window is not None:
            a.score_aggregation_window = _p(wl.score_aggregation_window)
            a.scores, a.scores_len = _p(scores), int(scores.shape[0])
        if wl.rotated_block_indices is not None:
            a.rotated_block_indices = _p(wl.rotated_block_indices)
            a.rotation_deltas = _p(wl.rotation_deltas)
            a.num_rotated_blocks = int(wl.rotated_block_indices.shape[0])
            a.rotation_trig_lut = _p(wl.rotation_trig_lut)
            a.rotation_lut_rows = int(wl.rotation_trig_lut.shape[0])
    return a


def make_host_data(wl):
    """q/k/v of the step and the keys/values of the past, all CPU tensors in the activation dtype."""
    q, k, v = workloads.random_activations(wl, "cpu")
    fill = workloads.past_as_write_step(wl)
    _, pk, pv = workloads.random_activations(fill, "cpu", seed_offset=1)
    return q, k, v, fill, pk, pv


def run_oracle(wl, data=None, threads=0):
    q, k, v, fill, pk, pv = data or make_host_data(wl)
    desc = desc_of(wl)
    nbytes = wl.num_blocks * block_bytes(wl)
    kc = np.zeros(nbytes, np.uint8)
    vc = np.zeros(nbytes, np.uint8)
    if fill.num_tokens:
        dummy = torch.zeros((fill.num_tokens, 1), dtype=wl.act_dtype)
        rc = pa_oracle.write_kv(desc, host_args(fill, dummy, pk, pv, dummy, kc, vc, with_eviction=False))
        assert rc == 0, rc
    out = torch.zeros_like(q)
    scores = np.full(wl.scores_len, np.nan, np.float32) if wl.score_aggregation_window is not None else None
    rc = pa_oracle.forward(desc, host_args(wl, q, k, v, out, kc, vc, scores), threads)
    assert rc == 0, rc
    return {"out_ref": out.float().numpy(), "kc_ref": kc, "vc_ref": vc, "scores_ref": scores}


def make_op(wl, device=0):
    return pkg.PagedAttentionExtension(wl.num_q_heads, wl.num_kv_heads, wl.head_size, wl.block_size, wl.act_dtype, wl.cache_dtype, device)


def run_gpu(wl, data=None, device=0, host_entry=False, op=None, caches=None):
    q, k, v, fill, pk, pv = data or make_host_data(wl)
    dev = torch.device("cuda", device)
    op = op or make_op(wl, device)
    kc, vc = caches if caches is not None else op.allocate_cache(wl.num_blocks, fill=0)   # caches: flat uint8 device tensors the caller owns
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev) if a is not None else None
    if fill.num_tokens:
        dummy = torch.zeros((fill.num_tokens, 1), dtype=wl.act_dtype, device=dev)
        args = op.make_args(dummy, pk.to(dev), pv.to(dev), dummy, kc, vc, t(fill.past_lens), t(fill.subsequence_begins),
                            t(fill.block_indices), t(fill.block_indices_begins), fill.scale, fill.max_context_len)
        op._check(op.lib.pa_b200_write_kv(op._h, C.byref(args)))
        torch.cuda.synchronize(dev)
    want_scores = wl.score_aggregation_window is not None
    if host_entry:
        out = torch.zeros_like(q)
        scores = np.full(wl.scores_len, np.nan, np.float32) if want_scores else None
        inputs = {"query": q, "key": k, "value": v, "key_cache": kc, "value_cache": vc, "past_lens": wl.past_lens,
                  "subsequence_begins": wl.subsequence_begins, "block_indices": wl.block_indices,
                  "block_indices_begins": wl.block_indices_begins, "scale": wl.scale, "max_context_len": wl.max_context_len,
                  "score_aggregation_window": wl.score_aggregation_window, "rotated_block_indices": wl.rotated_block_indices,
                  "rotation_deltas": wl.rotation_deltas, "rotation_trig_lut": wl.rotation_trig_lut}
        op.evaluate(inputs, {"output": out, "scores": scores})
        out_np, scores_np = out.float().numpy(), scores
    else:
        out = torch.zeros_like(q, device=dev)
        scores = torch.full((wl.scores_len,), float("nan"), dtype=torch.float32, device=dev) if want_scores else None
        inputs = {"query": q.to(dev), "key": k.to(dev), "value": v.to(dev), "key_cache": kc, "value_cache": vc,
                  "past_lens": t(wl.past_lens), "subsequence_begins": t(wl.subsequence_begins), "block_indices": t(wl.block_indices),
                  "block_indices_begins": t(wl.block_indices_begins), "scale": wl.scale, "max_context_len": wl.max_context_len,
                  "score_aggregation_window": t(wl.score_aggregation_window), "rotated_block_indices": t(wl.rotated_block_indices),
                  "rotation_deltas": t(wl.rotation_deltas), "rotation_trig_lut": t(wl.rotation_trig_lut)}
        op.evaluate(inputs, {"output": out, "scores": scores})
        torch.cuda.synchronize(dev)
        out_np = out.float().cpu().numpy()
        scores_np = scores.cpu().numpy() if want_scores else None
    status = op.device_status()
    return {"out_gpu": out_np, "kc_gpu": kc.cpu().numpy(), "vc_gpu": vc.cpu().numpy(), "scores_gpu": scores_np,
            "status": status, "launches": op.launch_count(), "prefill_kernel": op.last_prefill_kernel(), "op": op}


def run_both(wl, device=0, host_entry=False):
    data = make_host_data(wl)
    res = run_oracle(wl, data)
    res.update(run_gpu(wl, data, device, host_entry))
    return res


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    """max |a - b| relative to the largest reference magnitude."""
    denom = float(np.abs(b).max()) or 1.0
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / denom)


def wrap_device_bytes(ptr: int, nbytes: int, device=0) -> torch.Tensor:
    """A flat uint8 torch view of device memory that something else owns (no copy, no ownership)."""
    class _Mem:
        pass
    holder = _Mem()
    holder.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 3, "strides": None}
    return torch.as_tensor(holder, device=torch.device("cuda", device))
