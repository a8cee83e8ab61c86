"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

No dataset is involved: lengths, block tables and tensor values are drawn from numpy / torch
generators with fixed seeds.  The same builder serves the parity tests (small sizes, host tensors
that both the oracle and the CUDA path consume) and the benchmark (full sizes, device tensors).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch


@dataclass
class AttnWorkload:
    name: str
    num_q_heads: int
    num_kv_heads: int
    head_size: int
    block_size: int
    act_dtype: torch.dtype
    cache_dtype: str
    scale: float
    num_blocks: int
    past_lens: np.ndarray            # i32 [B]
    new_lens: np.ndarray             # i32 [B]
    subsequence_begins: np.ndarray   # i32 [B+1]
    block_indices: np.ndarray        # i32 [sum blocks]
    block_indices_begins: np.ndarray # i32 [B+1]
    max_context_len: int
    seed: int
    score_aggregation_window: Optional[np.ndarray] = None
    rotated_block_indices: Optional[np.ndarray] = None
    rotation_deltas: Optional[np.ndarray] = None
    rotation_trig_lut: Optional[np.ndarray] = None
    extra: dict = field(default_factory=dict)

    @property
    def num_sequences(self) -> int:
        return int(self.past_lens.shape[0])

    @property
    def num_tokens(self) -> int:
        return int(self.new_lens.sum())

    @property
    def scores_len(self) -> int:
        return int((self.past_lens.astype(np.int64) + self.new_lens).sum())

    def kv_token_bytes(self) -> int:
        """Cache bytes one context token occupies over all kv heads, keys + values."""
        per = self.head_size + 8 if self.cache_dtype == "u8" else 2 * self.head_size
        return 2 * self.num_kv_heads * per

    def decode_kv_bytes(self) -> int:
        """Algorithmic KV bytes one step reads for the decode rows: sum (past + 1) * bytes/token."""
        dec = self.new_lens == 1
        return int((self.past_lens[dec].astype(np.int64) + 1).sum()) * self.kv_token_bytes()

    def prefill_flops(self) -> int:
        """4 * Hq * D * sum over chunks of (n * past + n * (n + 1) / 2)."""
        pre = self.new_lens > 1
        n = self.new_lens[pre].astype(np.int64)
        p = self.past_lens[pre].astype(np.int64)
        return int(4 * self.num_q_heads * self.head_size * (n * p + n * (n + 1) // 2).sum())


def rotation_trig_lut(rows: int, block_size: int, head_size: int, theta: float) -> np.ndarray:
    """Row i: cos(i*bs*theta_j) for j < D/2, then -sin(i*bs*theta_j); theta_j = theta^(-2j/D).
    Same closed form as CacheRotationCalculator (cache/cache_eviction.cpp:543-573) laid out as
    pipeline_impl.cpp:273-287 does."""
    j = np.arange(head_size // 2, dtype=np.float64)
    base = np.power(float(theta), -2.0 * j / head_size)
    ang = np.arange(rows, dtype=np.float64)[:, None] * block_size * base[None, :]
    return np.concatenate([np.cos(ang), -np.sin(ang)], axis=1).astype(np.float32)


def _tables(rng: np.random.Generator, past: np.ndarray, new: np.ndarray, bs: int, num_blocks: int):
    nblk = (past.astype(np.int64) + new + bs - 1) // bs
    total = int(nblk.sum())
    if total > num_blocks:
        raise ValueError(f"workload needs {total} blocks, pool has {num_blocks}")
    perm = rng.permutation(num_blocks)[:total].astype(np.int32)
    begins = np.zeros(len(past) + 1, np.int32)
    begins[1:] = np.cumsum(nblk)
    return perm, begins


def make_workload(name: str, *, hq: int, hkv: int, d: int, bs: int, act: torch.dtype, cache: str, past: np.ndarray,
                  new: np.ndarray, num_blocks: int, seed: int, scale: Optional[float] = None) -> AttnWorkload:
    rng = np.random.default_rng(seed)
    past = past.astype(np.int32)
    new = new.astype(np.int32)
    block_indices, bib = _tables(rng, past, new, bs, num_blocks)
    sub = np.zeros(len(past) + 1, np.int32)
    sub[1:] = np.cumsum(new)
    return AttnWorkload(name=name, num_q_heads=hq, num_kv_heads=hkv, head_size=d, block_size=bs, act_dtype=act,
                        cache_dtype=cache, scale=scale if scale is not None else 1.0 / math.sqrt(d),
                        num_blocks=num_blocks, past_lens=past, new_lens=new, subsequence_begins=sub,
                        block_indices=block_indices, block_indices_begins=bib,
                        max_context_len=int((past.astype(np.int64) + new).max()), seed=seed)


def config_tinyllama_decode(num_seqs: int = 8, pool: int = 512, lo: int = 64, hi: int = 2048, seed: int = 1001) -> AttnWorkload:
    """TinyLlama-1.1B attention shape, f16 everything, 8 decode rows, 512-block pool."""
    rng = np.random.default_rng(seed)
    past = rng.integers(lo, hi + 1, size=num_seqs)
    return make_workload("tinyllama_f16_decode", hq=32, hkv=4, d=64, bs=32, act=torch.float16, cache="f16", past=past,
                         new=np.ones(num_seqs, np.int64), num_blocks=pool, seed=seed, scale=0.125)


def config_llama3_8b_decode(num_seqs: int = 64, pool: int = 20000, lo: int = 512, hi: int = 8192, seed: int = 1002) -> AttnWorkload:
    """Llama-3-8B attention shape, bf16 q, u8 by-token cache, 64 decode rows over a 20k-block pool."""
    rng = np.random.default_rng(seed)
    past = rng.integers(lo, hi + 1, size=num_seqs)
    return make_workload("llama3_8b_u8_decode", hq=32, hkv=8, d=128, bs=32, act=torch.bfloat16, cache="u8", past=past,
                         new=np.ones(num_seqs, np.int64), num_blocks=pool, seed=seed)


def config_qwen_mixed(num_prefill: int = 16, chunk: int = 256, prefill_hi: int = 4096, num_decode: int = 240,
                      decode_lo: int = 256, decode_hi: int = 16384, pool: Optional[int] = None, rotated_fraction: float = 0.1,
                      lut_rows: int = 513, theta: float = 1e6, seed: int = 1003, cache: str = "u8") -> AttnWorkload:
    """Qwen2.5-7B attention shape, one mixed step: prefill chunks + decode rows, u8 cache (or `cache` = "f16" / "bf16" with
    activations of the same type), score output (window 8 on prefill rows, 1 on decode rows) and 10 % of the blocks re-rotated."""
    rng = np.random.default_rng(seed)
    past = np.concatenate([rng.integers(0, prefill_hi + 1, size=num_prefill), rng.integers(decode_lo, decode_hi + 1, size=num_decode)])
    new = np.concatenate([np.full(num_prefill, chunk), np.ones(num_decode, np.int64)])
    need = int(((past + new + 31) // 32).sum())
    wl = make_workload("qwen25_7b_mixed", hq=28, hkv=4, d=128, bs=32, act=torch.float16 if cache == "f16" else torch.bfloat16, cache=cache, past=past, new=new,
                       num_blocks=pool or int(need * 1.1) + 1, seed=seed)
    wl.score_aggregation_window = np.concatenate([np.full(num_prefill, 8), np.ones(num_decode, np.int64)]).astype(np.int32)
    # rotate 10 % of every sequence's fully past blocks (blocks the chunk does not write)
    rot = []
    for s in range(wl.num_sequences):
        full = int(wl.past_lens[s]) // wl.block_size
        k = int(full * rotated_fraction)
        if k:
            b0 = wl.block_indices_begins[s]
            rot.append(wl.block_indices[b0 + rng.choice(full, size=k, replace=False)])
    if rot:
        wl.rotated_block_indices = np.concatenate(rot).astype(np.int32)
        wl.rotation_deltas = rng.integers(1, lut_rows, size=len(wl.rotated_block_indices)).astype(np.int32)
        wl.rotation_trig_lut = rotation_trig_lut(lut_rows, wl.block_size, wl.head_size, theta)
    return wl


def config_llama3_70b_decode(num_seqs: int = 1024, lo: int = 1024, hi: int = 32768, pool: Optional[int] = None, seed: int = 1005) -> AttnWorkload:
    """Llama-3-70B attention shape, block size 16, u8 cache, log-uniform context lengths."""
    rng = np.random.default_rng(seed)
    past = np.exp(rng.uniform(math.log(lo), math.log(hi), size=num_seqs)).astype(np.int64)
    need = int(((past + 1 + 15) // 16).sum())
    return make_workload("llama3_70b_u8_decode", hq=64, hkv=8, d=128, bs=16, act=torch.bfloat16, cache="u8", past=past,
                         new=np.ones(num_seqs, np.int64), num_blocks=pool or need + 16, seed=seed)


def random_activations(wl: AttnWorkload, device="cpu", seed_offset: int = 0):
    """q, k, v for the step's new tokens, N(0,1) rounded to the activation dtype."""
    gen = torch.Generator(device=device)
    gen.manual_seed(wl.seed * 7919 + seed_offset)
    t = wl.num_tokens
    mk = lambda h: torch.randn((t, h * wl.head_size), generator=gen, device=device, dtype=torch.float32).to(wl.act_dtype)
    return mk(wl.num_q_heads), mk(wl.num_kv_heads), mk(wl.num_kv_heads)


def past_as_write_step(wl: AttnWorkload) -> AttnWorkload:
    """The same block tables seen as one big chunk that writes tokens 0 .. past-1 of every
    sequence: used to populate a cache through the operator's own write path."""
    past = wl.past_lens
    sub = np.zeros(len(past) + 1, np.int32)
    sub[1:] = np.cumsum(past)
    return AttnWorkload(name=wl.name + "/fill", num_q_heads=wl.num_q_heads, num_kv_heads=wl.num_kv_heads,
                        head_size=wl.head_size, block_size=wl.block_size, act_dtype=wl.act_dtype, cache_dtype=wl.cache_dtype,
                        scale=wl.scale, num_blocks=wl.num_blocks, past_lens=np.zeros_like(past), new_lens=past.copy(),
                        subsequence_begins=sub, block_indices=wl.block_indices, block_indices_begins=wl.block_indices_begins,
                        max_context_len=int(past.max()) if len(past) else 0, seed=wl.seed + 1)


def fill_cache_on_device(op, wl: AttnWorkload, key_cache: torch.Tensor, value_cache: torch.Tensor, max_tokens_per_call: int = 1 << 20) -> None:
    """Writes N(0,1) keys / values for every past token through pa_b200_write_kv, a group of
    sequences at a time so the temporary activations stay small."""
    dev = key_cache.device
    gen = torch.Generator(device=dev)
    gen.manual_seed(wl.seed * 104729 + 17)
    s = 0
    B = wl.num_sequences
    while s < B:
        e, tok = s, 0
        while e < B and (tok == 0 or tok + int(wl.past_lens[e]) <= max_tokens_per_call):
            tok += int(wl.past_lens[e])
            e += 1
        if tok > 0:
            past = wl.past_lens[s:e]
            sub = np.zeros(e - s + 1, np.int32)
            sub[1:] = np.cumsum(past)
            bib = (wl.block_indices_begins[s:e + 1] - wl.block_indices_begins[s]).astype(np.int32)
            bi = wl.block_indices[wl.block_indices_begins[s]:wl.block_indices_begins[e]]
            k = torch.randn((tok, wl.num_kv_heads * wl.head_size), generator=gen, device=dev, dtype=torch.float32).to(wl.act_dtype)
            v = torch.randn((tok, wl.num_kv_heads * wl.head_size), generator=gen, device=dev, dtype=torch.float32).to(wl.act_dtype)
            q = torch.empty((tok, 1), device=dev, dtype=wl.act_dtype)  # unused by the write
            to_dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
            args = op.make_args(q, k, v, q, key_cache, value_cache, to_dev(np.zeros(e - s, np.int32)), to_dev(sub), to_dev(bi),
                                to_dev(bib), wl.scale, int(past.max()))
            op._check(op.lib.pa_b200_write_kv(op._h, __import__("ctypes").byref(args)))
            torch.cuda.synchronize(dev)
        s = e


# ---- Sampler workloads ---------------------------------------------------------------------------
def sampler_history(rng: np.random.Generator, rows: int, vocab: int, generated_len: int, prompt_len: int = 0):
    """CSR history of distinct ids per row for the Sampler step: prompt ids (flag 1), generated ids
    with their counts (flag 2), as `(offsets int64, ids int32, meta uint32)`."""
    offs, ids, meta = [0], [], []
    for _ in range(rows):
        gen = rng.integers(0, vocab, size=generated_len)
        prompt = rng.integers(0, vocab, size=prompt_len)
        uniq = {}
        for t in prompt:
            uniq.setdefault(int(t), [0, 0])[0] = 1
        for t in gen:
            uniq.setdefault(int(t), [0, 0])[1] += 1
        for t in sorted(uniq):
            flag = (1 if uniq[t][0] else 0) | (2 if uniq[t][1] else 0)
            ids.append(t)
            meta.append((uniq[t][1] << 3) | flag)
        offs.append(len(ids))
    return np.array(offs, np.int64), np.array(ids, np.int32), np.array(meta, np.uint32)


def config_qwen_sampler(rows: int = 256, vocab: int = 151936, greedy: bool = False, history: int = 1024, seed: int = 1004,
                        mode: Optional[str] = None):
    """Qwen2.5 vocabulary, 256 rows: logits N(0, 4) with 8 spikes of +15 per row, T 0.7, top_k 50,
    top_p 0.9, repetition 1.1, presence 0.2, frequency 0.1 over a 1024-token generated history.
    `mode` selects the other paths on the same logits: "top_p" (T 1, top_p 0.95 over the whole vocabulary, no
    penalties - the sampling a vLLM-style throughput benchmark uses) and "temperature" (T 0.8 only).
    Returns (logits f32 [rows, vocab], packed row parameters, history)."""
    from . import _sampler_abi as SA
    rng = np.random.default_rng(seed)
    logits = (rng.standard_normal((rows, vocab)) * 2.0).astype(np.float32)
    for r in range(rows):
        logits[r, rng.choice(vocab, size=8, replace=False)] += np.float32(15.0)
    hist = sampler_history(rng, rows, vocab, history)
    par = np.zeros(rows, dtype=np.dtype(SA.ROW_DTYPE))
    par["logits_row"] = np.arange(rows)
    par["top_k"] = SA.TOP_K_OFF if greedy else 50
    par["do_sample"] = 0 if greedy else 1
    par["temperature"] = 1.0 if greedy else 0.7
    par["top_p"] = 1.0 if greedy else 0.9
    par["repetition_penalty"] = 1.1
    par["presence_penalty"] = 0.2
    par["frequency_penalty"] = 0.1
    par["rand_u"] = np.random.default_rng(seed + 1).random(rows, dtype=np.float32)
    if mode in ("top_p", "temperature"):
        par["top_k"] = SA.TOP_K_OFF
        par["temperature"] = 1.0 if mode == "top_p" else 0.8
        par["top_p"] = 0.95 if mode == "top_p" else 1.0
        par["repetition_penalty"] = 1.0
        par["presence_penalty"] = 0.0
        par["frequency_penalty"] = 0.0
        hist = None
    return logits, par, hist
