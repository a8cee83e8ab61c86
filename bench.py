#!/usr/bin/env python
"""Benchmark of the paged-attention decode step (the headline metric: KV GB/s of one
PagedAttention decode step, as a fraction of the measured HBM peak) and, in the same line, of the
other steps the north star names.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Headline step: one PagedAttention operator call over the whole decode batch: write the new token's
K/V into the paged cache, split-K attention over every sequence's block table, merge.
Workload: Llama-3-8B attention shape, 64 sequences per GPU, past_lens U[512, 8192], u8 by-token KV
cache scattered over a 20k-block pool, bf16 q - seeded synthetic data.  The KV bytes touched per step
(~600 MB) exceed the 126 MB L2, so consecutive steps cannot be served from L2.

Prints ONE JSON line.  `value` is whole-job KV GB/s with every input resident in HBM (the K timed
steps); `repeats` holds the spread of further regions of K steps.  `e2e` is the same metric through
the host-tensor entry point (pa_b200_forward_host) with the step's q/k/v/metadata copied
host->device and the output device->host inside the timed region.  `secondary` holds, measured in
the same process: the sharded engine step (1024 sequences over all ranks: decode, full-vocabulary
sampler, all-gather of the ids) at every N, and at N = 1 the Sampler steps, the mixed step and the
tensor-core rate of prefill chunks.  `--workload NAME` prints one of those alone.
`--impl reference` times the CPU restatement of the operator (the reference's own operator lives in
the OpenVINO runtime, which is not available) on the host cores over a bounded sample.
"""
from __future__ import annotations

import argparse
import ctypes as C
import hashlib
import json
import math
import os
import re
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "paged_attn_decode_kv_gbps"
UNIT = "GB/s"
SAMPLER_WORKLOADS = ("qwen25_sampler_topk", "qwen25_sampler_greedy", "qwen25_sampler_topp", "qwen25_sampler_temperature")


def load_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm": float(d["hbm_gbs"]), "bf16": float(d.get("bf16_tflops_sustained", 1400.0)), "source": "measured"}
    return {"hbm": 6650.0, "bf16": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def build_workload(name: str, rank: int):
    from openvino_genai_b200 import workloads
    if name == "llama3_8b_u8_decode":
        return workloads.config_llama3_8b_decode(seed=1002 + 97 * rank)
    if name == "tinyllama_f16_decode":
        return workloads.config_tinyllama_decode(seed=1001 + 97 * rank)
    if name == "llama3_70b_u8_decode":
        return workloads.config_llama3_70b_decode(seed=1005 + 97 * rank)
    raise SystemExit(f"unknown workload {name}")


def config_of(wl, n_gpus: int) -> dict:
    return {"workload": wl.name, "num_q_heads": wl.num_q_heads, "num_kv_heads": wl.num_kv_heads, "head_size": wl.head_size,
            "block_size": wl.block_size, "kv_cache": wl.cache_dtype + (" by-token asymmetric" if wl.cache_dtype == "u8" else ""),
            "sequences_per_gpu": wl.num_sequences, "past_lens": f"U[{int(wl.past_lens.min())},{int(wl.past_lens.max())}]",
            "pool_blocks": wl.num_blocks, "parallelism": f"sequences and KV pools sharded over {n_gpus} rank(s), no data-path collective",
            "l2_policy": "KV bytes per step exceed L2 (inputs larger than L2)"}


class Env:
    """Process-wide state of one bench run: ranks, device, process group."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        import __graft_entry__ as entry
        self.torch, self.dist = torch, dist
        self.pkg = entry.load_package()
        self.pkg.load_library()  # fails loudly when the CUDA extension is missing
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.peaks = load_peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, values):
        t = self.torch.tensor(list(values), dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.cpu()]

    def sum_over_ranks(self, values):
        t = self.torch.tensor(list(values), dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return [float(x) for x in t.cpu()]

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
def cpu_sample_workload(wl_name: str, target_mb: float = 300.0):
    """The first sequences of the seeded workload up to ~target_mb of KV, with host data and a cache the
    CPU restatement filled: what the CPU legs time and what the parity field compares against."""
    import torch
    import __graft_entry__ as entry
    entry.load_package()
    from oracle import pa_oracle
    from tests import pa_harness as H
    from openvino_genai_b200 import workloads
    full = build_workload(wl_name, 0)
    per_tok = full.kv_token_bytes()
    take, acc = 0, 0
    while take < full.num_sequences and (take == 0 or acc + (int(full.past_lens[take]) + 1) * per_tok <= target_mb * 1e6):
        acc += (int(full.past_lens[take]) + 1) * per_tok
        take += 1
    wl = workloads.make_workload(full.name, hq=full.num_q_heads, hkv=full.num_kv_heads, d=full.head_size, bs=full.block_size,
                                 act=full.act_dtype, cache=full.cache_dtype, past=full.past_lens[:take].astype(np.int64),
                                 new=np.ones(take, np.int64), num_blocks=int(((full.past_lens[:take] + 1 + full.block_size - 1) // full.block_size).sum()) + 2,
                                 seed=full.seed, scale=full.scale)
    data = H.make_host_data(wl)
    q, k, v, fill, pk, pv = data
    desc = H.desc_of(wl)
    n = wl.num_blocks * H.block_bytes(wl)
    kc, vc = np.zeros(n, np.uint8), np.zeros(n, np.uint8)
    dummy = torch.zeros((fill.num_tokens, 1), dtype=wl.act_dtype)
    assert pa_oracle.write_kv(desc, H.host_args(fill, dummy, pk, pv, dummy, kc, vc, with_eviction=False)) == 0
    out = torch.zeros_like(q)
    args = H.host_args(wl, q, k, v, out, kc, vc)
    assert pa_oracle.write_kv(desc, args) == 0
    sample = f"first {take} of {full.num_sequences} sequences of the same seeded workload ({wl.decode_kv_bytes() / 1e6:.1f} MB of KV per step), attention only"
    # `args` holds raw addresses: every buffer it names stays referenced by the returned record
    return {"wl": wl, "full": full, "data": data, "desc": desc, "args": args, "out": out, "sample": sample, "buffers": (q, k, v, kc, vc, out)}


def cpu_reference_leg(wl_name: str, steps: int, warmup: int):
    """Times the CPU restatement of the operator (attention only, cache already written) on the bounded sample."""
    from oracle import pa_oracle
    smp = cpu_sample_workload(wl_name)
    cores = pa_oracle.hardware_threads()
    for _ in range(warmup):
        pa_oracle.attend(smp["desc"], smp["args"], cores)
    t0 = time.perf_counter()
    for _ in range(steps):
        assert pa_oracle.attend(smp["desc"], smp["args"], cores) == 0
    dt = (time.perf_counter() - t0) / max(steps, 1)
    gbps = smp["wl"].decode_kv_bytes() / dt / 1e9
    return gbps, dt * 1e3, cores, smp


def parity_against_oracle(smp) -> float:
    """The CUDA operator on the CPU leg's sample (same host data, cache filled through the CUDA write path):
    largest |difference| of the attention output relative to the largest reference magnitude."""
    from tests import pa_harness as H
    res = H.run_gpu(smp["wl"], smp["data"])
    if res["status"]:
        raise SystemExit(f"device status word {res['status']:#x} in the parity step")
    return H.rel_err(res["out_gpu"], smp["out"].float().numpy())


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    gbps, ms, cores, smp = cpu_reference_leg(args.workload, args.steps, args.warmup)
    line = {"metric": METRIC, "value": round(gbps, 4), "unit": UNIT, "impl": "reference", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config_of(smp["full"], args.gpus),
            "cpu_baseline": {"value": round(gbps, 4), "unit": UNIT, "cores": cores, "kind": "port", "sample": smp["sample"]},
            "e2e": {"value": round(gbps, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement of the operator contract (the reference's operator lives in the OpenVINO runtime, unavailable here)"}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
def stored_traffic(wl_name: str):
    """DRAM bytes per launch of the decode kernel from the committed ncu summary - a stored capture, not a value of
    this run: it is only reported while the kernel source still has the hash the summary was made from."""
    tp = ROOT / "profiles" / "decode_u8_llama3_8b.md"
    if wl_name != "llama3_8b_u8_decode" or not tp.exists():
        return None, None
    text = tp.read_text()
    m = re.search(r"dram_bytes_per_launch:\s*(\d+)", text)
    h = re.search(r"kernel_source_sha16:\s*([0-9a-f]{16})", text)
    src = ROOT / "openvino.genai_b200" / "csrc" / "pa_decode_shared.cu"
    now = hashlib.sha256(src.read_bytes()).hexdigest()[:16]
    if not m or not h or h.group(1) != now:
        return None, "no ncu capture of the current kernel source is committed"
    return int(m.group(1)), "profiles/decode_u8_llama3_8b.md (stored ncu capture of this kernel source, not of this run)"


def measure_headline(env: Env, args) -> dict:
    torch = env.torch
    from openvino_genai_b200 import workloads
    dev, rank, world = env.dev, env.rank, env.world
    wl = build_workload(args.workload, rank)
    op = env.pkg.PagedAttentionExtension(wl.num_q_heads, wl.num_kv_heads, wl.head_size, wl.block_size, wl.act_dtype, wl.cache_dtype, env.local)
    kc, vc = op.allocate_cache(wl.num_blocks, fill=0)
    workloads.fill_cache_on_device(op, wl, kc, vc)
    q, k, v = workloads.random_activations(wl, dev)
    out = torch.empty_like(q)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    meta = [t(wl.past_lens), t(wl.subsequence_begins), t(wl.block_indices), t(wl.block_indices_begins)]
    stream = torch.cuda.Stream(dev)
    torch.cuda.synchronize(dev)
    dargs = op.make_args(q, k, v, out, kc, vc, *meta, wl.scale, wl.max_context_len, stream=stream.cuda_stream)
    op._check(op.lib.pa_b200_reserve(op._h, wl.num_tokens, wl.num_sequences, wl.max_context_len, 0, len(wl.block_indices)))

    def region(steps):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        env.barrier()
        ev0.record(stream)
        for _ in range(steps):
            op.forward_args(dargs)
        ev1.record(stream)
        env.barrier()
        return ev0.elapsed_time(ev1)

    # ---- device-resident steps: the K timed steps, then more regions of K steps for the spread ----------
    for _ in range(args.warmup):
        op.forward_args(dargs)
    env.barrier()
    launches0 = op.launch_count()
    sampler = ClockSampler(env.local)
    if rank == 0:
        sampler.start()
    ms_total = region(args.steps)
    launches = op.launch_count() - launches0
    repeats = [region(args.steps) / args.steps for _ in range(args.repeats)]
    clocks = sampler.stop() if rank == 0 else None
    # the decode kernel alone, in a short loop of its own (event pairs around the kernel inside the operator)
    op._check(op.lib.pa_b200_set_kernel_timing(op._h, 1))
    for _ in range(20):
        op.forward_args(dargs)
    torch.cuda.synchronize(dev)
    op._check(op.lib.pa_b200_set_kernel_timing(op._h, 0))
    ktot, kcnt = C.c_double(0), C.c_int64(0)
    op._check(op.lib.pa_b200_get_kernel_timing(op._h, C.byref(ktot), C.byref(kcnt)))
    status = op.device_status()
    if status:
        raise SystemExit(f"device status word {status:#x} after the timed region")

    # ---- end to end through the host-tensor entry point -------------------------------------------
    hq, hk_, hv = (x.cpu().pin_memory() for x in (q, k, v))
    hout = torch.empty_like(hq).pin_memory()
    hargs = op.make_args(hq, hk_, hv, hout, kc, vc, wl.past_lens, wl.subsequence_begins, wl.block_indices, wl.block_indices_begins,
                         wl.scale, wl.max_context_len, stream=stream.cuda_stream)
    h2d = int(hq.numel() * hq.element_size() + 2 * hk_.numel() * hk_.element_size() +
              4 * (len(wl.past_lens) + len(wl.subsequence_begins) + len(wl.block_indices) + len(wl.block_indices_begins)))
    d2h = int(hout.numel() * hout.element_size())
    for _ in range(max(args.warmup, 1)):
        op.forward_args(hargs, host=True)
    env.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        op.forward_args(hargs, host=True)
    e1.record(stream)
    env.barrier()
    ms_e2e_total = e0.elapsed_time(e1)
    # the decode kernel hands tiles to its warps dynamically, so the order of its partial sums - and with it the last bits of
    # the output - differs between launches: the host-buffer call is compared with the device call at bf16 resolution
    same = torch.allclose(hout.to(dev).float(), out.float(), rtol=2e-2, atol=2e-3)

    # ---- reduce over ranks ------------------------------------------------------------------------
    kv_bytes = wl.decode_kv_bytes()
    ms_total, ms_e2e_total, kernel_ms, *rep = env.max_over_ranks([ms_total, ms_e2e_total, ktot.value / max(kcnt.value, 1)] + repeats)
    total_bytes, total_seqs, total_launches = env.sum_over_ranks([float(kv_bytes), float(wl.num_sequences), float(launches)])
    del kc, vc, op
    torch.cuda.empty_cache()
    if rank != 0:
        return {}
    peak = env.peaks["hbm"]
    ms_step = ms_total / args.steps
    value = total_bytes / (ms_step * 1e-3) / 1e9
    e2e_value = total_bytes / (ms_e2e_total / args.steps * 1e-3) / 1e9
    achieved = kv_bytes / (kernel_ms * 1e-3) / 1e9
    traffic, traffic_source = stored_traffic(wl.name)
    line = {"metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 mma / f32 accumulate",
            "data": "synthetic", "config": config_of(wl, world),
            "tokens_per_s": round(total_seqs / (ms_step * 1e-3), 1),
            "hbm_peak_frac_step": round(value / world / peak, 4),
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                         "traffic": traffic, "traffic_source": traffic_source, "kernel": "decode_shared_kernel (paged decode, one CTA per SM, tiles handed to its warps from shared-memory counters)", "kernel_ms": round(kernel_ms, 4),
                         "kernel_timed": "20 launches in a loop of their own, CUDA events around the kernel on its stream",
                         "algorithmic_bytes_per_launch": kv_bytes, "peak_source": env.peaks["source"]},
            "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": round(ms_e2e_total / args.steps, 4), "matches_device_path": bool(same)},
            "gpu_launches": int(total_launches), "clocks": clocks}
    if rep:
        line["repeats"] = {"regions": len(rep), "steps_per_region": args.steps, "ms_per_step_median": round(statistics.median(rep), 4),
                           "ms_per_step_min": round(min(rep), 4), "ms_per_step_max": round(max(rep), 4),
                           "value_median": round(total_bytes / (statistics.median(rep) * 1e-3) / 1e9, 2)}
    return line


# ------------------------------------------------------------------------------------------------
SECONDARY = {
    # name: (constructor keyword arguments of workloads.config_qwen_mixed, keep scores, what it is)
    "qwen25_7b_mixed": (dict(), True, "16 prefill chunks of 256 + 240 decode rows, score output, 10 % of the blocks re-rotated"),
    "qwen25_7b_prefill": (dict(num_decode=0, rotated_fraction=0.0), False, "16 prefill chunks of 256 tokens, past U[0,4096]"),
    "qwen25_7b_prefill_large": (dict(num_prefill=64, chunk=512, prefill_hi=8192, num_decode=0, rotated_fraction=0.0), False,
                                "64 prefill chunks of 512 tokens, past U[0,8192]"),
    "qwen25_7b_prefill_large_f16": (dict(num_prefill=64, chunk=512, prefill_hi=8192, num_decode=0, rotated_fraction=0.0, cache="f16"), False,
                                    "64 prefill chunks of 512 tokens, past U[0,8192], f16 cache and activations"),
    "qwen25_7b_prefill_large_bf16": (dict(num_prefill=64, chunk=512, prefill_hi=8192, num_decode=0, rotated_fraction=0.0, cache="bf16"), False,
                                     "64 prefill chunks of 512 tokens, past U[0,8192], bf16 cache and activations"),
}


def measure_pa_step(env: Env, name: str, steps: int, warmup: int) -> dict:
    """The mixed step (prefill chunks + decode rows + score output + rotation) and prefill-only steps that
    exercise the tcgen05 kernel: step time, and for prefill-only workloads the tensor-core rate of the whole
    step against the measured sustained bf16 peak."""
    torch = env.torch
    from openvino_genai_b200 import workloads
    kw, keep_scores, what = SECONDARY[name]
    dev = env.dev
    wl = workloads.config_qwen_mixed(**kw)
    if not keep_scores:
        wl.score_aggregation_window = None
    op = env.pkg.PagedAttentionExtension(wl.num_q_heads, wl.num_kv_heads, wl.head_size, wl.block_size, wl.act_dtype, wl.cache_dtype, env.local)
    kc, vc = op.allocate_cache(wl.num_blocks, fill=0)
    workloads.fill_cache_on_device(op, wl, kc, vc)
    q, k, v = workloads.random_activations(wl, dev)
    out = torch.empty_like(q)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev) if a is not None else None
    scores = torch.zeros(wl.scores_len, dtype=torch.float32, device=dev) if wl.score_aggregation_window is not None else None
    stream = torch.cuda.Stream(dev)
    torch.cuda.synchronize(dev)
    dargs = op.make_args(q, k, v, out, kc, vc, t(wl.past_lens), t(wl.subsequence_begins), t(wl.block_indices), t(wl.block_indices_begins),
                         wl.scale, wl.max_context_len, t(wl.score_aggregation_window), scores, t(wl.rotated_block_indices),
                         t(wl.rotation_deltas), t(wl.rotation_trig_lut), stream=stream.cuda_stream)
    for _ in range(max(warmup, 3)):
        op.forward_args(dargs)
    torch.cuda.synchronize(dev)
    launches0 = op.launch_count()
    sampler = ClockSampler(env.local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        op.forward_args(dargs)
    e1.record(stream)
    torch.cuda.synchronize(dev)
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / steps
    status = op.device_status()
    if status:
        raise SystemExit(f"device status word {status:#x} after the timed region")
    flops = wl.prefill_flops()
    res = {"metric": "pa_step_ms", "value": round(ms, 4), "unit": "ms", "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3),
           "ms_per_step": round(ms, 4), "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
           "dtype": ("bf16" if kw.get("cache") == "bf16" else "f16") + " tcgen05 / f32 accumulate", "data": "synthetic",
           "config": {"workload": name, "what": what, "tokens": int(wl.num_tokens), "sequences": int(wl.num_sequences),
                      "kv_cache": {"f16": "f16", "bf16": "bf16"}.get(kw.get("cache"), "u8 by-token asymmetric"), "prefill_gflop": round(flops / 1e9, 1),
                      "decode_kv_mb": round(wl.decode_kv_bytes() / 1e6, 1), "l2_policy": "KV bytes per step exceed L2"},
           "gpu_launches": int(op.launch_count() - launches0), "clocks": clocks}
    if wl.decode_kv_bytes() == 0 and flops:
        peak = env.peaks["bf16"]
        achieved = flops / (ms * 1e-3) / 1e12
        res["roofline"] = {"bound": "tensor", "achieved": round(achieved, 1), "peak": peak, "unit": "TFLOP/s", "frac": round(achieved / peak, 4),
                           "traffic": None, "kernel": "prefill_tc_kernel (whole step: cache write + attention)",
                           "algorithmic_flops_per_launch": int(flops), "peak_source": "bf16_tflops_sustained, " + env.peaks["source"]}
    del kc, vc, op
    torch.cuda.empty_cache()
    return res


def measure_sampler(env: Env, name: str, steps: int, warmup: int) -> dict:
    """One Sampler step over 256 x 151936 f32 logits, resident on the device and restored from a pristine copy
    before every step (the step applies the penalties in place).  Microseconds per step and the HBM roofline
    of one mandatory read of the logits."""
    torch = env.torch
    from openvino_genai_b200 import workloads, sampler as sampler_mod
    dev = env.dev
    greedy = name == "qwen25_sampler_greedy"
    mode = {"qwen25_sampler_topp": "top_p", "qwen25_sampler_temperature": "temperature"}.get(name)
    logits_h, par, hist = workloads.config_qwen_sampler(greedy=greedy, mode=mode)
    sampling = {"top_p": "T 1, top_p 0.95 over the whole vocabulary", "temperature": "T 0.8 over the whole vocabulary"}.get(
        mode, "greedy + penalties" if greedy else "top_k 50, T 0.7, top_p 0.9, repetition 1.1, presence 0.2, frequency 0.1")
    pristine = torch.from_numpy(logits_h).to(dev)
    work = pristine.clone()
    smp = sampler_mod.SamplerStep(env.local)
    staged = smp.stage(par, hist)
    stream = torch.cuda.Stream(dev)
    times = []
    sampler = ClockSampler(env.local)
    sampler.start()
    launches0 = smp.launch_count()
    with torch.cuda.stream(stream):
        for it in range(max(warmup, 3) + steps):
            work.copy_(pristine)      # also evicts the previous step's logits from L2 (311 MB moved)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            smp.step(work, staged, stream=stream.cuda_stream)
            e1.record(stream)
            stream.synchronize()
            if it >= max(warmup, 3):
                times.append(e0.elapsed_time(e1) * 1e3)
    clocks = sampler.stop()
    launches = smp.launch_count() - launches0
    us = statistics.median(times)
    peak = env.peaks["hbm"]
    achieved = logits_h.nbytes / (us * 1e-6) / 1e9
    res = {"metric": "sampler_step_us", "value": round(us, 1), "unit": "us", "n_gpus": 1, "steps": steps, "warmup": max(warmup, 3),
           "ms_per_step": round(us / 1e3, 4), "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": name, "rows": int(logits_h.shape[0]), "vocab": int(logits_h.shape[1]),
                      "sampling": sampling, "history": "none" if hist is None else "1024 generated ids per row", "l2_policy": "logits rewritten from a pristine copy before every step"},
           "min_us": round(min(times), 1), "max_us": round(max(times), 1),
           "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4), "traffic": None,
                        "kernel": "sampler_kernel (+ sampler_exact_kernel for full-vocabulary rows)", "algorithmic_bytes_per_launch": int(logits_h.nbytes),
                        "peak_source": env.peaks["source"]},
           "gpu_launches": int(launches), "clocks": clocks}
    smp.close()
    del pristine, work
    torch.cuda.empty_cache()
    return res


def measure_engine_step(env: Env, steps: int, warmup: int) -> dict:
    """One engine step of a sharded batch: Llama-3-70B attention shape, 1024 sequences with log-uniform contexts
    split over all ranks (balanced by context length), u8 cache with block size 16; paged decode, then the
    Sampler over [rows, 128256] f32 logits (T = 1, top_p 0.95: the full-vocabulary path) writing its ids
    straight into this rank's row of the exchange buffer, then ONE in-place ncclAllGather issued by the C++
    host layer on the same stream.  Strong scaling: whole-job tokens per second."""
    torch, dist = env.torch, env.dist
    from openvino_genai_b200 import workloads, sharding, sampler as sampler_mod, _sampler_abi as SA
    world, rank, dev = env.world, env.rank, env.dev
    total_seqs, vocab = 1024, 128256
    rng = np.random.default_rng(1005)
    past_all = np.exp(rng.uniform(math.log(1024), math.log(32768), size=total_seqs)).astype(np.int64)
    shards = sharding.shard_sequences(past_all + 1, world)
    mine = shards[rank]
    cap = max(len(x) for x in shards)
    past = past_all[mine]
    need = int(((past + 1 + 15) // 16).sum())
    wl = workloads.make_workload("llama3_70b_u8_step", hq=64, hkv=8, d=128, bs=16, act=torch.bfloat16, cache="u8", past=past,
                                 new=np.ones(len(past), np.int64), num_blocks=need + 16, seed=1005 + 97 * rank)
    op = env.pkg.PagedAttentionExtension(wl.num_q_heads, wl.num_kv_heads, wl.head_size, wl.block_size, wl.act_dtype, wl.cache_dtype, env.local)
    kc, vc = op.allocate_cache(wl.num_blocks, fill=0)
    workloads.fill_cache_on_device(op, wl, kc, vc)
    q, k, v = workloads.random_activations(wl, dev)
    out = torch.empty_like(q)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    stream = torch.cuda.Stream(dev)
    dargs = op.make_args(q, k, v, out, kc, vc, t(wl.past_lens), t(wl.subsequence_begins), t(wl.block_indices), t(wl.block_indices_begins),
                         wl.scale, wl.max_context_len, stream=stream.cuda_stream)
    n = len(past)
    gen = torch.Generator(device=dev)
    gen.manual_seed(4242 + rank)
    logits = torch.randn((n, vocab), generator=gen, device=dev, dtype=torch.float32) * 2.0
    rows = np.zeros(n, dtype=np.dtype(SA.ROW_DTYPE))
    rows["logits_row"] = np.arange(n)
    rows["top_k"] = SA.TOP_K_OFF
    rows["do_sample"] = 1
    rows["temperature"] = 1.0
    rows["top_p"] = 0.95
    rows["repetition_penalty"] = 1.0
    rows["rand_u"] = np.random.default_rng(77 + rank).random(n, dtype=np.float32)
    smp = sampler_mod.SamplerStep(env.local)
    staged = smp.stage(rows)
    exchange = sharding.TokenExchange(dev, cap) if world > 1 else None
    token_row = exchange.local_row if exchange else None
    torch.cuda.synchronize(dev)

    def step(ev=None):
        op.forward_args(dargs)
        if ev:
            ev[0].record(stream)
        tok, _ = smp.step(logits, staged, stream=stream.cuda_stream, out_tokens=token_row)
        if ev:
            ev[1].record(stream)
        if exchange:
            return exchange.all_gather(n, stream.cuda_stream)
        return tok

    for _ in range(max(warmup, 3)):
        ids = step()
    env.barrier()
    if exchange:
        got = ids.cpu().numpy()
        for r in range(world):
            assert (got[r, :len(shards[r])] >= 0).all() and (got[r, len(shards[r]):] == -1).all(), "a sampled id is missing after the all-gather"
    else:
        assert int((ids < 0).sum().item()) == 0
    launches0 = op.launch_count() + smp.launch_count()
    sampler = ClockSampler(env.local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    env.barrier()
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    env.barrier()
    clocks = sampler.stop() if rank == 0 else None
    launches = op.launch_count() + smp.launch_count() - launches0 + (steps if exchange else 0)
    # where the step's time goes: a few more steps with events between the operator, the sampler and the exchange
    att, sam, exc = [], [], []
    for _ in range(5):
        p = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        p[0].record(stream)
        step((p[1], p[2]))
        p[3].record(stream)
        env.barrier()
        att.append(p[0].elapsed_time(p[1])); sam.append(p[1].elapsed_time(p[2])); exc.append(p[2].elapsed_time(p[3]))
    ms_total, a_ms, s_ms, x_ms = env.max_over_ranks([e0.elapsed_time(e1), statistics.median(att), statistics.median(sam), statistics.median(exc)])
    kv_total, launches_total, kv_max, logit_max = env.sum_over_ranks([float(wl.decode_kv_bytes()), float(launches), 0.0, 0.0])
    kv_slowest, logits_slowest = env.max_over_ranks([float(wl.decode_kv_bytes()), float(n * vocab * 4)])
    if exchange:
        exchange.close()
    smp.close()
    del kc, vc, op, logits
    torch.cuda.empty_cache()
    if rank != 0:
        return {}
    ms = ms_total / steps
    peak = env.peaks["hbm"]
    return {"metric": "engine_step_tokens_per_s", "value": round(total_seqs / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": max(warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 mma / f32 accumulate; f32 sampler", "data": "synthetic",
            "config": {"workload": "llama3_70b_u8_step", "sequences_total": total_seqs, "contexts": "log-uniform [1024, 32768]",
                       "kv_cache": "u8 by-token asymmetric, block 16", "vocab": vocab, "sampler": "T 1, top_p 0.95 (full vocabulary)",
                       "exchange": "one in-place ncclAllGather of [world, cap] int64 ids from the C++ host layer, on the sampler's stream" if world > 1 else "none (one rank)",
                       "parallelism": f"sequences balanced by context length over {world} rank(s)", "l2_policy": "KV bytes per step exceed L2"},
            "kv_gbps": round(kv_total / (ms * 1e-3) / 1e9, 1),
            "attention_ms": round(a_ms, 4), "attention_hbm_frac": round(kv_slowest / (a_ms * 1e-3) / 1e9 / peak, 4),
            "sampler_ms": round(s_ms, 4), "sampler_hbm_frac_one_read": round(logits_slowest / (s_ms * 1e-3) / 1e9 / peak, 4),
            "allgather_ms": round(x_ms, 4), "parts": "max over ranks of the median of 5 separately timed steps",
            "gpu_launches": int(launches_total), "clocks": clocks}


def print_line(line: dict):
    if line:
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=30, help="further regions of --steps steps, for the spread of the headline")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama3_8b_u8_decode")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="headline only")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    args.warmup = max(args.warmup, 3)
    env = Env()
    try:
        if args.workload in SAMPLER_WORKLOADS:
            if env.world > 1:
                raise SystemExit("the sampler workloads run on one GPU")
            print_line(measure_sampler(env, args.workload, args.steps, args.warmup))
        elif args.workload == "llama3_70b_u8_step":
            print_line(measure_engine_step(env, args.steps, args.warmup))
        elif args.workload in SECONDARY:
            if env.world > 1:
                raise SystemExit("the secondary workloads run on one GPU")
            print_line(measure_pa_step(env, args.workload, args.steps, args.warmup))
        else:
            line = measure_headline(env, args)
            if not args.no_secondary and args.workload == "llama3_8b_u8_decode":
                keep = lambda d, keys: {k: d[k] for k in keys if k in d}
                sec = {}
                eng = measure_engine_step(env, 10, 3)
                if env.rank == 0:
                    sec["engine_step"] = keep(eng, ("metric", "value", "unit", "ms_per_step", "scaling", "kv_gbps", "attention_ms", "attention_hbm_frac", "sampler_ms",
                                                    "sampler_hbm_frac_one_read", "allgather_ms", "gpu_launches", "config"))
                if env.world == 1:
                    for key, name in (("sampler_topk", "qwen25_sampler_topk"), ("sampler_topp", "qwen25_sampler_topp")):
                        r = measure_sampler(env, name, 20, 3)
                        sec[key + "_us"] = r["value"]
                        sec[key] = {"min_us": r["min_us"], "max_us": r["max_us"], "hbm_frac_one_read": r["roofline"]["frac"], "sampling": r["config"]["sampling"]}
                    r = measure_pa_step(env, "qwen25_7b_mixed", 20, 3)
                    sec["mixed_step_ms"] = r["value"]
                    sec["mixed_step"] = keep(r["config"], ("what", "tokens", "prefill_gflop", "decode_kv_mb"))
                    r = measure_pa_step(env, "qwen25_7b_prefill_large", 10, 3)
                    sec["prefill_tensor_frac"] = r["roofline"]["frac"]
                    sec["prefill"] = {"tflops": r["roofline"]["achieved"], "peak_tflops": r["roofline"]["peak"], "ms_per_step": r["value"], "what": r["config"]["what"]}
                    r = measure_pa_step(env, "qwen25_7b_prefill", 20, 3)
                    sec["prefill_tensor_frac_16x256"] = r["roofline"]["frac"]
                    for cache in ("f16", "bf16"):   # the same 64 chunks over the 16-bit caches (activations of the cache's type)
                        r = measure_pa_step(env, "qwen25_7b_prefill_large_" + cache, 10, 3)
                        sec["prefill_tensor_frac_" + cache] = r["roofline"]["frac"]
                if env.rank == 0:
                    line["secondary"] = sec
            if env.rank == 0 and env.world == 1 and not args.no_cpu_baseline:
                gbps, ms, cores, smp = cpu_reference_leg(args.workload, 2, 1)
                line["cpu_baseline"] = {"value": round(gbps, 4), "unit": UNIT, "cores": cores, "kind": "port", "sample": smp["sample"]}
                line["parity_max_rel_err"] = round(parity_against_oracle(smp), 6)
                line["parity"] = "CUDA operator vs the CPU restatement on the cpu_baseline sample, max |diff| / max |reference|; bf16 output; the restatement itself is unpinned (no reference operator source)"
            print_line(line)
    finally:
        env.close()


if __name__ == "__main__":
    main()
