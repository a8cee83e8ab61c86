"""The allocation-free decode entry point (pa_b200_decode_step_static) against the regular one.

Some callers cannot allocate device memory at the point where they run the operator (code inside
an allocator callback, a server that handed out all device memory at start-up, a loop that must
not take the allocator's lock).  For them the decode step's scratch is a fixed device array inside
the library.  This test calls that entry point through the C ABI twice in a row - the array keeps
the first call's contents, so the second call checks that everything that must start clean is
rewritten - and compares each output with pa_b200_forward on the same inputs.
The file sorts last on purpose: a failure here stops a `-x` run only after every other test ran."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests import pa_harness as H

pytestmark = pytest.mark.gpu


def _device_inputs(wl, data, dev):
    q, k, v, fill, pk, pv = data
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    return {"q": q.to(dev), "k": k.to(dev), "v": v.to(dev), "past_lens": t(wl.past_lens), "sub": t(wl.subsequence_begins),
            "bi": t(wl.block_indices), "bib": t(wl.block_indices_begins)}


def _filled_cache(op, wl, data, dev):
    q, k, v, fill, pk, pv = data
    kc, vc = op.allocate_cache(wl.num_blocks, fill=0)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    dummy = torch.zeros((fill.num_tokens, 1), dtype=wl.act_dtype, device=dev)
    args = op.make_args(dummy, pk.to(dev), pv.to(dev), dummy, kc, vc, t(fill.past_lens), t(fill.subsequence_begins),
                        t(fill.block_indices), t(fill.block_indices_begins), fill.scale, fill.max_context_len)
    op._check(op.lib.pa_b200_write_kv(op._h, C.byref(args)))
    torch.cuda.synchronize(dev)
    return kc, vc


@pytest.mark.parametrize("cache,act,hq,hkv,d,bs", [
    ("u8", torch.bfloat16, 32, 8, 128, 32),
    ("f16", torch.float16, 32, 8, 128, 32),
    ("f16", torch.float16, 16, 4, 64, 16),      # the 16-token block / 64-dim instantiation
    ("u8", torch.bfloat16, 40, 2, 128, 32),     # 20 query heads per KV head: two head tiles, the second ragged
])
def test_static_scratch_entry_matches_regular_entry_twice(cache, act, hq, hkv, d, bs):
    dev = torch.device("cuda", 0)
    tol = 1e-2 if cache == "u8" else 2e-3
    # two different steps, the second shorter than the first so stale partials would show
    geo = dict(hq=hq, hkv=hkv, d=d, bs=bs, act=act, cache=cache)
    steps = [H.small_workload(**geo, past=[1500, 700, 33, 0, 4000, 257], new=[1] * 6, seed=301),
             H.small_workload(**geo, past=[90, 2100, 5], new=[1] * 3, seed=302)]
    for wl in steps:
        data = H.make_host_data(wl)
        op = H.make_op(wl)
        inp = _device_inputs(wl, data, dev)
        outs = []
        for static in (False, True):
            kc, vc = _filled_cache(op, wl, data, dev)
            out = torch.zeros_like(inp["q"])
            args = op.make_args(inp["q"], inp["k"], inp["v"], out, kc, vc, inp["past_lens"], inp["sub"], inp["bi"], inp["bib"],
                                wl.scale, wl.max_context_len)
            if static:
                rc = op.lib.pa_b200_decode_step_static(C.byref(op.desc), C.byref(args), 0)
                assert rc == 0, op.lib.pa_b200_last_error()
            else:
                op.forward_args(args)
            torch.cuda.synchronize(dev)
            outs.append((out.float().cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy()))
        (ref_out, ref_kc, ref_vc), (st_out, st_kc, st_vc) = outs
        assert np.array_equal(ref_kc, st_kc) and np.array_equal(ref_vc, st_vc), "cache bytes differ between the entry points"
        assert H.rel_err(st_out, ref_out) < tol
        oracle = H.run_oracle(wl, data)["out_ref"]
        assert H.rel_err(st_out, oracle) < max(tol, 8e-3 if act == torch.bfloat16 else tol)


def test_static_scratch_entry_rejects_what_it_cannot_hold():
    wl = H.small_workload(hq=32, hkv=8, d=128, bs=32, act=torch.bfloat16, cache="u8", past=[10], new=[1], seed=303)
    op = H.make_op(wl)
    from openvino_genai_b200 import _abi
    a = _abi.pa_forward_args()
    a.struct_size = C.sizeof(_abi.pa_forward_args)
    n = 60000
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    for f in ("query", "key", "value", "output", "key_cache", "value_cache", "past_lens", "subsequence_begins", "block_indices",
              "block_indices_begins"):
        setattr(a, f, dummy.data_ptr())
    a.num_tokens = a.num_sequences = n
    a.max_context_len = 64
    a.num_block_indices = n * 2
    a.num_blocks = 8
    rc = op.lib.pa_b200_decode_step_static(C.byref(op.desc), C.byref(a), 0)   # nothing is launched: rejected on the host
    assert rc == _abi.PA_ERR_TOO_LARGE
    assert b"scratch" in op.lib.pa_b200_last_error()
    a.num_tokens = n + 1                                                      # a prefill row: not a plain decode step
    assert op.lib.pa_b200_decode_step_static(C.byref(op.desc), C.byref(a), 0) == _abi.PA_ERR_UNSUPPORTED
