"""Host-side mirror of the PagedAttentionExtension operator interface.

The reference reaches this operator through named model tensors that ModelRunner::forward fills
(src/cpp/src/continuous_batching/model_runner.hpp:505-522, 802-853, 1420-1509); an OpenVINO
extension op would receive the same tensors in `evaluate(outputs, inputs)`
(tests/cpp/custom_op/custom_add.cpp:49-80).  `PagedAttentionExtension.evaluate` takes them by
those names and forwards to the C ABI: device tensors go to pa_b200_forward, host tensors to
pa_b200_forward_host.  Errors raise GenaiB200Error where the reference raises ov::Exception.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from . import _abi

_ACT = {torch.float32: _abi.PA_DTYPE_F32, torch.float16: _abi.PA_DTYPE_F16, torch.bfloat16: _abi.PA_DTYPE_BF16}
_CACHE = {"f16": _abi.PA_DTYPE_F16, "bf16": _abi.PA_DTYPE_BF16, "u8": _abi.PA_DTYPE_U8}


def _ptr(t) -> Optional[int]:
    if t is None:
        return None
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    return t.data_ptr()


class PagedAttentionExtension:
    """One attention layer's operator instance (owns a C-ABI handle and its scratch)."""

    def __init__(self, num_q_heads: int, num_kv_heads: int, head_size: int, block_size: int,
                 act_dtype: torch.dtype = torch.float16, cache_dtype: str = "f16", device: int = 0):
        from . import GenaiB200Error, load_library
        self._err = GenaiB200Error
        self.lib = load_library()
        self.desc = _abi.pa_model_desc(C.sizeof(_abi.pa_model_desc), num_q_heads, num_kv_heads, head_size, block_size,
                                       _ACT[act_dtype], _CACHE[cache_dtype])
        self.act_dtype = act_dtype
        self.cache_dtype = cache_dtype
        self.device = device
        self.num_q_heads, self.num_kv_heads, self.head_size, self.block_size = num_q_heads, num_kv_heads, head_size, block_size
        self._h = C.c_void_p()
        self._check(self.lib.pa_b200_create(C.byref(self.desc), device, C.byref(self._h)))

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self.lib.pa_b200_destroy(h)
            self._h = None

    def _check(self, rc: int) -> None:
        if rc != _abi.PA_OK:
            raise self._err(f"pa_b200 status {rc}: {self.lib.pa_b200_last_error().decode()}")

    # ---- cache ---------------------------------------------------------------------------------
    def cache_layout(self) -> _abi.pa_cache_layout:
        out = _abi.pa_cache_layout()
        out.struct_size = C.sizeof(_abi.pa_cache_layout)
        self._check(self.lib.pa_b200_query_cache_layout(C.byref(self.desc), C.byref(out)))
        return out

    def allocate_cache(self, num_blocks: int, fill: Optional[int] = 0):
        """Returns (key_cache, value_cache) as flat uint8 device tensors of the declared byte size."""
        lay = self.cache_layout()
        dev = torch.device("cuda", self.device)
        mk = (lambda n: torch.full((n,), fill, dtype=torch.uint8, device=dev)) if fill is not None else \
             (lambda n: torch.empty((n,), dtype=torch.uint8, device=dev))
        return mk(num_blocks * lay.key_block_bytes), mk(num_blocks * lay.value_block_bytes)

    # ---- the operator --------------------------------------------------------------------------
    def make_args(self, query, key, value, output, key_cache, value_cache, past_lens, subsequence_begins, block_indices,
                  block_indices_begins, scale=None, max_context_len=None, score_aggregation_window=None, scores=None,
                  rotated_block_indices=None, rotation_deltas=None, rotation_trig_lut=None, stream=None,
                  sliding_window=0, alibi_slopes=None) -> _abi.pa_forward_args:
        a = _abi.pa_forward_args()
        a.struct_size = C.sizeof(_abi.pa_forward_args)
        a.query, a.key, a.value, a.output = _ptr(query), _ptr(key), _ptr(value), _ptr(output)
        a.num_tokens = int(query.shape[0])
        a.key_cache, a.value_cache = _ptr(key_cache), _ptr(value_cache)
        lay = self.cache_layout()
        a.num_blocks = int(key_cache.numel() // lay.key_block_bytes)
        a.past_lens, a.subsequence_begins = _ptr(past_lens), _ptr(subsequence_begins)
        a.block_indices, a.block_indices_begins = _ptr(block_indices), _ptr(block_indices_begins)
        a.num_sequences = int(past_lens.shape[0])
        a.num_block_indices = int(block_indices.shape[0])
        a.max_context_len = int(max_context_len) if max_context_len is not None else 0
        a.scale = float(scale) if scale is not None else 0.0
        a.sliding_window = int(sliding_window)
        a.alibi_slopes = _ptr(alibi_slopes)
        a.score_aggregation_window = _ptr(score_aggregation_window)
        a.scores = _ptr(scores)
        a.scores_len = int(scores.shape[0]) if scores is not None else 0
        a.rotated_block_indices = _ptr(rotated_block_indices)
        a.rotation_deltas = _ptr(rotation_deltas)
        a.num_rotated_blocks = int(rotated_block_indices.shape[0]) if rotated_block_indices is not None else 0
        a.rotation_trig_lut = _ptr(rotation_trig_lut)
        a.rotation_lut_rows = int(rotation_trig_lut.shape[0]) if rotation_trig_lut is not None else 0
        if stream is None and isinstance(query, torch.Tensor) and query.is_cuda:
            stream = torch.cuda.current_stream(query.device).cuda_stream  # order after the caller's torch work
        if stream == 0:
            stream = 1  # cudaStreamLegacy: NULL would select the handle's own stream instead of the default stream
        a.stream = stream
        # the struct holds raw addresses: keep every buffer alive for as long as the struct is
        a._buffers = (query, key, value, output, key_cache, value_cache, past_lens, subsequence_begins, block_indices,
                      block_indices_begins, alibi_slopes, score_aggregation_window, scores, rotated_block_indices,
                      rotation_deltas, rotation_trig_lut)
        return a

    def forward_args(self, args: _abi.pa_forward_args, host: bool = False) -> None:
        fn = self.lib.pa_b200_forward_host if host else self.lib.pa_b200_forward
        self._check(fn(self._h, C.byref(args)))

    def evaluate(self, inputs: dict, outputs: dict) -> None:
        """inputs / outputs are keyed by the reference's tensor names; `output` (and `scores`)
        must be preallocated by the caller, who owns every buffer."""
        q = inputs["query"]
        host = isinstance(q, np.ndarray) or (isinstance(q, torch.Tensor) and not q.is_cuda)
        mcl = inputs.get("max_context_len")
        if mcl is not None and not isinstance(mcl, int):
            mcl = int(mcl.item() if hasattr(mcl, "item") else mcl)
        args = self.make_args(q, inputs["key"], inputs["value"], outputs["output"], inputs["key_cache"], inputs["value_cache"],
                              inputs["past_lens"], inputs["subsequence_begins"], inputs["block_indices"],
                              inputs["block_indices_begins"], inputs.get("scale"), mcl,
                              inputs.get("score_aggregation_window"), outputs.get("scores"),
                              inputs.get("rotated_block_indices"), inputs.get("rotation_deltas"),
                              inputs.get("rotation_trig_lut"), inputs.get("stream"),
                              inputs.get("sliding_window", 0), inputs.get("alibi_slopes"))
        self.forward_args(args, host=host)

    def device_status(self) -> int:
        bits = C.c_uint32(0)
        self._check(self.lib.pa_b200_last_device_status(self._h, C.byref(bits)))
        return bits.value

    def launch_count(self) -> int:
        return int(self.lib.pa_b200_launch_count(self._h))

    def last_prefill_kernel(self) -> str:
        """Which kernel served the prefill chunks of the last forward call: "none", "generic", "mma_sync" or "tcgen05"."""
        return ("none", "generic", "mma_sync", "tcgen05")[int(self.lib.pa_b200_last_prefill_kernel(self._h))]

    def copy_blocks(self, key_cache, value_cache, pairs, stream=None) -> None:
        lay = self.cache_layout()
        self._check(self.lib.pa_b200_copy_blocks(self._h, _ptr(key_cache), _ptr(value_cache),
                                                 int(key_cache.numel() // lay.key_block_bytes), _ptr(pairs),
                                                 int(pairs.shape[0]), stream))
