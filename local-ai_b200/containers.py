"""Host-side mirror of the KV containers: `QuantizedKvCache`
(local-engine/src/kv_cache/quant_cache.rs:73-700) over `lc_kv_cache_*`, and the lane admit / recycle
loop of `Pipeline::run_batched_to_completion` (local-engine/src/pipeline/runner.rs:123-214) over
`lc_lane_sched_*`.  Method names and argument order follow the Rust types."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .kernels import CommandBatch, CudaBuffer, CudaContext, Kernels, _check

STOP_REASONS = {0: None, 1: "Eos", 2: "MaxTokens", 3: "Capacity"}


class QuantizedKvCache:
    def __init__(self, ctx: CudaContext, n_kv_heads: int, head_dim: int, max_positions: int,
                 physical_positions: int | None = None, sliding_window: int = 0, bits: int = 2):
        self._lib, self.ctx = _lib.load(), ctx
        h = C.c_void_p()
        phys = max_positions if physical_positions is None else physical_positions
        _check(self._lib.lc_kv_cache_create(ctx._h, n_kv_heads, head_dim, max_positions, phys, sliding_window, bits, C.byref(h)))
        self._h = h
        self.n_kv_heads, self.head_dim, self.bits, self.max_positions = n_kv_heads, head_dim, bits, max_positions

    @classmethod
    def new_with_bits_and_ring(cls, ctx, n_kv_heads, head_dim, max_positions, physical_positions, sliding_window, bits):
        return cls(ctx, n_kv_heads, head_dim, max_positions, physical_positions, sliding_window, bits)

    def physical_positions(self) -> int:
        return self._lib.lc_kv_cache_physical_positions(self._h)

    def is_ringed(self) -> bool:
        return self.physical_positions() < self.max_positions

    def ring_capacity(self) -> int:
        return self._lib.lc_kv_cache_ring_capacity(self._h)

    def code_bytes(self) -> int:
        return self._lib.lc_kv_cache_code_bytes(self._h)

    def buffers(self) -> dict:
        hs = [C.c_void_p() for _ in range(6)]
        _check(self._lib.lc_kv_cache_buffers(self._h, *[C.byref(h) for h in hs]))
        names = ("keys_q", "key_norms", "values_q", "value_norms", "levels", "signs")
        return {n: CudaBuffer(self.ctx, h, self._lib.lc_buf_length(h)) for n, h in zip(names, hs)}

    def reset(self) -> None:
        _check(self._lib.lc_kv_cache_reset(self._h))

    def write_kv_gpu_into(self, batch: CommandBatch, kernels: Kernels, k_src: CudaBuffer, v_src: CudaBuffer, position: int,
                          n_rows: int) -> None:
        _check(self._lib.lc_kv_cache_write_kv_gpu_into(self._h, batch._h, kernels._h, k_src._h, v_src._h, position, n_rows))

    def fused_attention_into(self, batch, kernels, q, attn_out, seq_len, current_pos, n_q_heads, window, softmax_scale=1.0):
        _check(self._lib.lc_kv_cache_fused_attention_into(self._h, batch._h, kernels._h, q._h, attn_out._h, seq_len, current_pos,
                                                          n_q_heads, window, softmax_scale))

    def fused_attention_batch_into(self, batch, kernels, q, attn_out, kv_len, start_pos, n_rows, n_q_heads, window,
                                   softmax_scale=1.0):
        _check(self._lib.lc_kv_cache_fused_attention_batch_into(self._h, batch._h, kernels._h, q._h, attn_out._h, kv_len,
                                                                start_pos, n_rows, n_q_heads, window, softmax_scale))

    def max_snapshot_positions(self) -> int:
        return self._lib.lc_kv_cache_max_snapshot_positions(self._h)

    def snapshot_prefix(self, positions: int) -> dict:
        positions = min(positions, self.max_snapshot_positions())
        cb, nb = positions * self.n_kv_heads * self.code_bytes(), positions * self.n_kv_heads * 2
        snap = {"positions": positions, "keys_q": np.empty(cb, np.uint8), "values_q": np.empty(cb, np.uint8),
                "key_norms": np.empty(nb, np.uint8), "value_norms": np.empty(nb, np.uint8)}
        _check(self._lib.lc_kv_cache_snapshot_prefix(self._h, positions, snap["keys_q"].ctypes.data, snap["values_q"].ctypes.data,
                                                     snap["key_norms"].ctypes.data, snap["value_norms"].ctypes.data))
        return snap

    def restore_prefix(self, snap: dict, positions: int) -> None:
        positions = min(positions, snap["positions"])
        _check(self._lib.lc_kv_cache_restore_prefix(self._h, positions, snap["keys_q"].ctypes.data, snap["values_q"].ctypes.data,
                                                    snap["key_norms"].ctypes.data, snap["value_norms"].ctypes.data))

    def close(self) -> None:
        if self._h:
            self._lib.lc_kv_cache_destroy(self._h)
            self._h = None


class LaneScheduler:
    """Continuous batching over the lanes of a DecodeModel (or host logic only, with model=None)."""

    def __init__(self, model, n_lanes: int, lane_capacity: int, eos_token: int):
        self._lib = _lib.load()
        h = C.c_void_p()
        _check(self._lib.lc_lane_sched_create(model._h if model is not None else None, n_lanes, lane_capacity, eos_token, C.byref(h)))
        self._h, self.n_lanes = h, n_lanes
        self.tokens = np.zeros(n_lanes, np.uint32)
        self.positions = np.zeros(n_lanes, np.uint32)

    def submit(self, req_id: int, prompt, max_new_tokens: int) -> None:
        p = np.ascontiguousarray(prompt, dtype=np.uint32)
        _check(self._lib.lc_lane_sched_submit(self._h, req_id, p.ctypes.data, p.size, max_new_tokens))

    def prepare(self) -> int:
        n = C.c_uint32()
        _check(self._lib.lc_lane_sched_prepare(self._h, self.tokens.ctypes.data, self.positions.ctypes.data, C.addressof(n)))
        return n.value

    def consume(self, next_tokens) -> None:
        t = np.ascontiguousarray(next_tokens, dtype=np.uint32)
        assert t.size == self.n_lanes
        _check(self._lib.lc_lane_sched_consume(self._h, t.ctypes.data))

    def pop_finished(self):
        """(id, tokens, reason) of one completed request, or None."""
        rid, n, reason = C.c_uint64(), C.c_uint32(), C.c_int()
        _check(self._lib.lc_lane_sched_pop_finished(self._h, C.addressof(rid), None, 0, C.addressof(n), C.addressof(reason)))
        if reason.value == 0:
            return None
        out = np.empty(max(n.value, 1), np.uint32)
        _check(self._lib.lc_lane_sched_pop_finished(self._h, C.addressof(rid), out.ctypes.data, out.size, C.addressof(n),
                                                    C.addressof(reason)))
        return rid.value, out[: n.value].copy(), STOP_REASONS[reason.value]

    def pending(self) -> int:
        return self._lib.lc_lane_sched_pending(self._h)

    def close(self) -> None:
        if self._h:
            self._lib.lc_lane_sched_destroy(self._h)
            self._h = None
