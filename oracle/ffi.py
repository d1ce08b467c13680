"""numpy-facing ctypes wrapper of the CPU oracle (oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The CUDA library and its Python mirror never
import this module.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build as _build

Q4_0, TQ2_0 = 0, 1
_lib = None

u8p = C.c_void_p


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(_build.build()))
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_tq_encode.restype = C.c_uint16
        _lib.orc_tq_code_bytes.restype = C.c_size_t
        _lib.orc_tq_code_bytes.argtypes = [C.c_size_t, C.c_uint]
        _lib.orc_swa_ring_capacity.restype = C.c_size_t
        _lib.orc_swa_ring_capacity.argtypes = [C.c_size_t, C.c_size_t]
        _lib.orc_argmax.restype = C.c_uint32
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def _h(a) -> np.ndarray:
    """f16 array viewed as uint16 (the oracle's f16 carrier)."""
    return np.ascontiguousarray(a, dtype=np.float16).view(np.uint16)


def _sz(v):
    return C.c_size_t(int(v))


def _u(v):
    return C.c_uint(int(v))


def _f(v):
    return C.c_float(float(v))


def row_bytes(fmt: int, cols: int) -> int:
    return cols // 32 * 18 if fmt == Q4_0 else cols // 256 * 66


def dequant(fmt: int, data, num_elements: int) -> np.ndarray:
    data = _c(data, np.uint8)
    out = np.zeros(num_elements, dtype=np.uint16)
    fn = lib().orc_dequant_q4_0 if fmt == Q4_0 else lib().orc_dequant_tq2_0
    fn(_p(data), _sz(data.size), _sz(num_elements), _p(out))
    return out.view(np.float16)


def expand_f32(fmt: int, w, rows: int, cols: int) -> np.ndarray:
    w = _c(w, np.uint8)
    out = np.empty((rows, cols), dtype=np.float32)
    lib().orc_expand_f32(C.c_int(fmt), _p(w), _sz(rows), _sz(cols), _p(out))
    return out


def matmul_nt(fmt: int, a, w, m: int, k: int, n: int) -> np.ndarray:
    """c[m, n] f32 (f64 accumulate) = a[m, k] f16 x W[n, k]^T."""
    a, w = _h(a), _c(w, np.uint8)
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_matmul_nt_quant(C.c_int(fmt), _p(a), _p(w), _sz(m), _sz(k), _sz(n), _p(out))
    return out


def matvec(fmt: int, w, x, rows: int, cols: int) -> np.ndarray:
    return matmul_nt(fmt, x, w, 1, cols, rows).reshape(rows)


def baseline_matmul_nt(fmt: int, a, w, m: int, k: int, n: int, threads: int = 0) -> np.ndarray:
    a, w = _h(a), _c(w, np.uint8)
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_baseline_matmul_nt(C.c_int(fmt), _p(a), _p(w), _sz(m), _sz(k), _sz(n), _p(out), C.c_int(threads))
    return out


def tq2_dequant(packed, scales, n: int) -> np.ndarray:
    packed, scales = _c(packed, np.uint8), _h(scales)
    out = np.empty(n, dtype=np.uint16)
    lib().orc_tq2_dequant(_p(packed), _p(scales), _p(out), _sz(n))
    return out.view(np.float16)


def fwht_normalized(v) -> np.ndarray:
    v = _c(v, np.float32).copy()
    lib().orc_fwht_normalized(_p(v), _sz(v.size))
    return v


def tq_signs(dim: int, seed: int) -> np.ndarray:
    out = np.empty(dim, dtype=np.float32)
    lib().orc_tq_signs(_sz(dim), C.c_uint64(seed), _p(out))
    return out


def lloyd_max_gaussian(bits: int) -> np.ndarray:
    out = np.empty(1 << bits, dtype=np.float32)
    lib().orc_lloyd_max_gaussian(_u(bits), _p(out))
    return out


def tq_levels(dim: int, bits: int) -> np.ndarray:
    out = np.empty(1 << bits, dtype=np.float32)
    lib().orc_tq_levels(_sz(dim), _u(bits), _p(out))
    return out


def tq_code_bytes(dim: int, bits: int) -> int:
    return lib().orc_tq_code_bytes(dim, bits)


def tq_encode(x, bits: int, signs, levels, norm_mode: int = 0):
    """-> (codes uint8[code_bytes], norm as np.float16 scalar)."""
    x, signs, levels = _c(x, np.float32), _c(signs, np.float32), _c(levels, np.float32)
    codes = np.empty(tq_code_bytes(x.size, bits), dtype=np.uint8)
    nb = lib().orc_tq_encode(_p(x), _sz(x.size), _u(bits), _p(signs), _p(levels), _p(codes), C.c_int(norm_mode))
    return codes, np.array([nb], dtype=np.uint16).view(np.float16)[0]


def tq_decode(codes, norm, dim: int, bits: int, signs, levels) -> np.ndarray:
    codes, signs, levels = _c(codes, np.uint8), _c(signs, np.float32), _c(levels, np.float32)
    nb = int(np.array([norm], dtype=np.float16).view(np.uint16)[0])
    out = np.empty(dim, dtype=np.float32)
    lib().orc_tq_decode(_p(codes), C.c_uint16(nb), _sz(dim), _u(bits), _p(signs), _p(levels), _p(out))
    return out


def encode_kv(inp, levels, signs, packed, norms, hd, n_kv, num_tokens, bits, position, ring, norm_mode=0):
    """In place on `packed` (uint8) and `norms` (float16)."""
    lib().orc_encode_kv(_p(_h(inp)), _p(_c(levels, np.float32)), _p(_c(signs, np.float32)), _p(packed),
                        _p(norms.view(np.uint16)), _u(hd), _u(n_kv), _u(num_tokens), _u(bits), _u(position),
                        _u(ring), C.c_int(norm_mode))


def encode_kv_batched(inp, levels, signs, packed, norms, positions, hd, n_kv, lane_capacity, bits, n_lanes, ring,
                      norm_mode=0):
    lib().orc_encode_kv_batched(_p(_h(inp)), _p(_c(levels, np.float32)), _p(_c(signs, np.float32)), _p(packed),
                                _p(norms.view(np.uint16)), _p(_c(positions, np.uint32)), _u(hd), _u(n_kv),
                                _u(lane_capacity), _u(bits), _u(n_lanes), _u(ring), C.c_int(norm_mode))


def dequantize_kv(packed, norms, levels, signs, hd, n_kv, num_tokens, bits, token_start, ring) -> np.ndarray:
    out = np.zeros(num_tokens * n_kv * hd, dtype=np.uint16)
    lib().orc_dequantize_kv(_p(_c(packed, np.uint8)), _p(_h(norms)), _p(_c(levels, np.float32)),
                            _p(_c(signs, np.float32)), _p(out), _u(hd), _u(n_kv), _u(num_tokens), _u(bits),
                            _u(token_start), _u(ring))
    return out.view(np.float16)


def hadamard_rotate(x, signs, hd: int, heads: int, pre: bool, post: bool) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(heads * hd, dtype=np.float32)
    lib().orc_hadamard_rotate(_p(x), _p(_c(signs, np.float32)), _p(out), _u(hd), _u(heads), C.c_int(pre), C.c_int(post))
    return out


def flash_attention_tq(rq, kc, kn, vc, vn, levels, hd, kv_len, current_pos, n_q, n_kv, window, bits, ring,
                       scale=1.0) -> np.ndarray:
    out = np.empty(n_q * hd, dtype=np.float32)
    lib().orc_flash_attention_tq(_p(_c(rq, np.float32)), _p(_c(kc, np.uint8)), _p(_h(kn)), _p(_c(vc, np.uint8)),
                                 _p(_h(vn)), _p(_c(levels, np.float32)), _p(out), _u(hd), _u(kv_len),
                                 _u(current_pos), _u(n_q), _u(n_kv), _u(window), _u(bits), _u(ring), _f(scale))
    return out


def flash_attention_tq_batched(rq, kc, kn, vc, vn, levels, positions, hd, lane_capacity, n_q, n_kv, window, bits,
                               n_lanes, ring, scale=1.0) -> np.ndarray:
    out = np.empty(n_lanes * n_q * hd, dtype=np.float32)
    lib().orc_flash_attention_tq_batched(_p(_c(rq, np.float32)), _p(_c(kc, np.uint8)), _p(_h(kn)),
                                         _p(_c(vc, np.uint8)), _p(_h(vn)), _p(_c(levels, np.float32)), _p(out),
                                         _p(_c(positions, np.uint32)), _u(hd), _u(lane_capacity), _u(n_q), _u(n_kv),
                                         _u(window), _u(bits), _u(n_lanes), _u(ring), _f(scale))
    return out


def flash_attention_tq_prefill(rq, kc, kn, vc, vn, levels, hd, kv_len, start_pos, n_rows, n_q, n_kv, window, bits, ring,
                               scale=1.0, tiled=False) -> np.ndarray:
    """[n_rows, n_q, hd] f32; `tiled` selects the f16-tile arithmetic of the query-tiled shader."""
    out = np.empty(n_rows * n_q * hd, dtype=np.float32)
    fn = lib().orc_flash_attention_tq_prefill_tiled if tiled else lib().orc_flash_attention_tq_prefill
    fn(_p(_c(rq, np.float32)), _p(_c(kc, np.uint8)), _p(_h(kn)), _p(_c(vc, np.uint8)), _p(_h(vn)),
       _p(_c(levels, np.float32)), _p(out), _u(hd), _u(kv_len), _u(start_pos), _u(n_rows), _u(n_q), _u(n_kv), _u(window),
       _u(bits), _u(ring), _f(scale))
    return out


def tq_attention_fused(q, kc, kn, vc, vn, levels, signs, positions, hd, lane_capacity, n_q, n_kv, window, bits,
                       n_lanes, ring, scale=1.0, kv_len=0, current_pos=0) -> np.ndarray:
    out = np.empty(n_lanes * n_q * hd, dtype=np.uint16)
    pos = _p(_c(positions, np.uint32)) if positions is not None else None
    lib().orc_tq_attention_fused(_p(_h(q)), _p(_c(kc, np.uint8)), _p(_h(kn)), _p(_c(vc, np.uint8)), _p(_h(vn)),
                                 _p(_c(levels, np.float32)), _p(_c(signs, np.float32)), _p(out), pos, _u(hd),
                                 _u(lane_capacity), _u(n_q), _u(n_kv), _u(window), _u(bits), _u(n_lanes), _u(ring),
                                 _f(scale), _u(kv_len), _u(current_pos))
    return out.view(np.float16)


def attention_f16(q, k, v, hd, kv_len, current_pos, n_q, n_kv, window, scale=1.0) -> np.ndarray:
    out = np.empty(n_q * hd, dtype=np.uint16)
    lib().orc_attention_f16(_p(_h(q)), _p(_h(k)), _p(_h(v)), _p(out), _u(hd), _u(kv_len), _u(current_pos), _u(n_q),
                            _u(n_kv), _u(window), _f(scale))
    return out.view(np.float16)


def swa_ring_capacity(window: int, max_positions: int) -> int:
    return lib().orc_swa_ring_capacity(window, max_positions)


def rms_norm(x, weight, dim, rows, eps, residual=None) -> np.ndarray:
    out = np.empty(rows * dim, dtype=np.uint16)
    res = _p(_h(residual)) if residual is not None else None
    lib().orc_rms_norm(_p(_h(x)), _p(_h(weight)), res, _p(out), _u(dim), _u(rows), _f(eps))
    return out.view(np.float16)


def rope(qk, positions, theta, hd, heads, rows, factor=1.0) -> np.ndarray:
    out = _h(qk).copy()
    lib().orc_rope(_p(out), _p(_c(positions, np.uint32)), _f(theta), _u(hd), _u(heads), _u(rows), _f(factor))
    return out.view(np.float16)


def gelu_mul(a, b) -> np.ndarray:
    a, b = _h(a), _h(b)
    out = np.empty(a.size, dtype=np.uint16)
    lib().orc_gelu_mul(_p(a), _p(b), _p(out), _sz(a.size))
    return out.view(np.float16)


def residual_add(a, b) -> np.ndarray:
    a, b = _h(a), _h(b)
    out = np.empty(a.size, dtype=np.uint16)
    lib().orc_residual_add(_p(a), _p(b), _p(out), _sz(a.size))
    return out.view(np.float16)


def scale_in_place(x, scalar) -> np.ndarray:
    out = _h(x).copy()
    lib().orc_scale_in_place(_p(out), _f(scalar), _sz(out.size))
    return out.view(np.float16)


def gather_strided_f16(src, row_stride, base_off, pld, n_rows) -> np.ndarray:
    out = np.empty(n_rows * pld, dtype=np.uint16)
    lib().orc_gather_strided_f16(_p(_h(src)), _p(out), _u(row_stride), _u(base_off), _u(pld), _u(n_rows))
    return out.view(np.float16)


def logit_softcap(x, cap) -> np.ndarray:
    out = _c(x, np.float32).copy()
    lib().orc_logit_softcap(_p(out), _f(cap), _sz(out.size))
    return out


def argmax(v) -> int:
    v = _c(v, np.float32)
    return lib().orc_argmax(_p(v), _sz(v.size))


def embed_rows_q4_0(table, tokens, cols) -> np.ndarray:
    tokens = _c(tokens, np.uint32)
    out = np.empty(tokens.size * cols, dtype=np.uint16)
    lib().orc_embed_rows_q4_0(_p(_c(table, np.uint8)), _p(tokens), _u(tokens.size), _u(cols), _p(out))
    return out.view(np.float16)


def num_threads() -> int:
    return lib().orc_num_threads()


def set_num_threads(n: int) -> None:
    """OpenMP threads for every later call (a launcher may have exported OMP_NUM_THREADS=1)."""
    lib().orc_set_num_threads(C.c_int(int(n)))


def host_threads() -> int:
    """The host threads this process may use: its affinity mask, else the CPU count."""
    import os
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def set_step_baseline_matmul(on: bool) -> None:
    """Decode-step projections in the CPU baseline's arithmetic (weights rounded to f16, f32 dot) instead of the
    checker's f64 accumulation."""
    lib().orc_set_step_baseline_matmul(C.c_int(1 if on else 0))


# ---- decode step (composition) ----
class _OrcLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown", "attn_norm", "q_norm", "k_norm",
                                          "post_attn_norm", "ffn_norm", "post_ffn_norm", "k_codes", "v_codes", "k_norms",
                                          "v_norms")] + [(n, C.c_uint32) for n in ("window", "ring", "lane_rows")]


class _OrcModel(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("hidden", "n_q", "n_kv", "hd", "inter", "vocab", "n_layers", "bits")] + \
               [(n, C.c_float) for n in ("eps", "rope_theta", "softmax_scale", "embed_scale")] + \
               [(n, C.c_void_p) for n in ("embed", "final_norm", "levels", "signs", "layers")]


class OracleModel:
    """Host-memory twin of the decode-step model: same weights, its own KV pools."""

    def __init__(self, cfg, layers: list, embed, final_norm, pool_geometry: list):
        """cfg: any object with the lc_model_config field names; layers: list of dicts of numpy tensors;
        pool_geometry: per layer (lane_rows, ring, window)."""
        self.cfg = cfg
        self.keep = []
        self.levels, self.signs = tq_levels(cfg.head_dim, cfg.kv_bits), tq_signs(cfg.head_dim, 0x7459C0DE)
        cb = tq_code_bytes(cfg.head_dim, cfg.kv_bits)
        arr = (_OrcLayer * cfg.n_layers)()
        self.pools = []
        for i, (t, (lane_rows, ring, window)) in enumerate(zip(layers, pool_geometry)):
            rows = cfg.max_lanes * lane_rows * cfg.n_kv_heads
            pool = {"k_codes": np.zeros(rows * cb, np.uint8), "v_codes": np.zeros(rows * cb, np.uint8),
                    "k_norms": np.zeros(rows, np.float16), "v_norms": np.zeros(rows, np.float16)}
            self.pools.append(pool)
            for name in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown"):
                a = _c(t[name], np.uint8)
                self.keep.append(a)
                setattr(arr[i], name, a.ctypes.data)
            for name in ("attn_norm", "q_norm", "k_norm", "post_attn_norm", "ffn_norm", "post_ffn_norm"):
                a = _h(t[name])
                self.keep.append(a)
                setattr(arr[i], name, a.ctypes.data)
            for name in ("k_codes", "v_codes", "k_norms", "v_norms"):
                setattr(arr[i], name, pool[name].ctypes.data)
            arr[i].window, arr[i].ring, arr[i].lane_rows = window, ring, lane_rows
        self.layer_arr = arr
        self.embed, self.final_norm = _c(embed, np.uint8), _h(final_norm)
        self.m = _OrcModel(hidden=cfg.hidden, n_q=cfg.n_q_heads, n_kv=cfg.n_kv_heads, hd=cfg.head_dim, inter=cfg.inter,
                           vocab=cfg.vocab, n_layers=cfg.n_layers, bits=cfg.kv_bits, eps=cfg.rms_eps,
                           rope_theta=cfg.rope_theta, softmax_scale=cfg.softmax_scale, embed_scale=cfg.embed_scale,
                           embed=self.embed.ctypes.data, final_norm=self.final_norm.ctypes.data,
                           levels=self.levels.ctypes.data, signs=self.signs.ctypes.data,
                           layers=C.addressof(arr))

    def decode_batch_step(self, tokens, positions, want_logits=True, norm_mode=0):
        tokens, positions = _c(tokens, np.uint32), _c(positions, np.uint32)
        n = tokens.size
        logits = np.empty((n, self.cfg.vocab), np.float32) if want_logits else None
        hidden = np.empty((n, self.cfg.hidden), np.uint16)
        lib().orc_decode_batch_step(C.byref(self.m), _p(tokens), _p(positions), _u(n),
                                    _p(logits) if want_logits else None, _p(hidden), C.c_int(norm_mode))
        return logits, hidden.view(np.float16)
