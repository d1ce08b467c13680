"""Host-side mirror of the decode-step API (`lc_model_*`): the part of
`Pipeline` (local-engine/src/pipeline/batched.rs:271-456) that composes the hot-path
kernels, plus a seeded random-init builder for the synthetic Gemma-4-E2B-like decoder
the benchmark configurations describe."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib, synth
from .kernels import CommandBatch, CudaBuffer, CudaContext, Kernels, _check


class ModelConfig(C.Structure):
    """lc_model_config."""
    _fields_ = [(n, C.c_uint32) for n in ("hidden", "n_q_heads", "n_kv_heads", "head_dim", "inter", "vocab", "n_layers",
                                          "kv_bits", "max_lanes", "max_context", "swa_window", "swa_ring", "full_every")] + \
               [(n, C.c_float) for n in ("rms_eps", "rope_theta", "softmax_scale", "embed_scale")]


def e2b_like_config(max_lanes: int = 64, max_context: int = 8192 + 64, n_layers: int = 35, vocab: int = 262144,
                    kv_bits: int = 2, swa_ring: int = 512) -> ModelConfig:
    """35 layers, hidden 1536, 8 q heads / 1 kv head of 256, GeGLU 6144, RoPE theta 1e6,
    4:1 sliding(512):full pattern, softmax scale 1/sqrt(256)."""
    return ModelConfig(hidden=1536, n_q_heads=8, n_kv_heads=1, head_dim=256, inter=6144, vocab=vocab, n_layers=n_layers,
                       kv_bits=kv_bits, max_lanes=max_lanes, max_context=max_context, swa_window=512, swa_ring=swa_ring,
                       full_every=5, rms_eps=1e-6, rope_theta=1e6, softmax_scale=1.0 / 16.0,
                       embed_scale=float(np.sqrt(np.float32(1536))))


LAYER_TENSORS = ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown", "attn_norm", "q_norm", "k_norm", "post_attn_norm",
                 "ffn_norm", "post_ffn_norm")


def layer_shapes(cfg: ModelConfig) -> dict:
    qd, kd = cfg.n_q_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    return {"wq": (qd, cfg.hidden), "wk": (kd, cfg.hidden), "wv": (kd, cfg.hidden), "wo": (cfg.hidden, qd),
            "wgate": (cfg.inter, cfg.hidden), "wup": (cfg.inter, cfg.hidden), "wdown": (cfg.hidden, cfg.inter)}


def synth_layer(cfg: ModelConfig, layer: int, seed: int = 0) -> dict:
    """Random-init tensors of one layer: TQ2_0 projections with ternary codes and d ~ U[0.005, 0.05],
    f16 norm weights close to 1."""
    out = {}
    base = seed * 1000003 + layer * 101
    for i, (name, (rows, cols)) in enumerate(layer_shapes(cfg).items()):
        out[name] = synth.tq2_0_weights(rows, cols, seed=base + i)
    for i, name in enumerate(("attn_norm", "post_attn_norm", "ffn_norm", "post_ffn_norm")):
        out[name] = (1.0 + 0.05 * synth.normal(base + 20 + i, cfg.hidden)).astype(np.float16)
    for i, name in enumerate(("q_norm", "k_norm")):
        out[name] = (1.0 + 0.05 * synth.normal(base + 30 + i, cfg.head_dim)).astype(np.float16)
    return out


def synth_embedding(cfg: ModelConfig, seed: int = 0):
    emb = synth.q4_0_weights(cfg.vocab, cfg.hidden, seed=seed * 1000003 + 77)
    fnorm = (1.0 + 0.05 * synth.normal(seed * 1000003 + 78, cfg.hidden)).astype(np.float16)
    return emb, fnorm


class DecodeModel:
    def __init__(self, ctx: CudaContext, kernels: Kernels, cfg: ModelConfig):
        self._lib = _lib.load()
        self.ctx, self.kernels, self.cfg = ctx, kernels, cfg
        h = C.c_void_p()
        _check(self._lib.lc_model_create(ctx._h, kernels._h, C.addressof(cfg), C.byref(h)))
        self._h = h
        self._keep = []  # weight buffers must outlive the model

    def set_layer(self, layer: int, tensors: dict) -> None:
        bufs = [tensors[n] if isinstance(tensors[n], CudaBuffer) else CudaBuffer.from_slice(self.ctx, tensors[n])
                for n in LAYER_TENSORS]
        self._keep.append(bufs)
        _check(self._lib.lc_model_set_layer(self._h, layer, *[b._h for b in bufs]))

    def set_embedding(self, embed, final_norm) -> None:
        e = embed if isinstance(embed, CudaBuffer) else CudaBuffer.from_slice(self.ctx, embed)
        f = final_norm if isinstance(final_norm, CudaBuffer) else CudaBuffer.from_slice(self.ctx, final_norm)
        self._keep.append((e, f))
        _check(self._lib.lc_model_set_embedding(self._h, e._h, f._h))

    def _borrow(self, handle: C.c_void_p) -> CudaBuffer:
        return CudaBuffer(self.ctx, handle, self._lib.lc_buf_length(handle))

    def kv_buffers(self, layer: int) -> dict:
        hs = [C.c_void_p() for _ in range(4)]
        rows, ring, window = C.c_uint32(), C.c_uint32(), C.c_uint32()
        _check(self._lib.lc_model_kv_buffers(self._h, layer, *[C.byref(h) for h in hs], C.addressof(rows),
                                             C.addressof(ring), C.addressof(window)))
        kc, kn, vc, vn = [self._borrow(h) for h in hs]
        return {"k_codes": kc, "k_norms": kn, "v_codes": vc, "v_norms": vn, "lane_rows": rows.value,
                "ring": ring.value, "window": window.value}

    def logits_buffer(self) -> CudaBuffer:
        h = C.c_void_p()
        _check(self._lib.lc_model_logits_buffer(self._h, C.byref(h)))
        return self._borrow(h)

    def hidden_buffer(self) -> CudaBuffer:
        h = C.c_void_p()
        _check(self._lib.lc_model_hidden_buffer(self._h, C.byref(h)))
        return self._borrow(h)

    def reset_lane(self, lane: int) -> None:
        _check(self._lib.lc_model_reset_lane(self._h, lane))

    def decode_batch_step_into(self, batch: CommandBatch, tokens: CudaBuffer, positions: CudaBuffer, n_lanes: int,
                               want_logits: bool = True, next_tokens: CudaBuffer | None = None) -> None:
        _check(self._lib.lc_model_decode_batch_step_into(self._h, batch._h, tokens._h, positions._h, n_lanes,
                                                         1 if want_logits else 0,
                                                         next_tokens._h if next_tokens is not None else None))

    def close(self) -> None:
        if self._h:
            self._lib.lc_model_destroy(self._h)
            self._h = None
