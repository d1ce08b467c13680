"""Host-memory tensors of the synthetic decoder for the oracle's decode step (test / benchmark
infrastructure): the same seeded random-init rule as the package's model builder, written against
plain attribute configs so the CPU reference arm does not need the CUDA library."""
import numpy as np


def layer_shapes(cfg):
    qd, kd = cfg.n_q_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    return {"wq": (qd, cfg.hidden), "wk": (kd, cfg.hidden), "wv": (kd, cfg.hidden), "wo": (cfg.hidden, qd),
            "wgate": (cfg.inter, cfg.hidden), "wup": (cfg.inter, cfg.hidden), "wdown": (cfg.hidden, cfg.inter)}


def build(synth, cfg, context, seed=4, swa_window=512, swa_ring=512, full_every=5):
    layers, geo = [], []
    for layer in range(cfg.n_layers):
        base = seed * 1000003 + layer * 101
        t = {}
        for i, (name, (rows, cols)) in enumerate(layer_shapes(cfg).items()):
            t[name] = synth.tq2_0_weights(rows, cols, seed=base + i)
        for i, name in enumerate(("attn_norm", "post_attn_norm", "ffn_norm", "post_ffn_norm")):
            t[name] = (1.0 + 0.05 * synth.normal(base + 20 + i, cfg.hidden)).astype(np.float16)
        for i, name in enumerate(("q_norm", "k_norm")):
            t[name] = (1.0 + 0.05 * synth.normal(base + 30 + i, cfg.head_dim)).astype(np.float16)
        layers.append(t)
        full = layer % full_every == full_every - 1
        geo.append((cfg.max_context, 0, 0) if full else (swa_ring, swa_ring, swa_window))
    emb = synth.q4_0_weights(cfg.vocab, cfg.hidden, seed=seed * 1000003 + 77)
    fnorm = (1.0 + 0.05 * synth.normal(seed * 1000003 + 78, cfg.hidden)).astype(np.float16)
    return layers, emb, fnorm, geo
