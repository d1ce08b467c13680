"""Host-side partitioning for multi-GPU decode (one process per GPU).

The decode path shards by request only: lanes are independent, every rank holds all weights and the
KV rows of its own lanes, and no collective sits on the data path.  The one optional exchange is the
row-split vocabulary projection: rank r projects rows [lo_r, hi_r) of the table for ALL lanes (after an
all-gather of the final hidden rows), then either the f32 logit slices are all-gathered, or each rank
reduces its slice to (max value, first index) per lane and only those pairs are exchanged; the merge
rule reproduces the reference's first-maximum greedy choice (local-engine/src/sampler.rs:148-158).
"""
from __future__ import annotations

import numpy as np


def shard_lanes(contexts: np.ndarray, world: int) -> list[np.ndarray]:
    """Assign lanes to ranks so that every rank gets len/world lanes (+-1) and a near-equal sum of context
    lengths (attention cost is proportional to context).  Deterministic: longest first, to the lightest
    rank that still has room."""
    n = len(contexts)
    cap = [(n + world - 1 - r) // world for r in range(world)]  # sizes differ by at most one
    order = np.argsort(-contexts.astype(np.int64), kind="stable")
    load = np.zeros(world, dtype=np.int64)
    out: list[list[int]] = [[] for _ in range(world)]
    for lane in order:
        cands = [r for r in range(world) if len(out[r]) < cap[r]]
        r = min(cands, key=lambda i: (load[i], i))
        out[r].append(int(lane))
        load[r] += int(contexts[lane])
    return [np.array(sorted(x), dtype=np.int64) for x in out]


def vocab_rows(vocab: int, world: int, rank: int, align: int = 128) -> tuple[int, int]:
    """Rows [lo, hi) of the vocabulary table owned by `rank`; slices are multiples of `align` rows
    (the matmul's row tile) except possibly the last."""
    per = -(-vocab // world)
    per = -(-per // align) * align
    lo = min(vocab, rank * per)
    return lo, min(vocab, lo + per)


def merge_argmax(values: np.ndarray, indices: np.ndarray) -> np.ndarray:
    """values, indices: [world, lanes] per-shard (max, global first index).  Returns the global greedy token per
    lane: the largest value, and among equal values the smallest index — what a single first-maximum scan over
    the full row returns."""
    values = np.asarray(values, dtype=np.float64)
    indices = np.asarray(indices, dtype=np.int64)
    best, tok = values[0].copy(), indices[0].copy()
    for r in range(1, values.shape[0]):
        v, i = values[r], indices[r]
        better = (v > best) | ((v == best) & (i < tok))
        tok = np.where(better, i, tok)
        best = np.where(better, v, best)
    return tok.astype(np.uint32)


PAIR_DTYPE = np.dtype([("value", np.float32), ("index", np.uint32)])   # what lc_argmax_pairs_f32_into writes


def argmax_pairs(logits: np.ndarray, index_offset: int) -> np.ndarray:
    """Host twin of lc_argmax_pairs_f32_into: per row (max, first index + offset) with a strict '>' scan; an all
    -inf / NaN row reports (-inf, offset)."""
    logits = np.asarray(logits, dtype=np.float32)
    out = np.empty(logits.shape[0], dtype=PAIR_DTYPE)
    for r, row in enumerate(logits):
        bv, bi = np.float32(-np.inf), 0
        for i, x in enumerate(row):
            if x > bv:
                bv, bi = x, i
        out[r] = (bv, bi + index_offset)
    return out


def merge_argmax_pairs(pairs_all: np.ndarray) -> np.ndarray:
    """Host twin of lc_merge_argmax_pairs_into: pairs_all is [shards, rows] of PAIR_DTYPE, shards in index order.
    A later shard wins only with a strictly larger value, so equal maxima go to the lowest index; a row whose every
    shard reports -inf keeps the first shard's index."""
    pairs_all = np.asarray(pairs_all, dtype=PAIR_DTYPE)
    tok = pairs_all[0]["index"].copy()
    best = np.full(pairs_all.shape[1], -np.inf, np.float32)
    for s in range(pairs_all.shape[0]):
        better = pairs_all[s]["value"] > best
        tok = np.where(better, pairs_all[s]["index"], tok)
        best = np.where(better, pairs_all[s]["value"], best)
    return tok.astype(np.uint32)


def greedy_from_logit_slices(logits_all, rows: int):
    """The row-split vocabulary variant after the all-gather: `logits_all` is a torch tensor [world, lanes, rows]
    (shard r holds table rows [r * rows, (r + 1) * rows) for every lane).  Returns the greedy token per lane with the
    reference's first-maximum rule: torch's max / argmax return the first maximal index, and among shards holding the
    same maximum the lowest shard (= lowest rows) wins."""
    import torch
    vals, idx = logits_all.max(dim=2)                       # [world, lanes]
    best = vals.max(dim=0).values
    shard = (vals == best).to(torch.int32).argmax(dim=0)    # first shard holding the maximum
    return idx.gather(0, shard[None])[0] + shard * rows
