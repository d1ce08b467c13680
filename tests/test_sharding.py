"""Multi-GPU host logic on CPU: lane sharding, vocabulary row split, the greedy merge rule, and a
world-size-2 gloo run of the rank-side protocol (shard, 'decode', exchange (max, index), merge)."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_shard_lanes_balanced(la):
    ctxs = la.synth.lognormal_contexts(512, 9)
    for world in (1, 2, 4, 8):
        shards = la.sharding.shard_lanes(ctxs, world)
        allv = np.concatenate(shards)
        assert sorted(allv.tolist()) == list(range(512))
        sizes = [len(s) for s in shards]
        assert max(sizes) - min(sizes) <= 1
        loads = np.array([ctxs[s].sum() for s in shards], dtype=np.float64)
        assert loads.max() / loads.mean() < 1.15, loads
    assert [len(s) for s in la.sharding.shard_lanes(np.arange(5), 2)] == [3, 2]


def test_vocab_rows_cover_exactly(la):
    for vocab, world in ((262144, 8), (262144, 3), (1000, 4), (100, 8)):
        spans = [la.sharding.vocab_rows(vocab, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == vocab
        for (a, b), (c, d) in zip(spans, spans[1:]):
            assert b == c and a <= b
    assert la.sharding.vocab_rows(262144, 8, 3) == (98304, 131072)


def test_merge_argmax_equals_first_max_scan(la, orc):
    rng = np.random.default_rng(3)
    lanes, vocab, world = 7, 4096, 4
    logits = rng.standard_normal((lanes, vocab)).astype(np.float32)
    logits[1, 100] = logits[1, 3000] = 9.0      # tie across shards: lowest index wins
    logits[2, 2000] = logits[2, 2001] = 9.0     # tie inside a shard
    logits[3, :] = -np.inf                      # nothing beats -inf: index 0
    vals, idxs = [], []
    for r in range(world):
        lo, hi = la.sharding.vocab_rows(vocab, world, r)
        sl = logits[:, lo:hi]
        loc = np.array([orc.argmax(sl[i]) for i in range(lanes)])
        vals.append(sl[np.arange(lanes), loc])
        idxs.append(loc + lo)
    got = la.sharding.merge_argmax(np.array(vals), np.array(idxs))
    want = np.array([orc.argmax(logits[i]) for i in range(lanes)])
    assert got.tolist() == want.tolist()


def test_greedy_from_logit_slices_equals_first_max_scan(la, orc):
    import torch
    rng = np.random.default_rng(5)
    lanes, vocab, world = 9, 2048, 4
    logits = rng.standard_normal((lanes, vocab)).astype(np.float32)
    logits[1, 100] = logits[1, 1900] = 9.0      # tie across shards
    logits[2, 700] = logits[2, 701] = 9.0       # tie inside a shard
    logits[3, :] = -np.inf
    rows = vocab // world
    sl = torch.from_numpy(np.stack([logits[:, r * rows:(r + 1) * rows] for r in range(world)]))
    got = la.sharding.greedy_from_logit_slices(sl, rows).numpy()
    assert got.tolist() == [orc.argmax(logits[i]) for i in range(lanes)]


def test_pair_twins_equal_first_max_scan(la, orc):
    """The (max, index) records the device kernels exchange, merged shard by shard, give the single first-maximum
    scan (sampler.rs:148-158): ties across and inside shards, an all -inf row, a row with NaNs."""
    rng = np.random.default_rng(6)
    lanes, vocab, world = 7, 1024, 4
    logits = rng.standard_normal((lanes, vocab)).astype(np.float32)
    logits[1, 100] = logits[1, 900] = 9.0
    logits[2, 300] = logits[2, 301] = 9.0
    logits[3, :] = -np.inf
    logits[4, 5] = np.nan
    logits[4, 700] = 8.0
    rows = vocab // world
    pairs = np.stack([la.sharding.argmax_pairs(logits[:, r * rows:(r + 1) * rows], r * rows) for r in range(world)])
    got = la.sharding.merge_argmax_pairs(pairs)
    assert got.tolist() == [orc.argmax(logits[i]) for i in range(lanes)]
    assert got.tolist() == la.sharding.merge_argmax(pairs["value"], pairs["index"]).tolist()


def test_comm_entry_points_report_instead_of_failing_to_load(la):
    """NCCL is loaded at run time: the library itself loads without it, and lc_comm_available says which case holds."""
    lib = la._lib.load()
    assert lib.lc_comm_available() in (0, 11)   # LC_OK or LC_ERR_NCCL
    assert lib.lc_comm_rank(None) == 0 and lib.lc_comm_world(None) == 0


RANK_SCRIPT = textwrap.dedent('''
    import os, sys, numpy as np
    sys.path.insert(0, os.environ["REPO_ROOT"])
    import torch, torch.distributed as dist
    import importlib.util
    def load(name, path):
        spec = importlib.util.spec_from_file_location(name, path); m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m); return m
    root = os.environ["REPO_ROOT"]
    synth = load("synth", root + "/local-ai_b200/synth.py")
    sharding = load("sharding", root + "/local-ai_b200/sharding.py")
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    lanes, vocab, hidden = 12, 1024, 16
    ctxs = synth.lognormal_contexts(lanes, 5)
    mine = sharding.shard_lanes(ctxs, world)[rank]
    # every rank "decodes" its lanes: hidden rows are a deterministic function of the lane id
    table = synth.normal(1, vocab * hidden).reshape(vocab, hidden).astype(np.float32)
    h_local = np.stack([synth.normal(100 + int(l), hidden) for l in mine]).astype(np.float32)
    # row-split vocabulary projection: all-gather hidden rows, project own rows, exchange (max, index)
    sizes = [len(s) for s in sharding.shard_lanes(ctxs, world)]
    pad = max(sizes)
    buf = torch.zeros(pad, hidden); buf[: len(mine)] = torch.from_numpy(h_local)
    gathered = [torch.zeros(pad, hidden) for _ in range(world)]
    dist.all_gather(gathered, buf)
    order = np.concatenate(sharding.shard_lanes(ctxs, world))
    h_all = torch.cat([g[:n] for g, n in zip(gathered, sizes)]).numpy()
    lo, hi = sharding.vocab_rows(vocab, world, rank)
    logits = h_all @ table[lo:hi].T
    loc = logits.argmax(axis=1)
    pair = torch.tensor(np.stack([logits[np.arange(lanes), loc], (loc + lo).astype(np.float32)]))
    pairs = [torch.zeros_like(pair) for _ in range(world)]
    dist.all_gather(pairs, pair)
    vals = np.stack([p[0].numpy() for p in pairs]); idxs = np.stack([p[1].numpy().astype(np.int64) for p in pairs])
    tok = sharding.merge_argmax(vals, idxs)
    # the same exchange in the device kernels' record format (8 bytes per lane and shard), merged by their host twin
    rec = sharding.argmax_pairs(logits, lo)
    recs = [torch.zeros(lanes, 8, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(recs, torch.from_numpy(rec.view(np.uint8).reshape(lanes, 8).copy()))
    tok_rec = sharding.merge_argmax_pairs(np.stack([r.numpy().reshape(-1).view(sharding.PAIR_DTYPE) for r in recs]))
    assert tok_rec.tolist() == tok.tolist()
    full = np.stack([synth.normal(100 + int(l), hidden) for l in order]).astype(np.float32) @ table.T
    assert tok.tolist() == full.argmax(axis=1).tolist(), (tok, full.argmax(axis=1))
    # the variant that all-gathers the f32 logit slices themselves (equal slices: all_gather_into_tensor)
    rows = hi - lo
    assert vocab % world == 0 and rows == vocab // world
    sl = torch.from_numpy(np.ascontiguousarray(logits.astype(np.float32)))
    allsl = torch.empty(world * lanes, rows)          # gloo wants the concatenated form; NCCL also takes [world, ...]
    dist.all_gather_into_tensor(allsl, sl)
    tok2 = sharding.greedy_from_logit_slices(allsl.view(world, lanes, rows), rows).numpy()
    assert tok2.tolist() == full.argmax(axis=1).tolist()
    t = torch.tensor([float(rank + 1)]); dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == world
    dist.barrier(); dist.destroy_process_group()
    print("rank", rank, "ok")
''')


def test_two_rank_protocol_over_gloo(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    env = dict(os.environ, REPO_ROOT=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT="29617", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
    assert any("rank 0 ok" in o for o in outs) and any("rank 1 ok" in o for o in outs)
