"""NCCL behind the C ABI on two GPUs of one box (skipped with fewer): lc_comm_unique_id / lc_comm_create /
lc_comm_all_gather_into, and the row-split greedy choice built on them (per-shard argmax records, 8 bytes per lane
gathered, merged on the device) against the host twins.  One process per GPU; the unique id travels through a file."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

RANK_SCRIPT = textwrap.dedent('''
    import os, sys, time, numpy as np
    sys.path.insert(0, os.environ["REPO_ROOT"])
    import __graft_entry__ as entry
    la = entry.load_package()
    rank, world, box = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), os.environ["ID_FILE"]
    ctx = la.CudaContext.new(rank)
    k = la.Kernels.new(ctx)
    assert la.Communicator.available()
    if rank == 0:
        uid = la.Communicator.unique_id()
        with open(box + ".tmp", "wb") as f:
            f.write(uid)
        os.rename(box + ".tmp", box)
    else:
        t0 = time.time()
        while not os.path.exists(box):
            assert time.time() - t0 < 60, "no unique id from rank 0"
            time.sleep(0.05)
        uid = open(box, "rb").read()
    comm = la.Communicator(ctx, uid, rank, world)
    # 1. plain all-gather, in place
    n = 4096
    mine = np.full(n, rank + 1, np.uint8)
    recv = la.CudaBuffer.from_slice(ctx, np.zeros(world * n, np.uint8))
    recv.copy_from_bytes(np.concatenate([mine if r == rank else np.zeros(n, np.uint8) for r in range(world)]))
    b = la.CommandBatch.new(ctx)
    comm.all_gather_into(b, recv, rank * n, recv, n)
    b.commit_and_wait()
    got = recv.as_slice(np.uint8)
    assert all(np.all(got[r * n:(r + 1) * n] == r + 1) for r in range(world)), got[::n]
    # 2. row-split greedy choice: every rank holds its rows' logits for all lanes
    lanes, vocab = 11, 4096
    logits = la.synth.normal(77, lanes * vocab).astype(np.float32).reshape(lanes, vocab)
    logits[1, 5] = logits[1, 4000] = 40.0
    logits[2, :] = -np.inf
    lo, hi = la.sharding.vocab_rows(vocab, world, rank)
    sl = la.CudaBuffer.from_slice(ctx, np.ascontiguousarray(logits[:, lo:hi]))
    pairs_all = la.CudaBuffer.from_slice(ctx, np.zeros(world * lanes * 8, np.uint8))
    tok = la.CudaBuffer.empty(ctx, lanes * 4)
    b = la.CommandBatch.new(ctx)
    mine_pairs = la.CudaBuffer.wrap(ctx, pairs_all.device_ptr + rank * lanes * 8, lanes * 8)
    k.argmax_pairs_f32_into(b, sl, mine_pairs, lanes, hi - lo, lo)
    comm.all_gather_into(b, pairs_all, rank * lanes * 8, pairs_all, lanes * 8)
    k.merge_argmax_pairs_into(b, pairs_all, tok, lanes, world)
    b.commit_and_wait()
    want = [int(np.argmax(logits[i])) if np.isfinite(logits[i]).any() else 0 for i in range(lanes)]
    assert tok.as_slice(np.uint32).tolist() == want
    recs = pairs_all.as_slice(np.uint8).view(la.sharding.PAIR_DTYPE).reshape(world, lanes)
    assert la.sharding.merge_argmax_pairs(recs).tolist() == want
    comm.close()
    print("rank", rank, "ok")
''')


def test_all_gather_and_row_split_argmax_on_two_gpus(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    env = dict(os.environ, REPO_ROOT=str(ROOT), WORLD_SIZE="2", ID_FILE=str(tmp_path / "nccl_id"), NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=240)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0] + "\\n(timed out)")
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-3000:]
