"""The lane admit / recycle loop (lc_lane_sched_*) as host logic, against a plain-Python restatement of
Pipeline::run_batched_to_completion (local-engine/src/pipeline/runner.rs:123-214) with prompts fed one token per step.
No GPU: the scheduler is created without a model, and the "decode step" is a deterministic function of (token, position)."""
import numpy as np
import pytest


def fake_step(tokens, positions, vocab=97):
    """Stand-in for a greedy decode step: a lane's next token depends only on its own token and position."""
    return ((tokens.astype(np.uint64) * 31 + positions.astype(np.uint64) * 7 + 3) % vocab).astype(np.uint32)


def reference_loop(requests, n_lanes, capacity, eos, vocab=97):
    """runner.rs:123-214 restated: admit in lane order, check_stop after every generated token, recycle finished lanes."""
    queue, lanes, results = list(requests), [None] * n_lanes, []
    while True:
        for lane in range(n_lanes):          # finalize (step 2 of the reference loop, folded before admission)
            s = lanes[lane]
            if s is not None and s["stop"]:
                results.append((s["id"], s["out"], s["stop"]))
                lanes[lane] = None
        for lane in range(n_lanes):          # admit
            if lanes[lane] is None and queue:
                rid, prompt, max_new = queue.pop(0)
                lanes[lane] = {"id": rid, "prompt": list(prompt), "fed": 0, "pos": 0, "last": 0, "out": [], "max_new": max(max_new, 1),
                               "stop": None}
        active = [l for l in range(n_lanes) if lanes[l] is not None]
        if not active:
            if not queue:
                break
            continue
        tokens, positions = np.zeros(n_lanes, np.uint32), np.zeros(n_lanes, np.uint32)
        for l in active:
            s = lanes[l]
            tokens[l] = s["prompt"][s["fed"]] if s["fed"] < len(s["prompt"]) else s["last"]
            positions[l] = s["pos"]
        nxt = fake_step(tokens, positions, vocab)
        for l in active:
            s = lanes[l]
            in_prompt = s["fed"] < len(s["prompt"])
            if in_prompt:
                s["fed"] += 1
            s["pos"] += 1
            if in_prompt and s["fed"] < len(s["prompt"]):
                continue
            t = int(nxt[l])
            s["out"].append(t)
            s["last"] = t
            cap = capacity - 1 if len(s["out"]) == 1 else capacity      # runner.rs:160-163 vs :207
            if t == eos:
                s["stop"] = "Eos"
            elif len(s["out"]) >= s["max_new"]:
                s["stop"] = "MaxTokens"
            elif s["pos"] >= cap:
                s["stop"] = "Capacity"
    return results


def run_library(la, requests, n_lanes, capacity, eos):
    sched = la.LaneScheduler(None, n_lanes, capacity, eos)
    for rid, prompt, max_new in requests:
        sched.submit(rid, prompt, max_new)
    results, steps = [], 0
    while True:
        active = sched.prepare()
        while (f := sched.pop_finished()) is not None:
            results.append((f[0], list(map(int, f[1])), f[2]))
        if active == 0:
            assert sched.pending() == 0
            break
        idle = [l for l in range(n_lanes) if sched.positions[l] == 0 and sched.tokens[l] == 0]
        assert len(idle) >= n_lanes - active          # idle lanes carry token 0 at position 0
        sched.consume(fake_step(sched.tokens, sched.positions))
        steps += 1
        assert steps < 10_000
    sched.close()
    return results


@pytest.mark.parametrize("n_lanes,capacity", [(2, 24), (4, 12), (1, 40)])
def test_scheduler_matches_the_reference_loop(la, n_lanes, capacity):
    rng = np.random.default_rng(n_lanes * 100 + capacity)
    requests = []
    for rid in range(11):
        plen = int(rng.integers(1, min(capacity, 9)))
        requests.append((1000 + rid, rng.integers(1, 97, plen).astype(np.uint32), int(rng.integers(1, 20))))
    eos = 5
    want = reference_loop(requests, n_lanes, capacity, eos)
    got = run_library(la, requests, n_lanes, capacity, eos)
    assert [(r[0], list(r[1]), r[2]) for r in want] == got
    reasons = {r[2] for r in got}
    assert len(got) == len(requests) and "MaxTokens" in reasons


def test_stop_reasons_and_rejections(la):
    sched = la.LaneScheduler(None, 1, 6, eos_token=96)
    with pytest.raises(la.Error) as ei:
        sched.submit(1, np.arange(1, 8, dtype=np.uint32), 4)     # 7 tokens in a 6-row lane
    assert ei.value.kind == "InvalidArgument"
    with pytest.raises(la.Error):
        sched.submit(2, np.zeros(0, np.uint32), 4)
    sched.submit(3, np.array([4, 9, 2], np.uint32), 100)         # runs into the lane capacity
    out = None
    for _ in range(50):
        if sched.prepare() == 0:
            break
        sched.consume(fake_step(sched.tokens, sched.positions, vocab=90))   # never 96: no EOS
    out = sched.pop_finished()
    assert out is not None and out[0] == 3 and out[2] == "Capacity"
    # prompt at 0..2, first token generated with pos = 3, then one token per position until pos reaches 6
    assert len(out[1]) == 4
    sched.close()
