"""bench.py's contract, as far as it can be checked without a GPU: the reference arm runs on the host cores and
prints one JSON line with the agreed keys."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_the_contract_line():
    """Also: a launcher's OMP_NUM_THREADS=1 (torch.distributed.run exports it to every rank) must not throttle the
    CPU arm, and its config carries the main arm's keys."""
    import os
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "decode_b64_small",
                        "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    host = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    assert line["cpu_baseline"]["cores"] == host
    assert {"workload", "l2_policy", "launch", "replicas"} <= set(line["config"])
    assert line["impl"] == "reference" and line["metric"] == "decode_tok_s_batch64" and line["unit"] == "tok/s"
    assert line["higher_is_better"] is True and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"] and "model" not in line["config"]


def test_reference_arm_is_rank_zero_only():
    env = {"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29555"}
    import os
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                       capture_output=True, text=True, timeout=120, env=dict(os.environ, **env))
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_reference_arm_covers_the_attention_workloads():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "attention_2049x64",
                        "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["metric"] == "tq_decode_attention_hbm_gbs" and line["unit"] == "GB/s" and line["value"] > 0
