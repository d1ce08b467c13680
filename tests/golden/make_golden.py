"""Regenerates tests/golden/vectors.npz from the pinned CPU oracle (oracle/oracle.c).

The reference stores no output arrays of its own and cannot run here (Rust + Metal), so these vectors are the
oracle's answers on seeded inputs, frozen after the oracle was checked against every known-answer test the reference
holds for the path (tests/test_oracle_golden.py).  They guard the oracle against regressions (CPU test) and give the
CUDA path a fixed target that does not depend on the oracle being built (GPU test).

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

HD, N_KV, NTOK, N_Q = 256, 1, 12, 8
SEED = 0x7459C0DE


def inputs(synth):
    """Seeded inputs shared by the generator and the tests (counter-based splitmix64, see local-ai_b200/synth.py)."""
    return {
        "kv_rows": synth.normal_f16((NTOK, N_KV, HD), 901),
        "v_rows": synth.normal_f16((NTOK, N_KV, HD), 902, 0.7),
        "q": synth.normal_f16((N_Q, HD), 903),
        "w_q4": synth.q4_0_weights(48, 256, 904),
        "w_tq2": synth.tq2_0_weights(40, 512, 905, ncodes=4),
        "x256": synth.normal_f16((3, 256), 906),
        "x512": synth.normal_f16((3, 512), 907),
    }


def compute(orc, inp):
    out = {}
    signs = orc.tq_signs(HD, SEED)
    out["signs"] = signs
    for bits in (2, 3, 4):
        levels = orc.tq_levels(HD, bits)
        cb = orc.tq_code_bytes(HD, bits)
        out[f"levels{bits}"] = levels
        for name, rows in (("k", inp["kv_rows"]), ("v", inp["v_rows"])):
            codes, norms = np.zeros(NTOK * N_KV * cb, np.uint8), np.zeros(NTOK * N_KV, np.float16)
            orc.encode_kv(rows, levels, signs, codes, norms, HD, N_KV, NTOK, bits, 0, 0)
            out[f"{name}_codes{bits}"], out[f"{name}_norms{bits}"] = codes, norms.view(np.uint16)
        out[f"attn{bits}"] = orc.tq_attention_fused(
            inp["q"], out[f"k_codes{bits}"], out[f"k_norms{bits}"].view(np.float16), out[f"v_codes{bits}"],
            out[f"v_norms{bits}"].view(np.float16), levels, signs, None, HD, 0, N_Q, N_KV, 0, bits, 1, 0, 0.0625,
            kv_len=NTOK, current_pos=NTOK - 1).view(np.uint16)
    out["mm_q4"] = orc.matmul_nt(orc.Q4_0, inp["x256"], inp["w_q4"], 3, 256, 48)
    out["mm_tq2"] = orc.matmul_nt(orc.TQ2_0, inp["x512"], inp["w_tq2"], 3, 512, 40)
    return out


if __name__ == "__main__":
    la_synth = entry.load_package().synth
    orc = entry.load_oracle()
    vec = compute(orc, inputs(la_synth))
    np.savez_compressed(Path(__file__).with_name("vectors.npz"), **vec)
    print("wrote", Path(__file__).with_name("vectors.npz"), {k: v.shape for k, v in vec.items()})
