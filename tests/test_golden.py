"""Frozen answers of the pinned oracle on seeded inputs (tests/golden/vectors.npz, written by
tests/golden/make_golden.py): the oracle must keep reproducing them (CPU), and the CUDA path must meet them through
the C ABI (GPU) — packed codes and norms bit for bit, contractions and attention within the stated tolerance."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest

from gpu_util import Guarded, rel_close

GOLD = Path(__file__).parent / "golden"
spec = importlib.util.spec_from_file_location("make_golden", GOLD / "make_golden.py")
mg = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mg)


@pytest.fixture(scope="module")
def gold():
    return dict(np.load(GOLD / "vectors.npz"))


def test_oracle_reproduces_golden_vectors(la, orc, gold):
    got = mg.compute(orc, mg.inputs(la.synth))
    assert set(got) == set(gold)
    for name, want in gold.items():
        assert np.array_equal(np.asarray(got[name]).view(np.uint8), want.view(np.uint8)), name


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [2, 3, 4])
def test_cuda_encode_and_attention_meet_golden(la, ctx, kernels, gold, bits):
    inp = mg.inputs(la.synth)
    hd, n_kv, ntok, n_q = mg.HD, mg.N_KV, mg.NTOK, mg.N_Q
    levels, signs = la.tq_levels(hd, bits), la.tq_signs(hd, mg.SEED)
    assert np.array_equal(levels.view(np.uint32), gold[f"levels{bits}"].view(np.uint32))
    assert np.array_equal(signs.view(np.uint32), gold["signs"].view(np.uint32))
    cb = la.tq_code_bytes(hd, bits)
    d = lambda a: la.CudaBuffer.from_slice(ctx, a)
    bufs = {}
    for name, rows in (("k", inp["kv_rows"]), ("v", inp["v_rows"])):
        codes, norms = Guarded(la, ctx, ntok * n_kv * cb), Guarded(la, ctx, ntok * n_kv * 2)
        kernels.encode_kv_turboquant(ctx, d(rows), d(levels), d(signs), codes.view, norms.view, hd, n_kv, ntok, bits, 0, 0)
        assert np.array_equal(codes.read(np.uint8), gold[f"{name}_codes{bits}"]), f"{name} codes tq{bits}"
        assert np.array_equal(norms.read(np.uint16), gold[f"{name}_norms{bits}"]), f"{name} norms tq{bits}"
        bufs[name] = (codes, norms)
    out = Guarded(la, ctx, n_q * hd * 2)
    b = la.CommandBatch.new(ctx)
    kernels.tq_attention_into(b, d(inp["q"]), bufs["k"][0].view, bufs["k"][1].view, bufs["v"][0].view, bufs["v"][1].view,
                              d(levels), d(signs), out.view, hd, ntok, ntok - 1, n_q, n_kv, 0, bits, 0, 0.0625)
    b.commit_and_wait()
    rel_close(out.read(np.float16), gold[f"attn{bits}"].view(np.float16).astype(np.float32), 2e-3, f"attention tq{bits}")


@pytest.mark.gpu
def test_cuda_matmul_meets_golden(la, ctx, kernels, gold):
    inp = mg.inputs(la.synth)
    for name, w, x, k, n, fn in (("mm_q4", inp["w_q4"], inp["x256"], 256, 48, "matmul_nt_q4_0_into"),
                                 ("mm_tq2", inp["w_tq2"], inp["x512"], 512, 40, "matmul_nt_tq2_0_into")):
        out = Guarded(la, ctx, 3 * n * 2)
        b = la.CommandBatch.new(ctx)
        getattr(kernels, fn)(b, la.CudaBuffer.from_slice(ctx, x), la.CudaBuffer.from_slice(ctx, w), out.view, 3, k, n)
        b.commit_and_wait()
        rel_close(out.read(np.float16).astype(np.float32).reshape(3, n), gold[name], 1e-3, name)
