"""The C ABI loads, exports every symbol its header declares, and its host-side
pieces (error reporting, codec set-up) behave like the reference's. No GPU
compute is issued here."""
import ctypes as C
import os

import numpy as np
import pytest


def test_header_declares_the_dispatch_surface(la):
    decls = la._lib.declarations()
    assert len(decls) >= 80
    for name in ("lc_matvec_q4_0_into", "lc_matvec_tq2_0_f32out", "lc_matmul_nt_tq2_0_into",
                 "lc_encode_kv_turboquant_batched_into", "lc_flash_attention_tq_batched_into",
                 "lc_flash_decoding_into", "lc_attention_sliding", "lc_hadamard_rotate_hf_into",
                 "lc_tq2_dequant", "lc_batch_commit_and_wait", "lc_buf_upload"):
        assert name in decls, name


def test_library_exports_every_declared_symbol(la):
    lib = la._lib.load()  # raises if a declared symbol is missing
    for name in la._lib.declarations():
        assert getattr(lib, name) is not None
    assert lib.lc_version().decode().endswith("sm_100a")


def test_kernels_mirror_has_reference_method_names(la):
    for name in ("matvec_q4_0", "matvec_q4_0_into", "matvec_tq2_0_f32out_into", "matvec_tq2_0_soa_into",
                 "matmul_nt_q4_0_into", "multivec_nt_tq2_0_into", "encode_kv_turboquant",
                 "dequantize_kv_turboquant_into", "hadamard_rotate_fh_into", "flash_attention_tq_into",
                 "flash_split_count", "rms_norm_add_into", "rope_batch_decode_into", "gelu_mul_into"):
        assert callable(getattr(la.Kernels, name)), name


def test_null_arguments_are_reported_not_crashed(la):
    lib = la._lib.load()
    out = C.c_void_p()
    assert lib.lc_buf_alloc(None, 16, C.byref(out)) == 8  # InvalidArgument
    assert b"NULL" in lib.lc_last_error()
    assert lib.lc_status_name(8) == b"InvalidArgument"
    assert lib.lc_batch_begin(None, C.byref(out)) == 8
    assert lib.lc_matvec_q4_0_into(None, None, None, None, None, 1, 32) == 8
    assert lib.lc_tq_levels(256, 9, None) == 8


def test_no_device_is_an_error_not_a_fallback(la):
    try:
        ctx = la.CudaContext.new(0)
    except la.Error as e:
        assert e.kind == "NoDevice"
        return
    ctx.close()
    pytest.skip("a CUDA device is present")


def test_device_ordinal_out_of_range(la):
    with pytest.raises(la.Error) as ei:
        la.CudaContext.new(4096)
    assert ei.value.kind == "NoDevice"


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("dim", [64, 128, 256, 512])
def test_codec_setup_is_bit_identical_to_oracle(la, orc, dim, bits):
    assert np.array_equal(la.tq_levels(dim, bits), orc.tq_levels(dim, bits))
    assert np.array_equal(la.tq_signs(dim, la.TQ_SEED), orc.tq_signs(dim, la.TQ_SEED))
    assert la.tq_code_bytes(dim, bits) == orc.tq_code_bytes(dim, bits) == dim * bits // 8


def test_ring_capacity_and_kv_bits_env(la, orc, monkeypatch):
    for w, mp in ((512, 131072), (512, 600), (1024, 8192), (100, 1 << 20)):
        assert la.swa_ring_capacity(w, mp) == orc.swa_ring_capacity(w, mp)
    assert la.swa_ring_capacity(512, 131072) == 1024
    lib = la._lib.load()
    for val, want in ((None, 2), ("tq2", 2), ("tq3", 3), ("tq4", 4), ("bogus", 2)):
        if val is None:
            monkeypatch.delenv("LOCAL_AI_KV_QUANT", raising=False)
        else:
            monkeypatch.setenv("LOCAL_AI_KV_QUANT", val)
        assert lib.lc_kv_bits_from_env() == want


def test_product_never_imports_the_oracle():
    """The shipped package must not reach into oracle/ (it is the checker, not a fallback)."""
    import pathlib
    pkg = pathlib.Path(__file__).resolve().parent.parent / "local-ai_b200"
    for f in list(pkg.glob("*.py")) + list((pkg / "csrc").glob("*")):
        text = f.read_text(errors="ignore")
        assert "oracle" not in text.lower(), f.name
