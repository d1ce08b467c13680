"""Python restatement of the deterministic generators and the closeness check
the reference's own kernel tests use, so the parity tests here run on the same
inputs (local-metal/src/kernels.rs:8776-8880; local-engine/src/turboquant.rs
:344-355; local-engine/src/kv_cache/quant_cache.rs:710-721)."""
import numpy as np


def xorshift_bytes(seed: int, n: int) -> np.ndarray:
    """kernels.rs:8776-8787: 32-bit xorshift from seed|1, byte = (s >> 8) as u8."""
    s = (seed | 1) & 0xFFFFFFFF
    out = np.empty(n, dtype=np.uint8)
    for i in range(n):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        out[i] = (s >> 8) & 0xFF
    return out


def q4_0_payload(rows: int, cols: int, seed: int):
    """kernels.rs:8790-8811 -> (raw bytes, f32 expansion [rows, cols])."""
    bpr = cols // 32
    rnd = xorshift_bytes(seed, rows * bpr * 17).reshape(rows * bpr, 17)
    d = (np.float32(0.01) + rnd[:, 0].astype(np.float32) / np.float32(2550.0)).astype(np.float16)
    raw = np.empty((rows * bpr, 18), dtype=np.uint8)
    raw[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    raw[:, 2:] = rnd[:, 1:]
    q = rnd[:, 1:].astype(np.int32)
    df = d.astype(np.float32)[:, None]
    dq = np.empty((rows * bpr, 32), dtype=np.float32)
    dq[:, :16] = ((q & 15) - 8).astype(np.float32) * df
    dq[:, 16:] = ((q >> 4) - 8).astype(np.float32) * df
    return raw.reshape(-1), dq.reshape(rows, cols)


def tq2_0_payload(rows: int, cols: int, seed: int):
    """kernels.rs:8814-8840 -> (raw bytes, f32 expansion). All four 2-bit codes occur."""
    bpr = cols // 256
    rnd = xorshift_bytes(seed, rows * bpr * 65).reshape(rows * bpr, 65)
    qs = rnd[:, :64]
    d = (np.float32(0.05) + rnd[:, 64].astype(np.float32) / np.float32(1275.0)).astype(np.float16)
    raw = np.empty((rows * bpr, 66), dtype=np.uint8)
    raw[:, :64] = qs
    raw[:, 64:] = d.view(np.uint8).reshape(-1, 2)
    dq = np.empty((rows * bpr, 256), dtype=np.float32)
    j = np.arange(64)
    base = (j >> 5) * 128 + (j & 31)
    df = d.astype(np.float32)[:, None]
    for l in range(4):
        dq[:, base + l * 32] = (((qs >> (2 * l)) & 3).astype(np.float32) - 1.0) * df
    return raw.reshape(-1), dq.reshape(rows, cols)


def tq2_0_repack_soa(raw: np.ndarray, rows: int, cols: int):
    """kernels.rs:8845-8855 -> (qs bytes, f16 scales)."""
    blk = raw.reshape(-1, 66)
    return np.ascontiguousarray(blk[:, :64]).reshape(-1), np.ascontiguousarray(blk[:, 64:]).reshape(-1).view(np.float16)


def test_vector(cols: int) -> np.ndarray:
    """kernels.rs:8857-8863: f16(sin(0.731 i)) with the product formed in f32."""
    i = np.arange(cols, dtype=np.float32)
    return np.sin((i * np.float32(0.731)).astype(np.float32)).astype(np.float16)


test_vector.__test__ = False


def sin_matrix(m: int, k: int, freq: float, amp: float, fn=np.sin) -> np.ndarray:
    """The activation generators of the matmul tests (kernels.rs:9445-9447, 9569-9571)."""
    i = np.arange(m * k, dtype=np.float32)
    return (fn((i * np.float32(freq)).astype(np.float32)) * np.float32(amp)).astype(np.float16).reshape(m, k)


def cpu_matvec(dq: np.ndarray, v: np.ndarray) -> np.ndarray:
    """kernels.rs:8865-8869 (f64 accumulate here; the GPU result is compared with a tolerance)."""
    return (dq.astype(np.float64) @ v.astype(np.float64)).astype(np.float32)


def assert_close(got, want, tol: float, label: str) -> None:
    """kernels.rs:8871-8880: |g - w| <= tol * max(|w|, 1) elementwise."""
    got = np.asarray(got, dtype=np.float32).reshape(-1)
    want = np.asarray(want, dtype=np.float32).reshape(-1)
    assert got.shape == want.shape, f"{label}: length {got.shape} vs {want.shape}"
    err = np.abs(got - want)
    lim = tol * np.maximum(np.abs(want), 1.0)
    bad = np.flatnonzero(~(err <= lim))
    assert bad.size == 0, f"{label}[{bad[0]}]: got {got[bad[0]]}, want {want[bad[0]]} ({bad.size} of {got.size} off)"


def seeded_vec(n: int, seed: int) -> np.ndarray:
    """turboquant.rs:344-355: values in [-0.5, 0.5) from a two-round splitmix."""
    s = (seed | 1) & 0xFFFFFFFFFFFFFFFF
    out = np.empty(n, dtype=np.float32)
    M = 0xFFFFFFFFFFFFFFFF
    for i in range(n):
        s = (s + 0x9E3779B97F4A7C15) & M
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z ^= z >> 31
        out[i] = np.float32(np.float32(z >> 40) / np.float32(1 << 24)) - np.float32(0.5)
    return out
