"""Helpers for the GPU parity tests: guard-banded device buffers and tolerances."""
import numpy as np

CANARY = 0xA5
GUARD = 256  # bytes after the payload


class Guarded:
    """A device buffer with a canary band after the payload, checked after use
    (the stand-in for a memory checker: an out-of-bounds store shows up as a broken canary)."""

    def __init__(self, la, ctx, nbytes: int):
        self.nbytes = nbytes
        self.buf = la.CudaBuffer.from_slice(ctx, np.full(nbytes + GUARD, CANARY, dtype=np.uint8))
        # Present only the payload length to the library so its bounds checks stay exact.
        self.view = la.CudaBuffer.wrap(ctx, self.buf.device_ptr, nbytes)

    def read(self, dtype):
        raw = self.buf.as_slice(np.uint8)
        assert np.all(raw[self.nbytes:] == CANARY), "write past the end of the output buffer"
        return raw[: self.nbytes].view(dtype).copy()


def rel_close(got, want, tol, label=""):
    """|g - w| <= tol * max(|w|, 1): the reference's assert_close (kernels.rs:8871-8880)."""
    got = np.asarray(got, dtype=np.float32).reshape(-1)
    want = np.asarray(want, dtype=np.float32).reshape(-1)
    assert got.shape == want.shape, f"{label}: {got.shape} vs {want.shape}"
    err = np.abs(got - want)
    lim = tol * np.maximum(np.abs(want), 1.0)
    bad = np.flatnonzero(~(err <= lim))
    if bad.size:
        i = bad[np.argmax(err[bad])]
        raise AssertionError(f"{label}: {bad.size}/{got.size} off; worst [{i}] got {got[i]} want {want[i]} "
                             f"(err {err[i]:.3e}, max err {err.max():.3e})")
