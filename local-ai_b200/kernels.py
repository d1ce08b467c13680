"""Host-side mirror of local-metal's public types over the C ABI.

`CudaContext`, `CudaBuffer`, `CommandBatch`, `PendingCommandBuffer` and
`Kernels` carry the same method names, argument order and error behaviour as
`MetalContext` (local-metal/src/context.rs:31-101), `MetalBuffer`
(buffer.rs:17-144), `CommandBatch` / `PendingCommandBuffer` (batch.rs:120-292)
and `Kernels` (kernels.rs:18-6803), so a test written against the reference
reads the same here.  A failed call raises `Error` whose `kind` is the
reference's enum case (`InvalidArgument`, `BufferAllocation`, ...).

Every `Kernels` method is generated from the C header: `lc_<name>(kernels,
...)` becomes `Kernels.<name>(...)`.  Buffers, batches and contexts are passed
as the wrapper objects; scalars as Python numbers.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib


class Error(RuntimeError):
    """local_metal::Error (local-metal/src/error.rs:2-32) as an exception."""

    def __init__(self, status: int, message: str):
        lib = _lib.load()
        self.status = status
        self.kind = lib.lc_status_name(status).decode()
        super().__init__(f"{self.kind}: {message}")


def _check(status: int) -> None:
    if status != 0:
        raise Error(status, _lib.load().lc_last_error().decode())


def _handle(x):
    if x is None:
        return None
    h = getattr(x, "_h", None)
    if h is None:
        raise TypeError(f"expected a local-cuda object, got {type(x).__name__}")
    return h


class CudaContext:
    """MetalContext: one device, one in-order stream."""

    def __init__(self, device: int = 0):
        self._lib = _lib.load()
        h = C.c_void_p()
        _check(self._lib.lc_ctx_create(device, C.byref(h)))
        self._h = h
        self.device = device

    @classmethod
    def new(cls, device: int = 0) -> "CudaContext":
        return cls(device)

    def caps(self) -> dict:
        sm, smem, l2, tot = C.c_int(), C.c_size_t(), C.c_size_t(), C.c_size_t()
        _check(self._lib.lc_ctx_caps(self._h, C.byref(sm), C.byref(smem), C.byref(l2), C.byref(tot)))
        return {"sm_count": sm.value, "smem_per_cta": smem.value, "l2_bytes": l2.value, "total_mem": tot.value}

    @property
    def stream(self) -> int:
        return self._lib.lc_ctx_stream(self._h) or 0

    def synchronize(self) -> None:
        _check(self._lib.lc_ctx_synchronize(self._h))

    def close(self) -> None:
        if self._h:
            self._lib.lc_ctx_destroy(self._h)
            self._h = None


class CudaBuffer:
    """MetalBuffer.  Device memory; the CPU sees it through explicit copies."""

    def __init__(self, ctx: CudaContext, handle, nbytes: int):
        self._lib = ctx._lib
        self._ctx = ctx
        self._h = handle
        self.nbytes = nbytes

    @classmethod
    def from_slice(cls, ctx: CudaContext, data) -> "CudaBuffer":
        arr = np.ascontiguousarray(data)
        h = C.c_void_p()
        _check(ctx._lib.lc_buf_from_host(ctx._h, arr.ctypes.data, arr.nbytes, C.byref(h)))
        return cls(ctx, h, arr.nbytes)

    @classmethod
    def empty(cls, ctx: CudaContext, nbytes: int) -> "CudaBuffer":
        h = C.c_void_p()
        _check(ctx._lib.lc_buf_alloc(ctx._h, nbytes, C.byref(h)))
        return cls(ctx, h, nbytes)

    @classmethod
    def wrap(cls, ctx: CudaContext, device_ptr: int, nbytes: int) -> "CudaBuffer":
        h = C.c_void_p()
        _check(ctx._lib.lc_buf_wrap(ctx._h, device_ptr, nbytes, C.byref(h)))
        return cls(ctx, h, nbytes)

    def length(self) -> int:
        return self._lib.lc_buf_length(self._h)

    @property
    def device_ptr(self) -> int:
        return self._lib.lc_buf_device_ptr(self._h) or 0

    def as_slice(self, dtype, count: int | None = None, offset: int = 0) -> np.ndarray:
        """Copy `count` elements of `dtype` starting at byte `offset` to the host."""
        dt = np.dtype(dtype)
        if count is None:
            count = (self.nbytes - offset) // dt.itemsize
        out = np.empty(count, dtype=dt)
        _check(self._lib.lc_buf_download(self._h, offset, out.ctypes.data, out.nbytes))
        return out

    def copy_from_bytes(self, src, offset: int = 0) -> None:
        arr = np.ascontiguousarray(src)
        _check(self._lib.lc_buf_upload(self._h, offset, arr.ctypes.data, arr.nbytes))

    def zero(self, offset: int = 0, nbytes: int | None = None) -> None:
        _check(self._lib.lc_buf_zero(self._h, offset, self.nbytes - offset if nbytes is None else nbytes))

    def fill(self, value: int, offset: int = 0, nbytes: int | None = None) -> None:
        _check(self._lib.lc_buf_fill(self._h, offset, self.nbytes - offset if nbytes is None else nbytes, value))

    def free(self) -> None:
        if self._h:
            self._lib.lc_buf_free(self._h)
            self._h = None


class PendingCommandBuffer:
    def __init__(self, lib, handle):
        self._lib, self._h = lib, handle

    def wait(self) -> None:
        h, self._h = self._h, None
        _check(self._lib.lc_pending_wait(h))


class CudaGraph:
    """A captured batch that can be replayed (no twin in the reference)."""

    def __init__(self, lib, handle):
        self._lib, self._h = lib, handle

    def launch(self) -> None:
        _check(self._lib.lc_graph_launch(self._h))

    def destroy(self) -> None:
        if self._h:
            self._lib.lc_graph_destroy(self._h)
            self._h = None


class CommandBatch:
    """CommandBatch: dispatches run in encode order on the context's stream."""

    def __init__(self, ctx: CudaContext, capture: bool = False):
        self._lib = ctx._lib
        self._ctx = ctx
        h = C.c_void_p()
        fn = self._lib.lc_batch_begin_capture if capture else self._lib.lc_batch_begin
        _check(fn(ctx._h, C.byref(h)))
        self._h = h

    @classmethod
    def new(cls, ctx: CudaContext) -> "CommandBatch":
        return cls(ctx)

    @classmethod
    def capture(cls, ctx: CudaContext) -> "CommandBatch":
        return cls(ctx, capture=True)

    def dispatch_count(self) -> int:
        return self._lib.lc_batch_dispatch_count(self._h)

    def blit_buffer_copy(self, src: CudaBuffer, src_off: int, dst: CudaBuffer, dst_off: int, nbytes: int) -> None:
        _check(self._lib.lc_batch_copy(self._h, src._h, src_off, dst._h, dst_off, nbytes))

    def upload(self, dst: CudaBuffer, dst_off: int, host_ptr: int, nbytes: int) -> None:
        _check(self._lib.lc_batch_upload(self._h, dst._h, dst_off, host_ptr, nbytes))

    def download(self, src: CudaBuffer, src_off: int, host_ptr: int, nbytes: int) -> None:
        _check(self._lib.lc_batch_download(self._h, src._h, src_off, host_ptr, nbytes))

    def commit_and_wait(self) -> None:
        h, self._h = self._h, None
        _check(self._lib.lc_batch_commit_and_wait(h))

    def commit_async(self) -> PendingCommandBuffer:
        h, self._h = self._h, None
        p = C.c_void_p()
        _check(self._lib.lc_batch_commit_async(h, C.byref(p)))
        return PendingCommandBuffer(self._lib, p)

    def end_capture(self) -> CudaGraph:
        h, self._h = self._h, None
        g = C.c_void_p()
        _check(self._lib.lc_batch_end_capture(h, C.byref(g)))
        return CudaGraph(self._lib, g)


class PinnedHost:
    """Page-locked host array for asynchronous copies."""

    def __init__(self, nbytes: int, dtype=np.uint8):
        self._lib = _lib.load()
        p = C.c_void_p()
        _check(self._lib.lc_host_alloc(nbytes, C.byref(p)))
        self.ptr = p.value
        self.nbytes = nbytes
        buf = (C.c_uint8 * nbytes).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=dtype)

    def free(self) -> None:
        if self.ptr:
            self.array = None
            self._lib.lc_host_free(self.ptr)
            self.ptr = None


class Kernels:
    """Kernels (local-metal/src/kernels.rs): one method per dispatcher."""

    def __init__(self, ctx: CudaContext):
        self._lib = ctx._lib
        self._ctx = ctx
        h = C.c_void_p()
        _check(self._lib.lc_kernels_create(ctx._h, C.byref(h)))
        self._h = h

    @classmethod
    def new(cls, ctx: CudaContext) -> "Kernels":
        return cls(ctx)

    def close(self) -> None:
        if self._h:
            self._lib.lc_kernels_destroy(self._h)
            self._h = None


class Communicator:
    """NCCL behind the C ABI (lc_comm_*): one communicator per process / GPU.  `unique_id()` runs on one rank; the
    host carries the bytes to the others (a file, a socket, an existing process group); every rank then constructs
    its Communicator (collective)."""

    ID_BYTES = 128

    @staticmethod
    def available() -> bool:
        return _lib.load().lc_comm_available() == 0

    @staticmethod
    def unique_id() -> bytes:
        buf = (C.c_uint8 * Communicator.ID_BYTES)()
        _check(_lib.load().lc_comm_unique_id(buf))
        return bytes(buf)

    def __init__(self, ctx: CudaContext, uid: bytes, rank: int, world: int):
        assert len(uid) == self.ID_BYTES
        self._lib = ctx._lib
        self._ctx = ctx
        h = C.c_void_p()
        buf = (C.c_uint8 * self.ID_BYTES).from_buffer_copy(uid)
        _check(self._lib.lc_comm_create(ctx._h, buf, rank, world, C.byref(h)))
        self._h = h
        self.rank, self.world = rank, world

    def all_gather_into(self, batch, send: CudaBuffer, send_offset: int, recv: CudaBuffer, bytes_per_rank: int) -> None:
        _check(self._lib.lc_comm_all_gather_into(batch._h, self._h, send._h, send_offset, recv._h, bytes_per_rank))

    def close(self) -> None:
        if self._h:
            self._lib.lc_comm_destroy(self._h)
            self._h = None


def _make_method(cname: str, restype, argnames):
    def method(self, *args):
        if len(args) != len(argnames) - 1:
            raise TypeError(f"{cname[3:]}() takes {len(argnames) - 1} arguments ({', '.join(argnames[1:])}), got {len(args)}")
        conv = []
        for a in args:
            if isinstance(a, (list, tuple)):   # an array of handles (const lc_buf *const *)
                conv.append((C.c_void_p * len(a))(*[x._h for x in a]))
            else:
                conv.append(a._h if hasattr(a, "_h") else a)
        r = getattr(self._lib, cname)(self._h, *conv)
        if restype is C.c_int:
            _check(r)
            return None
        return r

    method.__name__ = cname[3:]
    method.__doc__ = f"{cname}({', '.join(argnames)}) from include/local_cuda.h"
    return method


def _install_kernel_methods() -> None:
    skip = {"lc_kernels_create", "lc_kernels_destroy"}
    for cname, (restype, argtypes, argnames) in _lib.declarations().items():
        if cname in skip or not argnames or argnames[0] != "k":
            continue
        setattr(Kernels, cname[3:], _make_method(cname, restype, argnames))


_install_kernel_methods()


# ---- host-side codec set-up (TurboQuant::new, turboquant.rs:187-199) ----
def tq_levels(dim: int, bits: int) -> np.ndarray:
    out = np.empty(1 << bits, dtype=np.float32)
    _check(_lib.load().lc_tq_levels(dim, bits, out.ctypes.data))
    return out


def tq_signs(dim: int, seed: int) -> np.ndarray:
    out = np.empty(dim, dtype=np.float32)
    _check(_lib.load().lc_tq_signs(dim, seed, out.ctypes.data))
    return out


def tq_code_bytes(dim: int, bits: int) -> int:
    return _lib.load().lc_tq_code_bytes(dim, bits)


def swa_ring_capacity(window: int, max_positions: int) -> int:
    return _lib.load().lc_swa_ring_capacity(window, max_positions)


TQ_SEED = 0x7459C0DE


def tq_attention_noalloc_into(batch: CommandBatch, q, k_codes, k_norms, v_codes, v_norms, levels, signs, attn_out,
                              head_dim, kv_len, current_pos, num_q_heads, num_kv_heads, window, bits, ring_capacity,
                              softmax_scale) -> None:
    """lc_tq_attention_noalloc_into: fused code-space attention whose split-K scratch is a fixed
    array inside the library, for callers that cannot allocate device memory (no `Kernels` needed)."""
    _check(_lib.load().lc_tq_attention_noalloc_into(
        batch._h, q._h, k_codes._h, k_norms._h, v_codes._h, v_norms._h, levels._h, signs._h, attn_out._h,
        head_dim, kv_len, current_pos, num_q_heads, num_kv_heads, window, bits, ring_capacity, softmax_scale))
