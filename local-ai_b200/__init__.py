"""local-ai_b200: B200 (sm_100a) backend for local-ai's decode hot path.

The product is the C-ABI shared library built from `csrc/` (declared in
`include/local_cuda.h`).  This package is its host-side mirror of the
reference's `local-metal` interface plus seeded synthetic inputs.

The directory name carries a hyphen, so import it through the loader in
`__graft_entry__.load_package()`, which registers it as `local_ai_b200`.
"""
from .kernels import (  # noqa: F401
    TQ_SEED,
    CommandBatch,
    Communicator,
    CudaBuffer,
    CudaContext,
    CudaGraph,
    Error,
    Kernels,
    PendingCommandBuffer,
    PinnedHost,
    swa_ring_capacity,
    tq_code_bytes,
    tq_levels,
    tq_signs,
)
from . import synth  # noqa: F401
from . import model  # noqa: F401
from . import sharding  # noqa: F401
from .model import DecodeModel, ModelConfig, e2b_like_config  # noqa: F401
from .containers import LaneScheduler, QuantizedKvCache  # noqa: F401
