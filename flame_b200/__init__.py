"""B200-native activation offload/restore path behind the flame-core API.

Only what the hot path needs: the CUDA kernels and C ABI (``csrc/``,
``libflame_offload.so``), and Python mirrors of the reference interface
(``ActivationOffloadPool``, ``PinnedHostBuffer``, ``PinnedPool``,
``CheckpointPolicy`` / ``CheckpointManager``, ``checkpoint_offload``, and
``BlockOffloader`` for block weights streamed through the same pool).

Importing the package does not load CUDA.  Every operation goes through the
shared library; there is no CPU or eager fallback, and a missing library is an
ImportError.
"""
from .pinned import PinnedAllocFlags, PinnedHostBuffer, StagingDeviceBuf  # noqa: F401
from .pinned_pool import PinnedPool  # noqa: F401
from .activation_offload import (  # noqa: F401
    ActivationOffloadPool,
    OffloadCompression,
    OffloadHandle,
    OffloadError,
    InvalidInput,
    InvalidOperation,
    Unsupported,
    CudaError,
)
from .errors import InvalidShape  # noqa: F401

from .block_offload import BlockOffloader  # noqa: F401,E402

__all__ = [
    "BlockOffloader",
    "PinnedAllocFlags", "PinnedHostBuffer", "StagingDeviceBuf", "PinnedPool",
    "ActivationOffloadPool", "OffloadCompression", "OffloadHandle",
    "OffloadError", "InvalidInput", "InvalidOperation", "InvalidShape", "Unsupported", "CudaError",
]
