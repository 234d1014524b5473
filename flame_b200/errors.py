"""Error classes: the variants of the reference's ``Error`` enum that this path raises."""


class OffloadError(RuntimeError):
    """Base class (crate::Error)."""


class InvalidInput(OffloadError):
    """Error::InvalidInput: empty tensor, tensor larger than a slot, zero sizes."""


class InvalidOperation(OffloadError):
    """Error::InvalidOperation: pool full, stale handle, slot out of range, double pull."""


class InvalidShape(OffloadError):
    """Error::InvalidShape: an output tensor whose element count does not match the weight."""


class Unsupported(OffloadError):
    """Error::Unsupported: dtype the path does not move, compression of a non-BF16 tensor."""


class CudaError(OffloadError):
    """Error::Cuda: a CUDA runtime call returned an error code."""


class Timeout(OffloadError):
    """A bounded host wait ran out (no counterpart in the reference, which never waits)."""


def raise_for_status(status: int, message: str) -> None:
    if status == 0:
        return
    cls = {1: InvalidInput, 2: Unsupported, 3: CudaError, 4: Timeout, 5: InvalidOperation}.get(status, OffloadError)
    raise cls(message)
