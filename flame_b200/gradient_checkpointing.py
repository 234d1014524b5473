"""CheckpointManager and friends: mirror of src/gradient_checkpointing.rs:19-358.

The reference's manager is a side channel consulted per saved tensor
(src/autograd.rs:894-907, 1867-1880); ``checkpoint_offload``'s save and restore
hooks consult this one the same way, behind ``CHECKPOINT_HAS_ENTRIES``.  Its ``CPUOffload`` policy is a device-side
clone placeholder (gradient_checkpointing.rs:92-97); here it really offloads
through the installed ``ActivationOffloadPool`` when there is one, and keeps the
clone behaviour when there is not.  ``Adaptive`` keeps its two fields and its
byte-counter rule; the measured-bandwidth planner lives in ``flame_b200.policy``.
"""
from __future__ import annotations

import enum
import itertools
import threading
import weakref
from dataclasses import dataclass
from typing import Callable, Optional

from . import checkpoint as _ckpt
from .errors import InvalidOperation


_NEXT_TENSOR_ID = itertools.count(1)


def tensor_id(t):
    """Identity of a tensor for the manager's registry (the reference's TensorId): a number given to the tensor
    object the first time it is asked for and kept on it.  Never derived from the address: a checkpointed block
    frees its saved tensors as it offloads them, and the allocator hands the same address to the next block's."""
    tid = getattr(t, "_flame_tensor_id", None)
    if tid is None:
        tid = next(_NEXT_TENSOR_ID)
        t._flame_tensor_id = tid
    return tid


class CheckpointPolicyKind(enum.Enum):
    CPU_OFFLOAD = "CPUOffload"
    RECOMPUTE = "Recompute"
    ADAPTIVE = "Adaptive"


@dataclass(frozen=True)
class CheckpointPolicy:
    """``CPUOffload`` | ``Recompute`` | ``Adaptive { memory_threshold, prefer_recompute }`` (gradient_checkpointing.rs:62-75)."""

    kind: CheckpointPolicyKind
    memory_threshold: int = 0
    prefer_recompute: bool = False

    @staticmethod
    def cpu_offload() -> "CheckpointPolicy":
        return CheckpointPolicy(CheckpointPolicyKind.CPU_OFFLOAD)

    @staticmethod
    def recompute() -> "CheckpointPolicy":
        return CheckpointPolicy(CheckpointPolicyKind.RECOMPUTE)

    @staticmethod
    def adaptive(memory_threshold: int, prefer_recompute: bool) -> "CheckpointPolicy":
        return CheckpointPolicy(CheckpointPolicyKind.ADAPTIVE, memory_threshold, prefer_recompute)


@dataclass
class CheckpointStats:
    memory_saved: int
    recompute_count: int
    checkpointed_tensors: int


class _OnDevice:
    def __init__(self, tensor):
        self.tensor = tensor


class _Offloaded:
    def __init__(self, pool, handle):
        self.pool, self.handle = pool, handle


class _Deleted:
    def __init__(self, compute_fn, shape, dtype):
        self.compute_fn, self.shape, self.dtype = compute_fn, shape, dtype


class CheckpointManager:
    def __init__(self):
        self._saved: dict = {}
        self._policy = CheckpointPolicy.recompute()  # gradient_checkpointing.rs:81
        self._device = None
        self._memory_saved = 0
        self._recompute_count = 0
        self._registry: dict = {}

    def _store(self, tensor):
        pool = _ckpt.activation_offload_pool()
        if pool is not None and tensor.is_cuda and tensor.is_contiguous():
            try:
                return _Offloaded(pool, pool.push(tensor))
            except Exception:
                pass
        return _OnDevice(tensor.clone())

    def _has_entries(self) -> None:
        global CHECKPOINT_HAS_ENTRIES
        CHECKPOINT_HAS_ENTRIES = bool(self._saved)

    def checkpoint_saved_tensor(self, tensor_id, tensor) -> None:
        if self._policy.kind == CheckpointPolicyKind.CPU_OFFLOAD:
            self._saved[tensor_id] = self._store(tensor)
            self._has_entries()

    def set_recompute_for(self, tensor_id, shape, dtype, compute_fn: Callable) -> None:
        self._saved[tensor_id] = _Deleted(compute_fn, shape, dtype)
        self._has_entries()

    def fetch_saved(self, tensor_id, device=None):
        """Some(restored) if a checkpoint exists, else None; the entry stays (gradient_checkpointing.rs:126-145)."""
        e = self._saved.get(tensor_id)
        if e is None:
            return None
        if isinstance(e, _OnDevice):
            return e.tensor.clone()
        if isinstance(e, _Offloaded):
            t = e.pool.pull(e.handle)
            self._saved[tensor_id] = _OnDevice(t)  # a handle can be pulled once
            return t.clone()
        return e.compute_fn()

    def set_policy(self, policy: CheckpointPolicy) -> None:
        self._policy = policy

    def set_device(self, device) -> None:
        self._device = device

    def register_tensor(self, tensor_id, tensor) -> None:
        self._registry[tensor_id] = weakref.ref(tensor)

    def checkpoint_tensor(self, tensor_id, compute_fn: Optional[Callable] = None) -> None:
        ref = self._registry.get(tensor_id)
        tensor = ref() if ref is not None else None
        if tensor is None:
            raise InvalidOperation("Tensor not found in registry")
        kind = self._policy.kind
        if kind == CheckpointPolicyKind.CPU_OFFLOAD:
            self._saved[tensor_id] = self._store(tensor)
        elif kind == CheckpointPolicyKind.RECOMPUTE:
            if compute_fn is not None:
                self._saved[tensor_id] = _Deleted(compute_fn, tuple(tensor.shape), tensor.dtype)
                self._memory_saved += tensor.numel() * 4
        else:
            if self._memory_saved < self._policy.memory_threshold and self._policy.prefer_recompute:
                if compute_fn is not None:
                    self._saved[tensor_id] = _Deleted(compute_fn, tuple(tensor.shape), tensor.dtype)
                    self._memory_saved += tensor.numel() * 4
            else:
                self._saved[tensor_id] = self._store(tensor)
                self._memory_saved += tensor.numel() * 2
        self._has_entries()

    def restore_tensor(self, tensor_id):
        e = self._saved.pop(tensor_id, None)
        if e is None:
            raise InvalidOperation("Checkpointed tensor not found")
        if self._device is None:
            raise InvalidOperation("Device not set")
        self._has_entries()
        if isinstance(e, _OnDevice):
            return e.tensor.clone()
        if isinstance(e, _Offloaded):
            return e.pool.pull(e.handle)
        self._recompute_count += 1
        return e.compute_fn()

    def stats(self) -> CheckpointStats:
        return CheckpointStats(self._memory_saved, self._recompute_count, len(self._saved))

    def clear(self) -> None:
        for e in self._saved.values():
            if isinstance(e, _Offloaded):
                try:
                    e.pool.discard(e.handle)
                except Exception:
                    pass
        self._saved.clear()
        self._memory_saved = 0
        self._recompute_count = 0
        self._has_entries()


CHECKPOINT_MANAGER = CheckpointManager()
CHECKPOINT_MANAGER_LOCK = threading.RLock()   # re-entrant: a CheckpointedBlock holds it while its forward runs the save hooks
CHECKPOINT_HAS_ENTRIES = False


class CheckpointedBlock:
    """Wrapper that runs a block's forward and hands its intermediate outputs to the manager
    (gradient_checkpointing.rs:278-327)."""

    def __init__(self, block_name: str, forward_fn: Callable):
        self.block_name, self.forward_fn = block_name, forward_fn

    def forward(self, inputs):
        with CHECKPOINT_MANAGER_LOCK:
            outputs = self.forward_fn(inputs)
            for i, out in enumerate(outputs):
                if i < len(outputs) - 1:  # the final output is not checkpointed
                    CHECKPOINT_MANAGER.register_tensor(tensor_id(out), out)
                    CHECKPOINT_MANAGER.checkpoint_tensor(tensor_id(out), None)
            return outputs


class CheckpointableModel:
    """Trait of models that can switch checkpointing on and off (gradient_checkpointing.rs:341-345)."""

    def enable_checkpointing(self) -> None:
        raise NotImplementedError

    def disable_checkpointing(self) -> None:
        raise NotImplementedError


def enable_gradient_checkpointing(model: CheckpointableModel, policy: CheckpointPolicy) -> None:
    with CHECKPOINT_MANAGER_LOCK:
        CHECKPOINT_MANAGER.set_policy(policy)
    model.enable_checkpointing()
