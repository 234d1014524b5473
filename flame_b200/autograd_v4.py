"""Shapes of what the reference's experimental autograd_v4 engine saves and the hook points around it.

Only the save-mode enum, the saved-tensor context, the statistics record and the
four hook slots are mirrored (src/autograd_v4/ops/sdpa.rs:48-96; tape and node
records, src/autograd_v4/graph.rs:12-66).  The attention math itself is a dense
contraction and is not part of the activation path.  ``SdpaCtx.offload`` /
``restore`` are the seam where this path attaches: a context's saved tensors go
through the installed pool exactly like a ``checkpoint_offload`` sub-tape entry.
"""
from __future__ import annotations

import enum
import threading
from dataclasses import dataclass, field
from typing import Callable, Optional


class SdpaSave(enum.Enum):
    SAVE_PROBS = "SaveProbs"
    SAVE_LSE = "SaveLSE"
    RECOMPUTE = "Recompute"


@dataclass
class SdpaStats:
    fwd_ms: float = 0.0
    bwd_ms: float = 0.0
    bytes_alloc: int = 0
    bytes_saved: int = 0
    nan_inf_hits: int = 0
    syncs: int = 0
    recompute_blocks: int = 0


@dataclass
class SdpaHooks:
    on_fwd_start: Callable = lambda cfg, shapes: None
    on_fwd_end: Callable = lambda stats: None
    on_bwd_start: Callable = lambda: None
    on_bwd_end: Callable = lambda stats: None


_SDPA_HOOKS: Optional[SdpaHooks] = None


def register_sdpa_hooks(hooks: SdpaHooks) -> bool:
    """Set once; returns False if hooks were already registered (sdpa.rs:76-79)."""
    global _SDPA_HOOKS
    if _SDPA_HOOKS is not None:
        return False
    _SDPA_HOOKS = hooks
    return True


@dataclass
class SdpaCtx:
    q: object
    k: object
    v: object
    attn_mask: Optional[object]
    scale: float
    save: SdpaSave
    causal: bool
    lse: Optional[object] = None      # [B,H,Q,1] FP32 if SaveLSE
    probs: Optional[object] = None    # [B,H,Q,K] BF16 if SaveProbs
    shapes: tuple = (0, 0, 0, 0)      # (B,H,Q,K)
    chunk_cfg: Optional[tuple] = None
    dropout_p: float = 0.0
    dropout_seed: Optional[int] = None
    _handles: dict = field(default_factory=dict, repr=False)

    _OFFLOADABLE = ("q", "k", "v", "probs")

    def offload(self, pool) -> int:
        """Pushes the BF16 saved tensors to `pool` and drops the device references; returns bytes offloaded."""
        import torch

        total = 0
        for name in self._OFFLOADABLE:
            t = getattr(self, name)
            if t is not None and t.dtype == torch.bfloat16 and t.is_contiguous():
                self._handles[name] = pool.push(t)
                setattr(self, name, None)
                total += t.numel() * 2
        return total

    def restore(self, pool) -> None:
        """Pulls back, in reverse push order, what `offload` pushed."""
        for name in reversed(list(self._handles)):
            setattr(self, name, pool.pull(self._handles.pop(name)))


@dataclass
class SdpaOp:
    """``Op::Sdpa { ctx, q_id, k_id, v_id }`` (graph.rs:12-19): the only backward op of the v4 engine."""

    ctx: SdpaCtx
    q_id: int
    k_id: int
    v_id: int


@dataclass
class GradNode:
    """Node of the backward tape (graph.rs:22-32)."""

    id: int
    parents: tuple
    op: SdpaOp


class Tape:
    """Nodes by tensor id plus their recording order (graph.rs:34-58)."""

    def __init__(self):
        self._nodes: dict = {}
        self._order: list = []

    def record(self, node: GradNode) -> None:
        self._order.append(node.id)
        self._nodes[node.id] = node

    def get(self, tensor_id: int) -> Optional[GradNode]:
        return self._nodes.get(tensor_id)

    def clear(self) -> None:
        self._nodes.clear()
        self._order.clear()

    def order(self) -> list:
        return self._order


_TLS = threading.local()


def _tape() -> Tape:
    if not hasattr(_TLS, "tape"):
        _TLS.tape = Tape()
    return _TLS.tape


def record_node(node: GradNode) -> None:
    """Thread-local tape, as graph.rs:60-66."""
    _tape().record(node)


def get_node(tensor_id: int) -> Optional[GradNode]:
    return _tape().get(tensor_id)


def clear_tape() -> None:
    _tape().clear()
