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

    _OFFLOADABLE = ("q", "k", "v", "probs", "lse")

    @classmethod
    def from_forward(cls, q, k, v, *, scale: float, save: SdpaSave, causal: bool = False, attn_mask=None,
                     probs=None, lse=None, chunk_cfg=None, dropout_p: float = 0.0, dropout_seed=None) -> "SdpaCtx":
        """The record ``sdpa_forward`` leaves for backward (sdpa.rs:260-274): q, k, v always; the probabilities
        [B,H,Q,K] in BF16 only under ``SaveProbs``; the log-sum-exp [B,H,Q,1] in FP32 only under ``SaveLSE``;
        neither under ``Recompute``.  What does not belong to the mode is refused, so that a context never holds
        more than its mode says it saves."""
        import torch

        b, h, ql, _ = q.shape
        kl = k.shape[2]
        if save == SdpaSave.SAVE_PROBS:
            if probs is None or lse is not None or tuple(probs.shape) != (b, h, ql, kl) or probs.dtype != torch.bfloat16:
                raise ValueError("SaveProbs keeps the probabilities [B,H,Q,K] in BF16 and no log-sum-exp")
        elif save == SdpaSave.SAVE_LSE:
            if lse is None or probs is not None or tuple(lse.shape) != (b, h, ql, 1) or lse.dtype != torch.float32:
                raise ValueError("SaveLSE keeps the log-sum-exp [B,H,Q,1] in FP32 and no probabilities")
        elif probs is not None or lse is not None:
            raise ValueError("Recompute keeps neither probabilities nor log-sum-exp")
        return cls(q=q, k=k, v=v, attn_mask=attn_mask, scale=float(scale), save=save, causal=causal, lse=lse, probs=probs,
                   shapes=(b, h, ql, kl), chunk_cfg=chunk_cfg, dropout_p=dropout_p, dropout_seed=dropout_seed)

    def saved_bytes(self) -> int:
        """Bytes the context keeps on the device right now (what SdpaStats.bytes_saved counts)."""
        return sum(t.numel() * t.element_size() for t in (getattr(self, n) for n in self._OFFLOADABLE) if t is not None)

    def offload(self, pool) -> int:
        """Pushes the saved tensors to `pool` and drops the device references; returns the bytes offloaded.

        BF16 tensors go through whatever compression the pool has; the FP32 log-sum-exp only through an
        uncompressed pool (compression is defined for BF16 only, src/activation_offload.rs:537-542) and stays
        resident otherwise.  A tensor that is not contiguous stays resident too."""
        import torch

        compressed = int(getattr(pool, "compression", 0)) != 0
        total = 0
        for name in self._OFFLOADABLE:
            t = getattr(self, name)
            if t is None or not t.is_contiguous():
                continue
            if t.dtype == torch.bfloat16 or (t.dtype == torch.float32 and not compressed):
                self._handles[name] = pool.push(t)
                setattr(self, name, None)
                total += t.numel() * t.element_size()
        return total

    def restore(self, pool) -> None:
        """Pulls back, in reverse push order (the pool's slot stack is last in, first out), what `offload` pushed."""
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
