"""Interfaces of the parts a model is put together from.

A model is described by data (``ModelSpec`` in parts/model.py): for every layer a
block arrangement, a mixer, a feed-forward and a norm, each named by ``kind`` with
its sizes and constants as parameters, plus the order in which layers run.  A part
never learns which model it is in: it gets its parameters, the prefix of its
tensors' names, and a ``BuildContext``.

Families and what each must provide:

``Norm``            ``forward(x) -> y`` and ``add_forward(h, delta) -> y`` which
                    first does ``h += delta`` in place (32-bit sum, rounded once).
``PositionEncoding`` either ``rotary_tables() -> (cos, sin, rot_dim)`` for the fused
                    rotate-and-store kernel, or ``apply(q, k, tok_pos)`` in place.
``Mixer``           ``memory_request()`` says what the cache must keep for it (keys
                    and values, all or a window; a fixed-size state; nothing) and
                    ``forward(x, batch, mem, shared) -> y`` mixes ``x[M, hidden]``
                    along each sequence.  Sequence b of the step brings
                    ``batch.seq_new[b]`` tokens that follow ``batch.seq_start[b]``
                    positions already in ``mem``; any mix of the two is allowed, and a
                    mixer must be right for all of them.  ``batch.mode`` names two
                    special cases a mixer may run faster: ``"start"`` (every start is
                    0) and ``"extend"`` (one token each; device tensors only, since
                    such a step may be captured into a CUDA graph); anything else is
                    ``"mixed"``.  A mixer whose ``"start"`` steps read device tensors
                    only as well says so with ``captures_start = True``: repeated
                    prompt shapes are then captured too, if every part of the model
                    agrees.  ``shared`` is a dict that lives for one
                    step and belongs to the schedule entry that owns ``mem``; an
                    entry that borrows another entry's memory gets the owner's dict.
                    When it holds a list ``"deferred"``, later entries still read
                    ``mem``: a write that would destroy what they read is appended
                    there as a callable instead of being done.
``FeedForward``     ``forward(x, batch) -> y`` per token.
``Embedding``       ``forward(token_ids[M]) -> h[M, hidden]`` and ``table()`` (the matrix a
                    tied head reads).
``Head``            ``forward(h, delta, rows) -> float32 logits [len(rows), vocab]`` of
                    the tokens at ``rows``; the hidden state is ``h + delta``.
``Block``           owns norm(s), a mixer and a feed-forward and arranges them;
                    ``forward(h, delta, batch, mem, shared) -> (h, delta)`` where the
                    true hidden state is ``h + delta`` (``delta`` may be ``None``), so
                    that the sum can be fused into the next norm.

The reference has none of this: src/transformer.cpp:483-636 spells one fixed layer
out inline.  The formulas of the parts implemented here cite it part by part.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional, Tuple

import torch


# ---------------------------------------------------------------------------
# parameters
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class ParamSpec:
    """A tensor a part expects under a given checkpoint name.

    role: "matrix" (follows the engine's dtype), "norm" (follows the engine's
    dtype, but a tensor stored in 32-bit stays 32-bit), "int_table" (int32).
    init: "normal" N(0, std), "one_plus_normal" 1 + N(0, std), "zeros", "ones".
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    std: float = 0.02


@dataclass(frozen=True)
class PartSpec:
    """Which implementation of a family, and its sizes and constants."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass
class BuildContext:
    """What every part may know at build time: compute dtype, device, the model's
    width, and the position encodings built so far (by name)."""

    dtype: torch.dtype
    device: torch.device
    hidden_size: int
    positions: Dict[str, "PositionEncoding"] = field(default_factory=dict)
    embedding: Optional["Embedding"] = None       # the model's embedding, once built (a tied head reads its table)


class Part:
    """Base of all parts.  ``param_specs`` maps full checkpoint names to specs;
    ``bind`` receives the loaded tensors under the same names and may repack them
    (and should drop what it no longer needs)."""

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def check_kernels(self, dtype: torch.dtype) -> None:
        """Raises (kernels.KernelError, with the kernel's own message) when the library's kernels
        do not take this part's sizes in ``dtype``.  Called when a model is built, before weights
        are read; a part that owns other parts passes the call on."""


# ---------------------------------------------------------------------------
# what a mixer asks of the cache
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class KVRequest:
    """Keys and values per token: ``window == 0`` keeps all of them, otherwise only
    the last ``window`` positions are ever read."""

    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateRequest:
    """A state of fixed size per sequence, zero when the sequence starts."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Norm(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, h: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    def add_pending(self, h: torch.Tensor, delta: Optional[torch.Tensor]):
        """As add_forward, but may leave the work to the reader's first product: a
        kernels.PendingNorm instead of a tensor (only for readers that say takes_pending_norm)."""
        return self.add_forward(h, delta)


class PositionEncoding(Part):
    def rotary_tables(self) -> Optional[Tuple[torch.Tensor, torch.Tensor, int]]:
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, tok_pos: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    takes_pending_norm = False      # forward() may be given a kernels.PendingNorm, used by K.linear first
    captures_start = False          # a "start" step reads nothing of the batch's host side and allocates through torch
                                    # only: the engine may capture it (a class attribute or a property)

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        """What, of a captured single-token step of ``n_seq`` sequences of which ``n_live`` are real
        (the others are padding of one position), depends on the length the step is planned for and
        on ``n_live`` (a hashable value).  Steps share one captured graph when every mixer answers the
        same for them.  The default, the length itself, shares graphs between numbers of real
        sequences only."""
        return plan_len

    def memory_request(self):
        return None

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    takes_pending_norm = False      # as for Mixer
    captures_start = False          # as for Mixer

    def forward(self, x, batch) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    def table(self) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    def ignorable_names(self) -> Tuple[str, ...]:
        return ()

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        """As Mixer.launch_plan, for the whole block."""
        return self.mixer.launch_plan(n_seq, plan_len, dtype, device, n_live)

    @property
    def captures_start(self) -> bool:
        """As Mixer.captures_start, for the whole block; a block that knows of a feed-forward asks it too."""
        return bool(self.mixer.captures_start)

    def forward(self, h, delta, batch, mem, shared):
        raise NotImplementedError


# ---------------------------------------------------------------------------
# registries of implementations, one per family
# ---------------------------------------------------------------------------
FAMILIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
_REGISTRY: Dict[str, Dict[str, Callable[..., Part]]] = {f: {} for f in FAMILIES}


def register_part(family: str, kind: str, factory: Callable[..., Part], replace: bool = False) -> None:
    """Make ``factory(ctx=BuildContext, prefix=str, **params)`` available as
    ``PartSpec(kind, params)`` of the given family."""
    if family not in _REGISTRY:
        raise ValueError(f"unknown part family {family!r}; families: {FAMILIES}")
    if kind in _REGISTRY[family] and not replace:
        raise ValueError(f"{family} part {kind!r} is already registered")
    _REGISTRY[family][kind] = factory


def unregister_part(family: str, kind: str) -> None:
    _REGISTRY[family].pop(kind, None)


def registered_parts(family: str) -> Tuple[str, ...]:
    return tuple(sorted(_REGISTRY[family]))


def build_part(family: str, spec: PartSpec, ctx: BuildContext, prefix: str) -> Part:
    try:
        factory = _REGISTRY[family][spec.kind]
    except KeyError:
        raise ValueError(
            f"unknown {family} part {spec.kind!r}; registered: {', '.join(registered_parts(family)) or '(none)'}"
        ) from None
    return factory(ctx=ctx, prefix=prefix, **spec.params)
