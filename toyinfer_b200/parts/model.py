"""A decoder described by data, and the object built from the description.

``ModelSpec`` holds what an architecture's ``describe(config)`` returns: the
embedding, the position encodings, one ``LayerSpec`` per layer (arrangement, norm,
mixer, feed-forward, each with its parameters), the schedule in which layers run,
the final norm and the head (or, for models whose ends differ from the usual, an
``embedding`` and a ``head`` part of their own: an embedding multiplier, a logit scale or
soft cap, no final norm).  The schedule is a list of ``ScheduleEntry``: an entry
names a layer (a layer may be named more than once: its weights are shared, each
entry has memory of its own) and may borrow the memory of an earlier entry
(``memory_of``), in which case its mixer reads what that entry stored.

``DecoderModel`` runs: the embedding part (src/prefill.cu:6-22), the scheduled blocks,
and for the rows whose logits are wanted the head part (parts/ends.py).  It also asks
every part, at build time and before any weight is read, whether the library's kernels
take its sizes (``Part.check_kernels``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .. import kernels as K
from ..tracing import ranged
from .base import BuildContext, ParamSpec, Part, PartSpec, build_part


@dataclass(frozen=True)
class LayerSpec:
    prefix: str                      # checkpoint prefix of the layer, e.g. "model.layers.3."
    block: PartSpec                  # arrangement; its params carry norm/mixer/feed_forward PartSpecs


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                       # index into ModelSpec.layers
    memory_of: Optional[int] = None  # index of an earlier entry whose memory this one reads


@dataclass
class ModelSpec:
    vocab_size: int
    hidden_size: int
    max_positions: int
    layers: List[LayerSpec]
    final_norm: Optional[PartSpec]                      # None: the head reads the hidden state as it is
    schedule: Optional[List[ScheduleEntry]] = None      # default: every layer once, in order
    positions: Dict[str, PartSpec] = field(default_factory=dict)
    tie_head: bool = False
    embed_name: str = "model.embed_tokens.weight"
    head_name: str = "lm_head.weight"
    final_norm_prefix: str = "model.norm."
    stop_token_ids: Tuple[int, ...] = ()
    ignorable: Tuple[str, ...] = ()                     # tensors a checkpoint may hold that are not used
    # The two ends as parts of their own; None: a plain token table (embed_name) and a linear head
    # (final_norm under final_norm_prefix, tie_head, head_name) without scales.
    embedding: Optional[PartSpec] = None
    head: Optional[PartSpec] = None

    def embedding_spec(self) -> PartSpec:
        if self.embedding is not None:
            return self.embedding
        return PartSpec("token_table", {"vocab_size": self.vocab_size, "name": self.embed_name})

    def head_spec(self) -> PartSpec:
        if self.head is not None:
            return self.head
        return PartSpec("linear", {"vocab_size": self.vocab_size, "norm": self.final_norm, "tied": self.tie_head,
                                   "name": self.head_name, "norm_prefix": self.final_norm_prefix})

    def run_order(self) -> List[ScheduleEntry]:
        if self.schedule is None:
            return [ScheduleEntry(i) for i in range(len(self.layers))]
        return list(self.schedule)


class DecoderModel(Part):
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        ctx = BuildContext(dtype=dtype, device=self.device, hidden_size=spec.hidden_size)
        for name, pspec in spec.positions.items():
            ctx.positions[name] = build_part("position", pspec, ctx, "")
        self.ctx = ctx
        self.embedding = build_part("embedding", spec.embedding_spec(), ctx, "")
        ctx.embedding = self.embedding
        self.blocks = [build_part("block", ls.block, ctx, ls.prefix) for ls in spec.layers]
        self.head = build_part("head", spec.head_spec(), ctx, "")
        self.schedule = spec.run_order()
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.blocks)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}; there are {len(self.blocks)}")
            if e.memory_of is not None:
                if not (0 <= e.memory_of < i):
                    raise ValueError(f"schedule entry {i} borrows memory of entry {e.memory_of}, which does not run before it")
                if self.schedule[e.memory_of].memory_of is not None:
                    raise ValueError(f"schedule entry {i} borrows from entry {e.memory_of}, which itself borrows")
        # every part says now, before any weight is read, whether the kernels take its sizes
        for part in [self.embedding, self.head, *self.ctx.positions.values(), *self.blocks]:
            part.check_kernels(dtype)

    # -- parameters ---------------------------------------------------------
    def param_specs(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = dict(self.embedding.param_specs())
        for b in self.blocks:
            out.update(b.param_specs())
        for p in self.ctx.positions.values():
            out.update(p.param_specs())
        out.update(self.head.param_specs())
        return out

    def ignorable_names(self) -> Tuple[str, ...]:
        return tuple(self.spec.ignorable) + tuple(self.head.ignorable_names())

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.embedding.bind(tensors)
        for p in self.ctx.positions.values():
            p.bind(tensors)
        for b in self.blocks:
            b.bind(tensors)
        self.head.bind(tensors)

    # -- what the cache must hold ---------------------------------------------
    def memory_requests(self) -> List[Any]:
        """One request (or None) per schedule entry; a borrowing entry asks for nothing."""
        out = []
        for e in self.schedule:
            out.append(None if e.memory_of is not None else self.blocks[e.layer].mixer.memory_request())
        return out

    def launch_plan(self, n_seq: int, plan_len: int, n_live: Optional[int] = None):
        """What of a captured single-token step depends on the length it is planned for and on how many
        of its sequences are real: the answers of all scheduled blocks (see Mixer.launch_plan)."""
        return tuple(self.blocks[e.layer].launch_plan(n_seq, plan_len, self.dtype, self.device, n_live) for e in self.schedule)

    def captures_start(self) -> bool:
        """Whether a step of whole prompts may be captured: every scheduled block says so."""
        return all(self.blocks[e.layer].captures_start for e in self.schedule)

    # -- one step -------------------------------------------------------------
    def forward_hidden(self, batch, memories: Sequence[Any]):
        """Runs the given tokens through all scheduled blocks.  Returns (h, delta):
        the hidden state is h + delta."""
        with ranged(batch, "embed"):
            h = self.embedding.forward(batch.token_ids)
        delta = None
        shared: List[dict] = [dict() for _ in self.schedule]
        owners = [i if e.memory_of is None else e.memory_of for i, e in enumerate(self.schedule)]
        last_use = {o: i for i, o in enumerate(owners)}
        for o, last in last_use.items():
            if last != o:
                shared[o]["deferred"] = []     # writes to the memory that must wait for its last reader
        for i, e in enumerate(self.schedule):
            owner = owners[i]
            h, delta = self.blocks[e.layer].forward(h, delta, batch, memories[owner], shared[owner])
            if last_use[owner] == i:
                for fn in shared[owner].get("deferred", ()):
                    fn()
                shared[owner].clear()      # what an entry left for its borrowers (this step's keys and values) is let go
        return h, delta

    def logits(self, h, delta, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] of the tokens at the given rows."""
        return self.head.forward(h, delta, rows)
