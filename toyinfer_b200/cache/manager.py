"""The cache: a slot per sequence, keys and values per layer in pages, and a
fixed-size state per sequence beside them.

Every schedule entry of the model that owns memory says what it needs
(parts.base.KVRequest or StateRequest).  Entries with the same key/value needs
(kv heads, head size, window) form a group with storage of its own:

  k, v            [entries, pages + 1, kv_heads, PAGE, head_dim]   engine dtype
  page table      [slots + 1, pages per sequence]                  int32

A sequence's position p lives in row (p mod PAGE) of page ``table[slot][p // PAGE]``.
A group with a window keeps a ring of ``ring_rows`` >= window positions per sequence
(position p at ring row p mod ring_rows), so its sequences never hold more than
``ring_rows / PAGE`` pages.  Page 0 and slot ``n_slots`` are scratch: padding of a
step points there and what it writes is never read.

Fixed-size states live in one tensor per entry, [slots + 1, *shape], and are zeroed
when a slot is handed out.  This architecture asks for none; the area exists so that a
mixer with a state can be added without touching the cache.

The reference keeps one sequence's keys and values as [layers, max_seq_len, kv_dim]
(src/transformer.cpp:188-195) and the position in a host variable
(src/engine_runtime.cpp:441).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import KVRequest, StateRequest
from .allocators import PAGE, CacheError, PagePool, SlotAllocator


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


@dataclass
class KVView:
    """What a mixer's kernels need to reach one entry's keys and values."""

    k_pages: torch.Tensor          # [pages + 1, kv_heads, PAGE, head_dim]
    v_pages: torch.Tensor
    page_table: torch.Tensor       # [slots + 1, pages_per_seq] int32, on the device
    n_kv_heads: int
    head_dim: int
    window: int                    # 0: all positions kept
    ring_rows: int                 # 0: position p is row p; else row p mod ring_rows
    page_size: int = PAGE


@dataclass
class StateView:
    state: torch.Tensor            # [slots + 1, *shape]


class _KVGroup:
    def __init__(self, req: KVRequest, entries: List[int], n_slots: int, max_tokens: int,
                 max_seq_len: int, dtype, device):
        self.req = req
        self.entries = entries
        self.ring_pages = pages_for(req.window) if req.window > 0 else 0
        self.ring_rows = self.ring_pages * PAGE
        self.pages_per_seq = pages_for(max_seq_len)
        if self.ring_pages:
            self.pages_per_seq = min(self.pages_per_seq, self.ring_pages)
        n_pages = pages_for(max_tokens)
        if self.ring_pages:
            n_pages = min(n_pages, n_slots * self.ring_pages)
        self.pool = PagePool(n_pages)
        shape = (len(entries), n_pages + 1, req.n_kv_heads, PAGE, req.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.table_host = np.zeros((n_slots + 1, self.pages_per_seq), dtype=np.int32)
        self.table = torch.zeros((n_slots + 1, self.pages_per_seq), dtype=torch.int32, device=device)
        self.slot_pages: Dict[int, List[int]] = {}
        self.dirty: Dict[int, Tuple[int, int]] = {}

    def pages_needed(self, length: int) -> int:
        n = pages_for(length)
        return min(n, self.ring_pages) if self.ring_pages else n

    def grow(self, slot: int, length: int) -> None:
        have = self.slot_pages.setdefault(slot, [])
        need = self.pages_needed(length)
        if need > self.pages_per_seq:
            raise CacheError(
                f"a sequence of {length} positions needs {need} pages; the cache was sized for "
                f"{self.pages_per_seq} per sequence"
            )
        if need > len(have):
            new = self.pool.allocate(need - len(have))
            a = len(have)
            have.extend(new)
            self.table_host[slot, a:need] = new
            lo, hi = self.dirty.get(slot, (a, need))
            self.dirty[slot] = (min(lo, a), max(hi, need))

    def drop(self, slot: int) -> None:
        pages = self.slot_pages.pop(slot, [])
        self.pool.release(pages)
        self.table_host[slot, :] = 0
        self.dirty.pop(slot, None)

    def flush(self) -> None:
        for slot, (lo, hi) in self.dirty.items():
            self.table[slot, lo:hi].copy_(torch.from_numpy(self.table_host[slot, lo:hi]))
        self.dirty.clear()

    def view(self, entry: int) -> KVView:
        i = self.entries.index(entry)
        return KVView(self.k[i], self.v[i], self.table, self.req.n_kv_heads, self.req.head_dim,
                      self.req.window, self.ring_rows)


def bytes_per_token(requests: Sequence[Any], dtype: torch.dtype) -> int:
    """Bytes of cache that one position of one sequence takes, over all schedule entries' requests
    (keys and values; fixed-size states do not grow with the length and count nothing here)."""
    elem = torch.empty((), dtype=dtype).element_size()
    return sum(2 * r.n_kv_heads * r.head_dim * elem for r in requests if isinstance(r, KVRequest))


class CacheManager:
    """Owns all groups, the slots and each live sequence's length."""

    def __init__(self, requests: Sequence[Any], max_tokens: int, n_slots: int, max_seq_len: int,
                 dtype: torch.dtype, device):
        if max_tokens <= 0 or max_seq_len <= 0:
            raise CacheError("the cache needs a positive token capacity and sequence length")
        self.n_slots = int(n_slots)
        self.scratch_slot = self.n_slots
        self.max_tokens = pages_for(max_tokens) * PAGE
        self.max_seq_len = int(max_seq_len)
        self.slots = SlotAllocator(self.n_slots)
        self.length: Dict[int, int] = {}
        self.kv_groups: List[_KVGroup] = []
        self.states: Dict[int, torch.Tensor] = {}
        by_key: Dict[KVRequest, List[int]] = {}
        for entry, req in enumerate(requests):
            if req is None:
                continue
            if isinstance(req, KVRequest):
                by_key.setdefault(req, []).append(entry)
            elif isinstance(req, StateRequest):
                self.states[entry] = torch.zeros((self.n_slots + 1,) + tuple(req.shape),
                                                 dtype=req.dtype, device=device)
            else:
                raise CacheError(f"schedule entry {entry} asks for memory of unknown kind {type(req).__name__}")
        for req, entries in by_key.items():
            self.kv_groups.append(_KVGroup(req, entries, self.n_slots, self.max_tokens,
                                           self.max_seq_len, dtype, device))
        self._views: Dict[int, Any] = {}
        for g in self.kv_groups:
            for e in g.entries:
                self._views[e] = g.view(e)
        for e, t in self.states.items():
            self._views[e] = StateView(t)

    # -- slots ----------------------------------------------------------------
    def allocate_slot(self) -> int:
        slot = self.slots.allocate()
        self.length[slot] = 0
        for t in self.states.values():
            t[slot].zero_()
        return slot

    def reserve(self, slot: int, new_length: int) -> None:
        """Makes room for the sequence in ``slot`` to reach ``new_length`` positions."""
        if not self.slots.is_live(slot):
            raise CacheError(f"slot {slot} is not in use")
        if new_length > self.max_seq_len:
            raise CacheError(f"a sequence of {new_length} positions exceeds the limit of {self.max_seq_len}")
        for g in self.kv_groups:
            g.grow(slot, new_length)

    def commit(self, slot: int, new_length: int) -> None:
        self.length[slot] = new_length

    def release(self, slot: int) -> None:
        self.slots.release(slot)          # raises if the slot is not in use
        for g in self.kv_groups:
            g.drop(slot)
        del self.length[slot]

    def flush(self) -> None:
        """Copies page-table rows that changed to the device."""
        for g in self.kv_groups:
            g.flush()

    # -- views ------------------------------------------------------------------
    def view(self, entry: int):
        return self._views.get(entry)

    def views(self, n_entries: int) -> List[Any]:
        return [self._views.get(e) for e in range(n_entries)]

    # -- accounting -------------------------------------------------------------
    def tokens_held(self) -> int:
        """Positions held by live sequences, each rounded up to whole pages."""
        return sum(pages_for(n) * PAGE for n in self.length.values())

    def free_tokens(self) -> int:
        full = [g for g in self.kv_groups if not g.ring_pages]
        if full:
            return min(g.pool.n_free for g in full) * PAGE
        return self.max_tokens - self.tokens_held()

    def bytes(self) -> int:
        n = 0
        for g in self.kv_groups:
            n += 2 * g.k.numel() * g.k.element_size()
        for t in self.states.values():
            n += t.numel() * t.element_size()
        return n
