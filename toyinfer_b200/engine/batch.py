"""What a step's kernels know about its tokens and sequences.

All index arrays of a step live in one int32 buffer on the device, filled from one
pinned host buffer with one copy: the token ids, each token's position and sequence,
and each sequence's slot, start, count of new tokens, length after the step, and the
offsets of its tokens.  A decode step that is replayed from a CUDA graph keeps its
buffers and only refreshes their contents, as the reference does with its position
word (src/transformer.cpp:494-495).  Padding rows (a graph's batch size is a bucket)
point at the cache's scratch slot, hold one token at position 0, and are never read.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


def _round4(n: int) -> int:
    return (n + 3) & ~3


class BatchBuffers:
    """Pinned host and device storage for a step of up to ``n_seq`` sequences and
    ``n_tok`` tokens; tensors of a ``StepBatch`` are views into the device buffer."""

    FIELDS = ("token_ids", "tok_pos", "tok_seq", "seq_slot", "seq_start", "seq_new", "seq_len", "cu_new")

    def __init__(self, n_seq: int, n_tok: int, device):
        self.n_seq, self.n_tok = n_seq, n_tok
        sizes = {"token_ids": n_tok, "tok_pos": n_tok, "tok_seq": n_tok, "seq_slot": n_seq,
                 "seq_start": n_seq, "seq_new": n_seq, "seq_len": n_seq, "cu_new": n_seq + 1}
        self.offsets = {}
        off = 0
        for name in self.FIELDS:
            self.offsets[name] = (off, sizes[name])
            off += _round4(sizes[name])
        self.total = off
        device = torch.device(device)
        pin = device.type == "cuda"
        self.host = torch.zeros(self.total, dtype=torch.int32, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=device)
        self._copied = torch.cuda.Event() if pin else None
        self._pending = False

    def host_view(self, name: str) -> np.ndarray:
        off, n = self.offsets[name]
        return self.host_np[off:off + n]

    def dev_view(self, name: str) -> torch.Tensor:
        off, n = self.offsets[name]
        return self.dev[off:off + n]

    def begin_fill(self) -> None:
        """The host buffer may be rewritten only after its last upload has left it."""
        if self._pending:
            self._copied.synchronize()
            self._pending = False

    def upload(self) -> None:
        self.dev.copy_(self.host, non_blocking=True)
        if self._copied is not None:
            self._copied.record()
            self._pending = True


@dataclass
class StepBatch:
    mode: str                 # "start": every sequence begins at position 0; "extend": one new token each;
                              # "mixed": any start and any number of new tokens per sequence
    n_seq: int                # sequences, padding included
    n_tok: int                # tokens, padding included
    n_real_seq: int
    n_real_tok: int
    max_new: int              # most new tokens of one sequence
    max_pos_after: int        # longest length after the step
    plan_len: int             # length that launch shapes are planned for (the engine's limit)
    token_ids: torch.Tensor
    tok_pos: torch.Tensor
    tok_seq: torch.Tensor
    seq_slot: torch.Tensor
    seq_start: torch.Tensor
    seq_new: torch.Tensor
    seq_len: torch.Tensor
    cu_new: torch.Tensor
    # host copies for parts written without kernels of their own
    host_slots: List[int] = field(default_factory=list)
    host_starts: List[int] = field(default_factory=list)
    host_new: List[int] = field(default_factory=list)
    # set by a mixer's attention kernels for the product after them: whether their last kernel was
    # started only when the SMs had drained (kernels/attention.py); a matter of speed only
    drained_after_attention: bool = False
    trace: object = None      # the engine's tracing.Tracer (parts wrap their stages in its ranges); None: no tracing


def fill_batch(buf: BatchBuffers, mode: str, slots: Sequence[int], starts: Sequence[int],
               tokens: Sequence[Sequence[int]], scratch_slot: int, plan_len: int,
               pad_seqs: int = 0, total_tok: Optional[int] = None, new_bound: Optional[int] = None) -> StepBatch:
    """Writes a step into ``buf`` (host side), uploads it and returns the views.
    ``pad_seqs`` extra sequences of one token each are appended as padding.  With ``total_tok``
    the step has that many token rows whatever it holds (a captured step's launches are fixed):
    the spare rows after the last sequence's are nobody's.  They hold token 0 at position 0 of a
    stand-in sequence one past the step's own (index ``n_seq``: the scratch slot, no new tokens;
    the views of the per-sequence arrays are one entry longer for it, and ``buf`` must have the
    room), so that whatever is stored for them goes to the scratch slot; no sequence's count
    includes them and their results are never read.  ``new_bound`` stands for the longest run of
    new tokens and the longest length wherever launches are sized."""
    n_real = len(slots)
    n_seq = n_real + pad_seqs
    new = [len(t) for t in tokens]
    n_real_tok = sum(new)
    n_used = n_real_tok + pad_seqs
    n_tok = n_used if total_tok is None else int(total_tok)
    spare = n_tok > n_used
    if n_seq + spare > buf.n_seq or n_tok > buf.n_tok or n_used > n_tok:
        raise ValueError(f"step of {n_seq + spare} sequences / {max(n_tok, n_used)} tokens exceeds buffers for {buf.n_seq} / {buf.n_tok}")
    buf.begin_fill()
    ids, pos, seq = buf.host_view("token_ids"), buf.host_view("tok_pos"), buf.host_view("tok_seq")
    sl, st, nw, ln, cu = (buf.host_view("seq_slot"), buf.host_view("seq_start"), buf.host_view("seq_new"),
                          buf.host_view("seq_len"), buf.host_view("cu_new"))
    o = 0
    for i in range(n_real):
        n = new[i]
        ids[o:o + n] = tokens[i]
        pos[o:o + n] = np.arange(starts[i], starts[i] + n, dtype=np.int32)
        seq[o:o + n] = i
        sl[i], st[i], nw[i], ln[i], cu[i] = slots[i], starts[i], n, starts[i] + n, o
        o += n
    for i in range(n_real, n_seq):
        ids[o], pos[o], seq[o] = 0, 0, i
        sl[i], st[i], nw[i], ln[i], cu[i] = scratch_slot, 0, 1, 1, o
        o += 1
    cu[n_seq] = o
    # entries past the used part keep harmless values for kernels launched over the full buffers
    ids[o:] = 0
    pos[o:] = 0
    seq[o:] = n_seq if spare else max(n_seq - 1, 0)
    sl[n_seq:] = scratch_slot
    st[n_seq:] = 0
    nw[n_seq:] = 0
    ln[n_seq:] = 1
    cu[n_seq + 1:] = o
    buf.upload()
    return StepBatch(
        mode=mode, n_seq=n_seq, n_tok=n_tok, n_real_seq=n_real, n_real_tok=n_real_tok,
        max_new=new_bound if new_bound is not None else max(new + [1 if pad_seqs else 0]),
        max_pos_after=new_bound if new_bound is not None else max([s + n for s, n in zip(starts, new)] + [1]),
        plan_len=plan_len,
        token_ids=buf.dev_view("token_ids")[:n_tok], tok_pos=buf.dev_view("tok_pos")[:n_tok],
        tok_seq=buf.dev_view("tok_seq")[:n_tok], seq_slot=buf.dev_view("seq_slot")[:n_seq + spare],
        seq_start=buf.dev_view("seq_start")[:n_seq + spare], seq_new=buf.dev_view("seq_new")[:n_seq + spare],
        seq_len=buf.dev_view("seq_len")[:n_seq + spare], cu_new=buf.dev_view("cu_new")[:n_seq + 1 + spare],
        host_slots=list(slots) + [scratch_slot] * pad_seqs, host_starts=list(starts) + [0] * pad_seqs,
        host_new=new + [1] * pad_seqs,
    )
