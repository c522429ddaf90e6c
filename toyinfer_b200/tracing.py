"""Named ranges around the stages of a step: NVTX markers for a profiler's timeline and,
when asked for, device timers.

The reference wraps every stage in a scoped NVTX range (include/profiling.h:26-53; call
sites src/transformer.cpp:329, :350, :363, :428, :498, :511, :567, :595, :639) and, with
``--detail_time``, brackets the stages of every layer with CUDA events and reports their
sums (src/transformer.cpp:74-116, src/engine_runtime.cpp:207-261).  Here one object does
both: ``with tracer.range("layer.attn_block"):`` pushes an NVTX range and, if ``timing``
is on, records a CUDA event on the current stream at either end.  ``report()`` waits for
the device and returns, per name, how often the range ran and its total milliseconds.
A range that opens before this library has launched anything since the last range closed
starts at that range's end event instead of a new one: stages that follow one another then
add up to the step that holds them, with no host time between a stage's end and the next
stage's start counted against either.

Names are joined to the enclosing step's kind, which the engine sets: a range
``layer.attn_block`` inside a prompt step is reported as ``prefill.layer.attn_block``,
inside a step of single tokens as ``decode.layer.attn_block``.  A step replayed from a
CUDA graph runs no Python and therefore has no inner ranges: only the whole step is timed,
as in the reference ("N/A (CUDA graph enabled)", src/engine_runtime.cpp:255-260).
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Dict, List, Tuple

import torch


class Tracer:
    def __init__(self, nvtx: bool = True, timing: bool = False):
        cuda = torch.cuda.is_available()
        self.nvtx = bool(nvtx) and cuda
        self.timing = bool(timing) and cuda
        self.kind = ""                     # "prefill" or "decode": set by the engine around a step
        self.capturing = False             # inside a CUDA graph capture no timing events are recorded
        self._open: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        self._sums: Dict[str, List[float]] = {}     # name -> [count, total ms]
        self._last = None                  # the event recorded last, and the library's launch count then
        self._last_count = -1

    @property
    def active(self) -> bool:
        return self.nvtx or self.timing

    def _event(self, fresh: bool):
        from . import kernels as K
        n = K.launch_count
        if not fresh and self._last is not None and self._last_count == n:
            return self._last
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._last, self._last_count = ev, n
        return ev

    @contextmanager
    def range(self, name: str, fresh_start: bool = False):
        if not (self.nvtx or self.timing):
            yield
            return
        full = f"{self.kind}.{name}" if self.kind else name
        timed = self.timing and not self.capturing
        if self.nvtx:
            torch.cuda.nvtx.range_push(full)
        if timed:
            start = self._event(fresh_start)
        try:
            yield
        finally:
            if timed:
                self._open.append((full, start, self._event(True)))
            if self.nvtx:
                torch.cuda.nvtx.range_pop()

    @contextmanager
    def step(self, kind: str):
        """The whole of one step; ``kind`` prefixes the names of the ranges inside."""
        with self.range(f"{kind}_step", fresh_start=True):
            before, self.kind = self.kind, kind
            try:
                yield
            finally:
                self.kind = before

    def _collect(self) -> None:
        if not self._open:
            return
        torch.cuda.synchronize()
        for name, start, end in self._open:
            s = self._sums.setdefault(name, [0, 0.0])
            s[0] += 1
            s[1] += start.elapsed_time(end)
        self._open.clear()

    def report(self) -> Dict[str, Tuple[int, float]]:
        """name -> (times the range ran, total milliseconds on the device)."""
        self._collect()
        return {k: (int(v[0]), float(v[1])) for k, v in self._sums.items()}

    def reset(self) -> None:
        self._collect()
        self._sums.clear()


NULL = Tracer(nvtx=False, timing=False)


@contextmanager
def _nothing():
    yield


def ranged(batch, name: str):
    """``batch.trace.range(name)`` when the step is traced, else a context that does nothing."""
    trace = getattr(batch, "trace", None)
    if trace is None or not trace.active:
        return _nothing()
    return trace.range(name)
