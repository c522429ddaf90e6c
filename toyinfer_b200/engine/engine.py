"""The step function: runs exactly the tokens it is given, as one batch, from the cache.

``Engine.step(entries, want)`` takes for each sequence its slot and its next tokens: any
number of them (at least one), following whatever the sequence holds already.  Prompts of
unequal lengths in one step, one token each, a prompt fed in pieces, a prompt beside
sequences that decode: all are one call, and all give the same logits beyond rounding.
It returns float32 logits [wanted, vocab] for the wanted places, in the order of the
entries.  Finished sequences are simply absent from the next step; ``end_sequence`` gives
their slot and pages back.

The reference has two entry points for one sequence, ``prefill(ids, n)`` and
``forward(id, pos)`` (include/transformer.h:110-111), and cannot continue a sequence by
more than one token (its prefill writes cache rows [0, n) at positions 0..n-1,
src/transformer.cpp:393-398, src/prefill.cu:185-208).  Its decode body is captured once
into a CUDA graph and replayed (src/transformer.cpp:647-669).  Here a step in which every
sequence goes on by one token is captured per batch-size bucket; the graph reads slots,
lengths and token ids from device buffers refreshed before each replay.  Steps of whole
prompts with few tokens, which the host's launches would hold up, are captured as well when
their shape comes back (``Engine._prompt_graph``).
"""
from __future__ import annotations

import gc
import os
import weakref
from collections import OrderedDict
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..cache import CacheError, CacheManager, PAGE, pages_for
from ..config.registry import load_config
from ..parts.model import DecoderModel, ModelSpec
from ..tracing import Tracer
from ..weights import load_parameters, random_parameters
from .batch import BatchBuffers, StepBatch, fill_batch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not supported (bfloat16 or float32)")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype {name!r} is not supported (bfloat16 or float32)") from None


class StepError(ValueError):
    """A step that cannot be run as asked; nothing was changed."""


# A prompt step launched from Python costs the host about 20 us per kernel, some eight kernels a layer,
# whatever its size; the device needs about 2 flops per weight and token at some 1e15 flop/s, and it
# still waits for the host now and then while it has less than one and a half times the host's time to
# do (measured on the 4B shape: 1,024 tokens 9.4 ms as launches, 8.6 replayed; the host alone 5.9).  Steps
# of fewer token rows than that are worth capturing (4B shape: 1,152; 0.6B: 7,616; 32B: 192); longer ones
# keep the device busy anyway.
HOST_SECONDS_PER_LAUNCH = 20e-6
LAUNCHES_PER_LAYER = 8
DEVICE_FLOPS = 1.0e15
MAX_PROMPT_GRAPH_TOKENS = 8192


def prompt_graph_limit(n_layers: int, weights_per_token: int) -> int:
    """Token rows up to which a step of whole prompts is held up by the host's launches (a multiple of 64)."""
    host = n_layers * LAUNCHES_PER_LAYER * HOST_SECONDS_PER_LAUNCH
    rows = int(1.5 * host * DEVICE_FLOPS / (2.0 * max(weights_per_token, 1)))
    return max(64, min(MAX_PROMPT_GRAPH_TOKENS, rows // 64 * 64))


def _row_bucket(n: int) -> int:
    """Token rows of a captured prompt step: a multiple of 64 up to 1,024, then of 128, 256, 512 as the count
    doubles, so that rounding wastes a sixteenth of the rows at most and the shapes stay few."""
    unit = 64
    while n > 16 * unit:
        unit *= 2
    return -(-n // unit) * unit


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


def _bucket(n: int, cap: int) -> int:
    b = 1
    while b < n:
        b <<= 1
    return min(b, cap) if cap >= n else n


class Engine:
    def __init__(self, model: DecoderModel, max_tokens: int, max_batch: int = 64,
                 max_seq_len: Optional[int] = None, n_slots: Optional[int] = None,
                 use_cuda_graph: bool = True, tracer: Optional[Tracer] = None):
        self.model = model
        # NVTX ranges around steps and stages by default; device timers when the caller asks (tracing.py)
        self.tracer = tracer if tracer is not None else Tracer(nvtx=torch.device(model.device).type == "cuda")
        self.spec: ModelSpec = model.spec
        self.device = model.device
        self.dtype = model.dtype
        self.max_batch = int(max_batch)
        limit = self.spec.max_positions
        self.max_seq_len = int(min(max_seq_len or limit, limit))
        self.max_tokens = int(max_tokens)
        if n_slots is None:
            n_slots = max(self.max_batch, min(pages_for(self.max_tokens), 1024))
        self.cache = CacheManager(model.memory_requests(), self.max_tokens, n_slots, self.max_seq_len,
                                  self.dtype, self.device)
        self.memories = self.cache.views(len(model.schedule))
        self.use_cuda_graph = bool(use_cuda_graph) and self.device.type == "cuda"
        self._eager_bufs: Dict[Tuple[int, int], BatchBuffers] = {}
        self._graphs: Dict[Tuple[int, Any], "_CapturedStep"] = {}     # (batch bucket, launch plan of its length class) -> captured step
        self._plans: Dict[Tuple[int, int, int], Any] = {}            # (batch bucket, length class, real sequences) -> the model's launch plan
        # All captured steps draw their intermediate buffers from one pool: steps run one at a time,
        # so what one graph freed during its capture another may use.  Each graph still keeps its
        # own [bucket, vocab] float32 logits (alive at the end of its capture).
        self._graph_pool = None
        self.graph_replays = 0
        # Steps of whole prompts with few tokens are bound by the host's launches, not by the device:
        # a shape that comes back (token rows and the longest prompt rounded up, see _prompt_graph) is captured when
        # it is seen the second time, if the model's parts allow it.  The least recently used go first.
        self.prompt_graph_tokens = 0
        if self.use_cuda_graph and model.captures_start():
            # the weights every token meets: the scheduled blocks' matrices (the embedding is looked up, and the
            # head reads one row per sequence)
            per_token = sum(_numel(sp.shape) for e in model.schedule for sp in model.blocks[e.layer].param_specs().values()
                            if sp.role == "matrix")
            self.prompt_graph_tokens = prompt_graph_limit(len(model.schedule), per_token)
        self.max_prompt_graphs = 16
        self._prompt_graphs: "OrderedDict[Tuple[int, int, int], _CapturedStep]" = OrderedDict()
        self._prompt_shapes_seen: Dict[Tuple[int, int, int], int] = {}

    # -- construction -----------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", device="cuda", **kw) -> "Engine":
        """Model folder (config.json + safetensors) -> engine; the model class is the one
        that config.json names."""
        from .. import models  # noqa: F401  (registers the architectures)
        arch, cfg = load_config(model_dir)
        dt = parse_dtype(dtype)
        model = DecoderModel(arch.describe(cfg), dt, device)
        tensors = load_parameters(model.param_specs(), model_dir, dt, model.device,
                                  ignorable=model.ignorable_names())
        model.bind(tensors)
        eng = cls(model, **kw)
        eng.config = cfg
        return eng

    @classmethod
    def from_config(cls, config: dict, seed: int = 0, dtype="bfloat16", device="cuda", **kw) -> "Engine":
        """Random weights drawn on the device, without a file (for measurements)."""
        from .. import models  # noqa: F401
        from ..config.registry import architecture_of
        arch = architecture_of(config)
        cfg = arch.config_cls.from_dict(config)
        dt = parse_dtype(dtype)
        model = DecoderModel(arch.describe(cfg), dt, device)
        model.bind(random_parameters(model.param_specs(), seed, dt, model.device))
        eng = cls(model, **kw)
        eng.config = cfg
        return eng

    # -- sequences ----------------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.allocate_slot()

    def end_sequence(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length[slot]

    # -- one step -------------------------------------------------------------------
    def step(self, entries: Sequence[Tuple[int, Optional[Sequence[int]]]],
             want: Optional[Sequence[Sequence[int]]] = None,
             token_source: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """entries: (slot, next tokens) per sequence.  want: per entry the places among its
        tokens whose logits are asked for (None: the last place of each).  Returns float32
        [wanted, vocab] on the device, or None when nothing is wanted.  The tensor may be
        a buffer that the next step overwrites: use or copy it before stepping again.

        With ``token_source`` (int32 on the device, one id per entry, in the entries' order)
        every entry's tokens are None and each sequence goes on by the id found there when
        the step runs: tokens that an earlier kernel drew need not pass through the host.
        Their range is the caller's duty."""
        n = len(entries)
        if n == 0:
            return None
        if n > self.max_batch:
            raise StepError(f"a step of {n} sequences exceeds max_batch {self.max_batch}")
        slots = [int(s) for s, _ in entries]
        if token_source is not None:
            if any(t is not None for _, t in entries):
                raise StepError("with token_source every entry's tokens are None")
            if token_source.dtype != torch.int32 or token_source.dim() != 1 or token_source.shape[0] != n \
                    or token_source.device.type != self.device.type:
                raise StepError(f"token_source must be int32 [{n}] on {self.device}")
            tokens = [[0] for _ in entries]
        else:
            if any(t is None for _, t in entries):
                raise StepError("an entry without tokens needs token_source")
            tokens = [list(t) for _, t in entries]
        if len(set(slots)) != n:
            raise StepError("a slot appears twice in one step")
        for s in slots:
            if s not in self.cache.length:
                raise StepError(f"slot {s} is not in use")
        for s, t in zip(slots, tokens):
            if not t:
                raise StepError(f"slot {s}: a step needs at least one token per sequence")
            for tok in t:
                if not (0 <= tok < self.spec.vocab_size):
                    raise StepError(f"slot {s}: token id {tok} is outside the vocabulary of {self.spec.vocab_size}")
        starts = [self.cache.length[s] for s in slots]
        # two special cases have faster kernels; everything else is the general form
        if all(st == 0 for st in starts) and token_source is None:
            mode = "start"
        elif all(len(t) == 1 for t in tokens):
            mode = "extend"
        else:
            mode = "mixed"
        if want is None:
            want = [[len(t) - 1] for t in tokens]
        if len(want) != n:
            raise StepError("want needs one list per entry")
        for w, t in zip(want, tokens):
            for p in w:
                if not (0 <= p < len(t)):
                    raise StepError(f"wanted place {p} is outside the entry's {len(t)} tokens")
        for s, st, t in zip(slots, starts, tokens):
            if st + len(t) > self.max_seq_len:
                raise StepError(f"slot {s}: {st + len(t)} positions exceed the limit of {self.max_seq_len}")
        for s, st, t in zip(slots, starts, tokens):
            self.cache.reserve(s, st + len(t))      # CacheError when the cache is full
        self.cache.flush()

        logits = self._run(mode, slots, starts, tokens, want, token_source)
        for s, st, t in zip(slots, starts, tokens):
            self.cache.commit(s, st + len(t))
        return logits

    def _run(self, mode, slots, starts, tokens, want, token_source):
        n = len(slots)
        if mode == "extend" and self.use_cuda_graph:
            logits_all = self._decode_graph(slots, starts, tokens, token_source)
            rows = [i for i, w in enumerate(want) if w]
            if not rows:
                return None
            if len(rows) == n:
                return logits_all[:n]
            return logits_all[torch.tensor(rows, device=self.device)]
        # (a prompt step whose stages are to be timed runs as plain launches: a replay has no stages)
        if mode == "start" and self.prompt_graph_tokens and not self.tracer.timing \
                and all(list(w) == [len(t) - 1] for w, t in zip(want, tokens)):
            logits_all = self._prompt_graph(slots, starts, tokens)
            if logits_all is not None:
                return logits_all
        batch = self._eager_batch(mode, slots, starts, tokens)
        if token_source is not None:
            batch.token_ids[:n].copy_(token_source)
        rows, o = [], 0
        for w, t in zip(want, tokens):
            rows.extend(o + p for p in w)
            o += len(t)
        rows_dev = torch.tensor(rows, dtype=torch.int32, device=self.device) if rows else None
        # the step's range holds the launches of the model only, not the host's preparation of the batch
        with self.tracer.step("decode" if mode == "extend" else "prefill"):
            h, delta = self.model.forward_hidden(batch, self.memories)
            if rows_dev is None:
                return None
            with self.tracer.range("head"):
                return self.model.logits(h, delta, rows_dev)

    # -- accounting for measurements ----------------------------------------------------
    def launches_per_step(self, n_seq: int) -> int:
        """Kernels that one captured decode step of ``n_seq`` sequences launches."""
        g = self._graph_of_bucket(_bucket(n_seq, self.max_batch))
        return g.launches if g is not None else 0

    def decode_metadata_bytes(self, n_seq: int) -> int:
        """Bytes copied host to device before each decode step of ``n_seq`` sequences."""
        g = self._graph_of_bucket(_bucket(n_seq, self.max_batch))
        return g.buf.total * 4 if g is not None else 0

    def _graph_of_bucket(self, bucket: int):
        for (b, _), g in self._graphs.items():
            if b == bucket:
                return g
        return None

    # -- helpers ----------------------------------------------------------------------
    def _eager_batch(self, mode, slots, starts, tokens) -> StepBatch:
        n_seq, n_tok = len(slots), sum(len(t) for t in tokens)
        key = (_bucket(n_seq, 1 << 30), _bucket(n_tok, 1 << 30))
        buf = self._eager_bufs.get(key)
        if buf is None:
            buf = self._eager_bufs[key] = BatchBuffers(key[0], key[1], self.device)
        batch = fill_batch(buf, mode, slots, starts, tokens, self.cache.scratch_slot, self.max_seq_len)
        batch.trace = self.tracer
        return batch

    def _decode_graph(self, slots, starts, tokens, token_source=None) -> torch.Tensor:
        n = len(slots)
        b = _bucket(n, self.max_batch)
        # Launch shapes that depend on how long sequences are (how the keys of a sequence are split
        # over blocks) are planned for a class of lengths, not for the engine's limit: powers of two
        # from 1,024 positions up.  A batch that grows past its class moves to the next graph.
        longest = max(starts) + 1
        cls = 1024
        while cls < longest:
            cls <<= 1
        cls = min(cls, self.max_seq_len)
        # ... unless nothing in the model's launches tells the two classes apart (with eight sequences of
        # 32 heads over 8 the keys are split four ways from 512 positions on): one graph serves both
        plan = self._plans.get((b, cls, n))
        if plan is None:
            plan = self._plans[(b, cls, n)] = self.model.launch_plan(b, cls, n)
        g = self._graphs.get((b, plan))
        if g is None:
            g = self._graphs[(b, plan)] = _CapturedStep(self, "extend", b, b, cls)
        return g.run(slots, starts, tokens, token_source)


    def _prompt_graph(self, slots, starts, tokens) -> Optional[torch.Tensor]:
        """Runs a step of whole prompts from a captured graph, or returns None (run it as it is).
        Shapes are rounded up so that fewer graphs serve more steps: token rows as _row_bucket says
        (the spare rows are nobody's, see fill_batch), the longest prompt to a power of two."""
        n_seq = len(slots)
        n_tok = _row_bucket(sum(len(t) for t in tokens))
        if n_tok > self.prompt_graph_tokens:
            return None
        bound = min(_bucket(max(len(t) for t in tokens), 1 << 30), n_tok, self.max_seq_len)
        key = (n_seq, n_tok, bound)
        g = self._prompt_graphs.get(key)
        if g is None:
            seen = self._prompt_shapes_seen[key] = self._prompt_shapes_seen.get(key, 0) + 1
            if seen < 2:
                return None
            while len(self._prompt_graphs) >= self.max_prompt_graphs:
                self._prompt_graphs.popitem(last=False)
            g = self._prompt_graphs[key] = _CapturedStep(self, "start", n_seq, n_tok, self.max_seq_len, bound)
        else:
            self._prompt_graphs.move_to_end(key)
        return g.run(slots, starts, tokens)


class _CapturedStep:
    """A step of fixed launches captured into a CUDA graph: ``n_seq`` sequences that go on by one
    token each ("extend"), or that start with up to ``n_tok`` tokens altogether and at most
    ``new_bound`` each ("start").  It refers to its engine weakly: engine and graphs then form
    no cycle, and both are released (with their device memory) when the last reference to the
    engine goes, not at some later collection."""

    def __init__(self, engine: Engine, mode: str, n_seq: int, n_tok: int, plan_len: int,
                 new_bound: Optional[int] = None):
        self._engine = weakref.ref(engine)
        self.mode = mode
        self.bucket = n_seq
        self.n_tok = n_tok
        self.plan_len = plan_len
        self.new_bound = new_bound
        self.buf = BatchBuffers(n_seq + (mode == "start"), n_tok, engine.device)     # a prompt step's spare rows need a stand-in
        # the rows whose logits are wanted: every row of single tokens, each sequence's last otherwise
        self.rows = torch.arange(n_seq, dtype=torch.int32, device=engine.device) if mode == "extend" else None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.launches = 0

    @property
    def engine(self) -> Engine:
        e = self._engine()
        if e is None:
            raise RuntimeError("the engine of this captured step is gone")
        return e

    def _body(self, batch: StepBatch) -> torch.Tensor:
        e = self.engine
        h, delta = e.model.forward_hidden(batch, e.memories)
        # each sequence's last row, found on the device: the graph is replayed with other lengths
        rows = self.rows if self.rows is not None else batch.cu_new[1:batch.n_seq + 1] - 1
        with e.tracer.range("head"):
            return e.model.logits(h, delta, rows)

    def run(self, slots, starts, tokens, token_source=None) -> torch.Tensor:
        e = self.engine
        name = "decode" if self.mode == "extend" else "prefill"
        if self.mode == "extend":
            batch = fill_batch(self.buf, "extend", slots, starts, tokens, e.cache.scratch_slot,
                               self.plan_len, pad_seqs=self.bucket - len(slots))
        else:
            batch = fill_batch(self.buf, "start", slots, starts, tokens, e.cache.scratch_slot,
                               self.plan_len, total_tok=self.n_tok, new_bound=self.new_bound)
        batch.trace = e.tracer
        if token_source is not None:
            batch.token_ids[:len(slots)].copy_(token_source)      # after the upload, before the replay
        if self.graph is None:
            # one eager run first: it is this step's result, and it lets every kernel do its
            # one-time set-up outside the capture
            from .. import kernels as K
            before = K.launch_count
            # the stages inside this run and inside the capture are not timed: replays have none
            was_capturing = e.tracer.capturing
            with e.tracer.step(name):
                e.tracer.capturing = True
                try:
                    out = self._body(batch)
                finally:
                    e.tracer.capturing = was_capturing
            self.launches = K.launch_count - before
            torch.cuda.current_stream().synchronize()
            g = torch.cuda.CUDAGraph()
            # The capture only records; nothing runs until the first replay.  No collection of
            # Python garbage may fall into it: objects that own device memory, events or other
            # graphs would be destroyed in the middle of the capture, which ends it with an error.
            gc.collect()
            was_enabled = gc.isenabled()
            gc.disable()
            e.tracer.capturing = True
            try:
                if e._graph_pool is None:
                    e._graph_pool = torch.cuda.graph_pool_handle()
                with torch.cuda.graph(g, pool=e._graph_pool):
                    self.logits = self._body(batch)
            finally:
                e.tracer.capturing = was_capturing
                if was_enabled:
                    gc.enable()
            self.graph = g
            return out
        with e.tracer.step(name):
            self.graph.replay()
        e.graph_replays += 1
        return self.logits
