"""The generation loop above the step function.

Requests are taken in order and grouped into batches (``plan_batches``); a batch's
prompts, of unequal lengths, run in one step, then every live sequence gets one token
per step.  A sequence ends at a stop token (which is not part of its output, as in the
reference, src/engine_runtime.cpp:448-450), after ``max_new_tokens``, or when it holds
``max_seq_len`` positions (src/engine_runtime.cpp:459-463); it leaves the batch at that
step and its slot goes back to the cache.  No request joins a running batch; the next
batch starts when the last sequence of this one has ended.

With ``prefill_chunk`` the prompts of a batch are fed in pieces: a step takes at most that
many prompt tokens in all, dealt out in request order, so the activations of a step stay
bounded however long the prompts are; sequences whose prompt is done decode in the same
steps meanwhile (the step function takes any mix of the two; the reference can do
neither).

The loop only decides; it runs steps and draws tokens through a ``stepper`` with
``new_sequence()``, ``end_sequence(slot)``, ``step(entries, want) -> logits`` and
``sample(logits, keys, steps) -> list of ints``, so its decisions can be tested
without a device.

A stepper may also offer ``draw(logits, keys, steps) -> handle``, ``step_from(slots,
handle) -> logits``, ``read(handle) -> list of ints`` and ``rows(logits, indices)``.
Then, while every live sequence is decoding and none is about to reach a length limit,
the loop starts the next step from the drawn tokens where they lie (on the device)
before it reads them: the device goes on while the host decides.  A sequence that turns
out to have drawn a stop token has then run one step too many; its row of that step is
dropped and its slot is released as usual, and no other sequence's result depends on it.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..cache.allocators import PAGE


@dataclass
class GenerationResult:
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""          # "stop", "length" (max_new_tokens) or "context" (max_seq_len)


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    decode_steps: int = 0
    batches: int = 0


def _held(n: int) -> int:
    return (n + PAGE - 1) // PAGE * PAGE


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, max_batch: int,
                 capacity_tokens: int, max_seq_len: int) -> List[List[int]]:
    """Request indices of each batch, in order.  A batch takes requests while it has fewer
    than ``max_batch`` and the positions they may come to hold (each rounded up to whole
    pages) fit the cache."""
    batches: List[List[int]] = []
    cur: List[int] = []
    held = 0
    for i, n in enumerate(prompt_lens):
        if n <= 0:
            raise ValueError(f"request {i}: the prompt is empty")
        if n > max_seq_len:
            raise ValueError(f"request {i}: a prompt of {n} tokens exceeds max_seq_len {max_seq_len}")
        need = _held(min(n + max_new_tokens, max_seq_len))
        if need > capacity_tokens:
            raise ValueError(f"request {i}: {need} positions do not fit the cache's {capacity_tokens}")
        if cur and (len(cur) >= max_batch or held + need > capacity_tokens):
            batches.append(cur)
            cur, held = [], 0
        cur.append(i)
        held += need
    if cur:
        batches.append(cur)
    return batches


class GenerationLoop:
    def __init__(self, stepper, stop_ids: Sequence[int], max_batch: int, max_seq_len: int,
                 capacity_tokens: int, ignore_eos: bool = False, dedicated_prefill: bool = True,
                 prefill_chunk: Optional[int] = None):
        self.stepper = stepper
        self.stop_ids = frozenset(int(s) for s in stop_ids)
        self.max_batch = max_batch
        self.max_seq_len = max_seq_len
        self.capacity_tokens = capacity_tokens
        self.ignore_eos = ignore_eos
        # False: prompts are fed one token per step through the decode path, the
        # reference's --use_dedicated_prefill=0 (src/engine_runtime.cpp:314-322)
        self.dedicated_prefill = dedicated_prefill
        if prefill_chunk is not None and prefill_chunk <= 0:
            raise ValueError(f"prefill_chunk must be positive, got {prefill_chunk}")
        self.prefill_chunk = prefill_chunk      # most prompt tokens one step takes (None: whole prompts)
        self.stats = GenerationStats()

    def _accept(self, res: GenerationResult, prompt_len: int, token: int, max_new: int) -> bool:
        """Adds a drawn token to a sequence's output; True when the sequence goes on."""
        if token in self.stop_ids and not self.ignore_eos:
            res.finish_reason = "stop"
            return False
        res.tokens.append(token)
        if len(res.tokens) >= max_new:
            res.finish_reason = "length"
            return False
        if prompt_len + len(res.tokens) >= self.max_seq_len:
            res.finish_reason = "context"
            return False
        return True

    def run(self, prompts: Sequence[Sequence[int]], max_new_tokens: int,
            keys: Optional[Sequence[int]] = None) -> List[GenerationResult]:
        results = [GenerationResult() for _ in prompts]
        if max_new_tokens <= 0:
            for r in results:
                r.finish_reason = "length"
            return results
        keys = list(keys) if keys is not None else list(range(len(prompts)))
        lens = [len(p) for p in prompts]
        for batch in plan_batches(lens, max_new_tokens, self.max_batch, self.capacity_tokens, self.max_seq_len):
            self._run_batch(batch, prompts, keys, max_new_tokens, results)
        return results

    def _at_limit_after_next(self, res: GenerationResult, prompt_len: int, max_new: int) -> bool:
        """True when the sequence ends by a length limit with the token it draws now."""
        n = len(res.tokens) + 1
        return n >= max_new or prompt_len + n >= self.max_seq_len

    def _run_batch(self, batch, prompts, keys, max_new, results) -> None:
        st = self.stepper
        can_look_ahead = all(hasattr(st, name) for name in ("draw", "step_from", "read", "rows"))
        self.stats.batches += 1
        live: List[Tuple[int, int]] = []          # (request index, slot)
        for i in batch:
            if len(prompts[i]) >= self.max_seq_len:   # no room for a single new token
                results[i].finish_reason = "context"
                continue
            live.append((i, st.new_sequence()))
        fed = {i: 0 for i, _ in live}             # prompt tokens already run
        last: Dict[int, int] = {}                 # the token each sequence drew last
        ahead = None                              # (logits, sequences) of a step already started
        try:
            while live:
                t0 = time.perf_counter()
                in_prompt = False
                if ahead is not None:
                    logits, started = ahead
                    ahead = None
                    if len(started) != len(live):         # some of them ended meanwhile
                        alive = {i for i, _ in live}
                        logits = st.rows(logits, [r for r, (i, _) in enumerate(started) if i in alive])
                    want = [[0] for _ in live]
                    n_prompt = 0
                    stepping = live
                else:
                    entries, want, stepping = [], [], []
                    n_prompt = 0
                    budget = self.prefill_chunk if self.prefill_chunk is not None else None
                    for i, slot in live:
                        p = prompts[i]
                        if fed[i] < len(p):
                            in_prompt = True
                            if not self.dedicated_prefill:
                                n = 1
                            elif budget is None:
                                n = len(p) - fed[i]
                            else:
                                n = min(len(p) - fed[i], budget)
                                budget -= n
                            if n == 0:
                                continue              # this step's prompt tokens are dealt out: the sequence waits
                            toks = list(p[fed[i]:fed[i] + n])
                            fed[i] += n
                            n_prompt += n
                            want.append([n - 1] if fed[i] == len(p) else [])
                        else:
                            toks = [last[i]]
                            want.append([0])
                        entries.append((slot, toks))
                        stepping.append((i, slot))
                    logits = st.step(entries, want)
                drawing = [(i, slot) for (i, slot), w in zip(stepping, want) if w]
                draw_keys = [keys[i] for i, _ in drawing]
                draw_steps = [len(results[i].tokens) for i, _ in drawing]
                if not drawing:
                    drawn = []
                elif can_look_ahead:
                    handle = st.draw(logits, draw_keys, draw_steps)
                    if len(drawing) == len(live) and not any(
                            self._at_limit_after_next(results[i], len(prompts[i]), max_new) for i, _ in live):
                        ahead = (st.step_from([slot for _, slot in live], handle), list(live))
                    drawn = st.read(handle)
                else:
                    drawn = st.sample(logits, draw_keys, draw_steps)
                goes_on = {}
                for (i, slot), tok in zip(drawing, drawn):
                    goes_on[i] = self._accept(results[i], len(prompts[i]), int(tok), max_new)
                    last[i] = int(tok)
                nxt = []
                for i, slot in live:
                    if goes_on.get(i, True):
                        nxt.append((i, slot))
                    else:
                        st.end_sequence(slot)
                live = nxt
                dt = time.perf_counter() - t0
                if in_prompt:
                    self.stats.prefill_seconds += dt
                    self.stats.prompt_tokens += n_prompt
                else:
                    self.stats.decode_seconds += dt
                    self.stats.decode_steps += 1
        except BaseException:
            for _, slot in live:
                try:
                    st.end_sequence(slot)
                except Exception:
                    pass
            raise
        self.stats.generated_tokens = sum(len(r.tokens) for r in results)
