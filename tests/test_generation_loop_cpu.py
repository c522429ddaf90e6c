"""The generation loop's decisions, with a scripted stepper in place of the engine:
batching of requests, stop tokens, sequences that end earlier, slot hand-back."""
from __future__ import annotations

import pytest
import torch

import cpu_kernels
from conftest import TINY, prompts_for
from plain import qwen3_plain as plain
from toyinfer_b200.engine.generate import GenerationLoop, plan_batches


class ScriptedStepper:
    """Draws, for a sequence whose prompt starts with p0, the tokens p0+1, p0+2, ...;
    records every step."""

    def __init__(self):
        self.free = list(range(100))
        self.live = {}
        self.steps = []
        self.ended = []

    def new_sequence(self):
        s = self.free.pop(0)
        self.live[s] = []
        return s

    def end_sequence(self, slot):
        assert slot in self.live, "slot ended twice"
        del self.live[slot]
        self.ended.append(slot)
        self.free.insert(0, slot)

    def step(self, entries, want):
        self.steps.append([(s, list(t)) for s, t in entries])
        rows = []
        for (s, toks), w in zip(entries, want if want is not None else [[len(t) - 1] for _, t in entries]):
            assert s in self.live
            self.live[s].extend(toks)
            if w:
                rows.append(s)
        return rows

    def sample(self, logits, keys, steps):
        return [self.live[s][-1] + 1 for s in logits]


def test_plan_batches():
    assert plan_batches([5, 9, 2, 7, 1], 8, 2, 10 ** 6, 128) == [[0, 1], [2, 3], [4]]
    # capacity: each request may hold roundup64(n + 8); 3 pages fit
    assert plan_batches([60, 60, 100, 10], 8, 8, 64 * 3, 256) == [[0], [1], [2, 3]]
    with pytest.raises(ValueError):
        plan_batches([300], 8, 8, 64 * 3, 512)
    with pytest.raises(ValueError):
        plan_batches([0], 8, 8, 64, 512)
    with pytest.raises(ValueError):
        plan_batches([600], 8, 8, 6400, 512)


def test_stop_tokens_lengths_and_early_ends():
    st = ScriptedStepper()
    loop = GenerationLoop(st, stop_ids=[13, 55], max_batch=3, max_seq_len=64, capacity_tokens=10 ** 6)
    prompts = [[10], [50, 51], [20, 0, 0], [30]]
    res = loop.run(prompts, max_new_tokens=6)
    assert res[0].tokens == [11, 12] and res[0].finish_reason == "stop"          # 13 is not emitted
    assert res[1].tokens == [52, 53, 54] and res[1].finish_reason == "stop"
    assert res[2].tokens == [1, 2, 3, 4, 5, 6] and res[2].finish_reason == "length"
    assert res[3].tokens == [31, 32, 33, 34, 35, 36]
    # first batch: three prompts in one step, then shrinking steps; the fourth request waits
    assert [len(s) for s in st.steps[:7]] == [3, 3, 3, 2, 1, 1, 1]
    assert st.steps[0] == [(0, [10]), (1, [50, 51]), (2, [20, 0, 0])]
    assert all(len(t) == 1 for s in st.steps[1:6] for _, t in s)
    assert not st.live and len(st.ended) == 4 and len(set(st.ended)) == 3       # a slot was used again
    assert loop.stats.batches == 2 and loop.stats.generated_tokens == 17


def test_ignore_eos_and_context_limit():
    st = ScriptedStepper()
    loop = GenerationLoop(st, stop_ids=[12], max_batch=4, max_seq_len=8, capacity_tokens=10 ** 6, ignore_eos=True)
    res = loop.run([[10], [1, 2, 3, 4, 5, 6], [9] * 8], max_new_tokens=5)
    assert res[0].tokens == [11, 12, 13, 14, 15]
    assert res[1].tokens == [7, 8] and res[1].finish_reason == "context"        # 6 + 2 = max_seq_len
    assert res[2].tokens == [] and res[2].finish_reason == "context"
    assert not st.live


def test_prompt_token_by_token():
    st = ScriptedStepper()
    loop = GenerationLoop(st, stop_ids=[], max_batch=4, max_seq_len=64, capacity_tokens=10 ** 6,
                          dedicated_prefill=False)
    res = loop.run([[10, 20, 30], [40]], max_new_tokens=3)
    assert res[0].tokens == [31, 32, 33] and res[1].tokens == [41, 42, 43]
    assert st.steps[0] == [(0, [10]), (1, [40])]
    assert st.steps[1] == [(0, [20]), (1, [41])] and st.steps[2] == [(0, [30]), (1, [42])]


def test_slots_come_back_after_an_error():
    class Failing(ScriptedStepper):
        def step(self, entries, want):
            if len(self.steps) == 2:
                raise RuntimeError("boom")
            return super().step(entries, want)

    st = Failing()
    loop = GenerationLoop(st, stop_ids=[], max_batch=4, max_seq_len=64, capacity_tokens=10 ** 6)
    with pytest.raises(RuntimeError):
        loop.run([[1], [2]], max_new_tokens=5)
    assert not st.live


class AheadStepper(ScriptedStepper):
    """The scripted stepper with the calls that let the loop start a step from tokens it
    has not read yet.  ``step_from`` gets the handle of the draw and works the tokens out
    itself, as a device would; it records which steps were started that way."""

    def __init__(self):
        super().__init__()
        self.from_handle = []

    def draw(self, logits, keys, steps):
        return list(self.sample(logits, keys, steps))

    def step_from(self, slots, handle):
        assert len(slots) == len(handle)
        self.from_handle.append(len(self.steps))
        return self.step([(s, [t]) for s, t in zip(slots, handle)], [[0] for _ in slots])

    def read(self, handle):
        return list(handle)

    def rows(self, logits, indices):
        return [logits[r] for r in indices]


@pytest.mark.parametrize("prompts, kw, max_new", [
    ([[10], [50, 51], [20, 0, 0], [30]], dict(stop_ids=[13, 55], max_batch=3, max_seq_len=64), 6),
    ([[10], [1, 2, 3, 4, 5, 6], [9] * 8], dict(stop_ids=[12], max_batch=4, max_seq_len=8, ignore_eos=True), 5),
    ([[10, 20, 30], [40]], dict(stop_ids=[], max_batch=4, max_seq_len=64, dedicated_prefill=False), 3),
    ([[10], [11], [12]], dict(stop_ids=[14], max_batch=3, max_seq_len=64), 9),      # three stops in three steps running
    ([[7]], dict(stop_ids=[], max_batch=1, max_seq_len=64), 1),
])
def test_starting_ahead_changes_no_result(prompts, kw, max_new):
    plain_st, ahead_st = ScriptedStepper(), AheadStepper()
    a = GenerationLoop(plain_st, capacity_tokens=10 ** 6, **kw).run(prompts, max_new_tokens=max_new)
    b = GenerationLoop(ahead_st, capacity_tokens=10 ** 6, **kw).run(prompts, max_new_tokens=max_new)
    assert [(r.tokens, r.finish_reason) for r in a] == [(r.tokens, r.finish_reason) for r in b]
    assert not ahead_st.live and sorted(ahead_st.ended) == sorted(plain_st.ended)


def test_starting_ahead_is_used_and_bounded():
    st = AheadStepper()
    loop = GenerationLoop(st, stop_ids=[13], max_batch=2, max_seq_len=64, capacity_tokens=10 ** 6)
    res = loop.run([[10], [20]], max_new_tokens=5)
    assert res[0].tokens == [11, 12] and res[1].tokens == [21, 22, 23, 24, 25]
    # steps: prompts; then steps started ahead, the third of them still with the sequence that
    # had drawn its stop token; none is started when a sequence is about to reach its length
    assert [len(s) for s in st.steps] == [2, 2, 2, 2, 1]
    assert st.from_handle == [1, 2, 3, 4]
    assert st.steps[3] == [(0, [13]), (1, [23])]            # one step too many for slot 0, dropped
    assert len(st.steps) == 5                               # no step after the last token


def test_generation_through_the_engine_matches_plain(monkeypatch, model_folders):
    """The real loop over the real engine (CPU stand-in kernels): greedy tokens equal the
    plain implementation's, for a batch of unequal prompts with a stop token in play."""
    cpu_kernels.install(monkeypatch)
    from toyinfer_b200 import LLM, SamplingParams
    name = "A"
    llm = LLM(model_folders[name], dtype="float32", device="cpu", max_seq_len=128, max_batch=2, max_tokens=512,
              enable_cuda_graph=False)
    prompts = prompts_for(name, [5, 9, 2], seed=40)
    w, cfg = plain.read_weights(model_folders[name]), plain.read_config(model_folders[name])
    free_run = [plain.generate(w, cfg, p, 8) for p in prompts]
    stop = free_run[1][3]                                   # make request 1 stop after three tokens
    got = llm.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=8, stop_token_ids=[stop])
    want = [plain.generate(w, cfg, p, 8, stop_ids=(stop, 7)) for p in prompts]
    assert [r.tokens for r in got] == want
    assert llm.engine.cache.slots.n_free == llm.engine.cache.n_slots


def test_prompts_fed_in_pieces():
    """prefill_chunk = 10: a step takes at most 10 prompt tokens in all, dealt out in request
    order; a sequence whose prompt is done decodes beside the pieces of the others; the tokens
    drawn are those of whole prompts."""
    prompts = [[100 + j for j in range(4)], [200 + j for j in range(23)], [300 + j for j in range(7)]]
    whole = ScriptedStepper()
    want = GenerationLoop(whole, [], 8, 1000, 10 ** 6).run(prompts, 3)
    st = ScriptedStepper()
    loop = GenerationLoop(st, [], 8, 1000, 10 ** 6, prefill_chunk=10)
    got = loop.run(prompts, 3)
    assert [r.tokens for r in got] == [r.tokens for r in want]
    # first step: 4 tokens of request 0 and 6 of request 1; request 2 waits
    assert [(s, len(t)) for s, t in st.steps[0]] == [(0, 4), (1, 6)]
    # second step: request 0 decodes, request 1 takes all 10 prompt tokens, request 2 still waits
    assert [(s, len(t)) for s, t in st.steps[1]] == [(0, 1), (1, 10)]
    # third: request 0 decodes, request 1 its last 7, request 2 gets the 3 that are left
    assert [(s, len(t)) for s, t in st.steps[2]] == [(0, 1), (1, 7), (2, 3)]
    assert loop.stats.prompt_tokens == 4 + 23 + 7
    assert not st.live and sorted(st.ended) == [0, 1, 2]
    with pytest.raises(ValueError):
        GenerationLoop(st, [], 8, 1000, 10 ** 6, prefill_chunk=0)


def test_prompts_in_pieces_on_the_engine(monkeypatch, model_folders):
    """The same through the library's engine on the CPU stand-ins: greedy tokens with prompts fed
    16 tokens a step equal those of whole prompts and the plain implementation's."""
    from toyinfer_b200 import LLM, SamplingParams
    cpu_kernels.install(monkeypatch)
    prompts = prompts_for("C", [70, 3, 45], seed=91)
    w, cfg = plain.read_weights(model_folders["C"]), plain.read_config(model_folders["C"])
    want = [plain.generate(w, cfg, p, 5) for p in prompts]
    for chunk in (None, 16):
        llm = LLM(model_folders["C"], dtype="float32", device="cpu", max_seq_len=320, max_batch=4, max_tokens=1024,
                  enable_cuda_graph=False, prefill_chunk=chunk)
        got = llm.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=5, ignore_eos=True)
        assert [r.tokens for r in got] == want, chunk
