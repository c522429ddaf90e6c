"""Generation through the entry point and the command line on the GPU: greedy tokens
equal the plain implementation's; sampled tokens follow the fixed seed whatever the
batch; the workloads named for the two tiny configurations (three greedy prompts, four sampled ones)."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT, TINY, prompts_for
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def _plain(folder):
    return plain.read_weights(folder), plain.read_config(folder)


@pytest.mark.parametrize("graph", [True, False])
def test_greedy_matches_plain_tiny_a(model_folders, graph):
    """Tiny A workload: prompts of 5, 9 and 2 tokens, 8 greedy tokens each, float32."""
    from toyinfer_b200 import LLM, SamplingParams
    f = model_folders["A"]
    llm = LLM(f, dtype="float32", max_seq_len=128, max_batch=4, max_tokens=1024, enable_cuda_graph=graph)
    prompts = prompts_for("A", [5, 9, 2], seed=50)
    got = llm.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=8, ignore_eos=True)
    w, cfg = _plain(f)
    assert [r.tokens for r in got] == [plain.generate(w, cfg, p, 8) for p in prompts]
    assert llm.engine.cache.slots.n_free == llm.engine.cache.n_slots


def test_temperature_sampling_tiny_b(model_folders):
    """Tiny B workload: prompts of 17, 1, 40 and 8 tokens, 12 tokens at temperature 0.8
    with a fixed seed.  The same request draws the same tokens alone and in the batch, and
    they are the plain sampler's (float32 engine, so logits agree to rounding)."""
    from toyinfer_b200 import LLM, SamplingParams
    f = model_folders["B"]
    params = SamplingParams(temperature=0.8, top_k=0, top_p=1.0, seed=321)
    prompts = prompts_for("B", [17, 1, 40, 8], seed=51)
    llm = LLM(f, dtype="float32", max_seq_len=256, max_batch=4, max_tokens=2048)
    together = [r.tokens for r in llm.generate(prompts, params, max_new_tokens=12, ignore_eos=True)]
    w, cfg = _plain(f)
    for i, p in enumerate(prompts):
        want = plain.generate(w, cfg, p, 12, temperature=0.8, top_k=0, top_p=1.0, seed=321, key=i)
        assert together[i] == want, (i, together[i], want)
    llm2 = LLM(f, dtype="float32", max_seq_len=256, max_batch=1, max_tokens=2048)
    one_by_one = [r.tokens for r in llm2.generate(prompts, params, max_new_tokens=12, ignore_eos=True)]
    assert one_by_one == together


def test_nucleus_sampling_without_top_k(model_folders):
    """temperature 0.7, top_k off, top_p 0.9 (a common setting that needs the sampler's tiered kernel)
    through the entry point: the plain sampler's tokens, alone and in a batch."""
    from toyinfer_b200 import LLM, SamplingParams
    f = model_folders["A"]
    params = SamplingParams(temperature=0.7, top_k=0, top_p=0.9, seed=77)
    prompts = prompts_for("A", [6, 21, 3], seed=57)
    llm = LLM(f, dtype="float32", max_seq_len=128, max_batch=4, max_tokens=1024)
    got = [r.tokens for r in llm.generate(prompts, params, max_new_tokens=10, ignore_eos=True)]
    w, cfg = _plain(f)
    for i, p in enumerate(prompts):
        assert got[i] == plain.generate(w, cfg, p, 10, temperature=0.7, top_k=0, top_p=0.9, seed=77, key=i), i
    llm2 = LLM(f, dtype="float32", max_seq_len=128, max_batch=1, max_tokens=1024)
    assert [r.tokens for r in llm2.generate(prompts, params, max_new_tokens=10, ignore_eos=True)] == got


def test_bfloat16_greedy_follows_its_own_logits(model_folders):
    """In bfloat16 near-ties may resolve differently from the plain result, so each drawn
    token is checked against the plain logits of the engine's own sequence: it must be the
    maximum or within rounding of it."""
    from toyinfer_b200 import LLM, SamplingParams
    f = model_folders["C"]
    llm = LLM(f, dtype="bfloat16", max_seq_len=320, max_batch=4, max_tokens=2048)
    prompts = prompts_for("C", [70, 3, 130], seed=52)
    got = llm.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=20, ignore_eos=True)
    w, cfg = _plain(f)
    for p, r in zip(prompts, got):
        assert len(r.tokens) == 20
        logits = plain.forward(w, cfg, p + r.tokens, torch.bfloat16)
        for t, tok in enumerate(r.tokens):
            row = logits[len(p) + t - 1]
            assert row[tok] >= row.max() - 0.03 * row.abs().max()


def test_stop_token_and_queue_of_batches(model_folders):
    from toyinfer_b200 import LLM, SamplingParams
    f = model_folders["A"]
    w, cfg = _plain(f)
    prompts = prompts_for("A", [5, 9, 2, 30, 4, 11, 7], seed=53)
    free = [plain.generate(w, cfg, p, 10) for p in prompts]
    stop = free[3][2]
    llm = LLM(f, dtype="float32", max_seq_len=128, max_batch=3, max_tokens=64 * 4)
    got = llm.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=10, stop_token_ids=[stop])
    want = [plain.generate(w, cfg, p, 10, stop_ids=(stop, 7)) for p in prompts]
    assert [r.tokens for r in got] == want
    assert llm.last_stats.batches >= 3
    assert llm.engine.cache.slots.n_free == llm.engine.cache.n_slots


def test_starting_the_next_step_ahead_changes_no_token(model_folders):
    """The loop starts each decode step from the drawn tokens on the device before it has read
    them.  The same requests through a stepper without that ability (every token read first)
    give the same tokens, with sequences that stop in the middle of a batch.  (In 32-bit: the
    two orders run some steps with different batch sizes, hence through different kernels, and
    in bfloat16 a near-tie may then fall the other way.)"""
    from toyinfer_b200 import LLM, SamplingParams
    from toyinfer_b200.engine.generate import GenerationLoop
    from toyinfer_b200.sampling import Sampler

    class OneByOne:
        def __init__(self, inner):
            self.new_sequence, self.end_sequence = inner.new_sequence, inner.end_sequence
            self.step, self.sample = inner.step, inner.sample

    for name, dtype, params in (("A", "float32", SamplingParams(temperature=0.0)),
                                ("C", "float32", SamplingParams(temperature=0.9, top_k=12, top_p=0.9, seed=5))):
        llm = LLM(model_folders[name], dtype=dtype, max_seq_len=128, max_batch=4, max_tokens=64 * 16)
        prompts = prompts_for(name, [5, 9, 2, 30, 4, 11], seed=56)
        free = llm.generate(prompts, params, max_new_tokens=12, ignore_eos=True)
        stops = [free[1].tokens[3], free[4].tokens[7]]
        ahead = llm.generate(prompts, params, max_new_tokens=12, stop_token_ids=stops)
        assert any(r.finish_reason == "stop" for r in ahead) and any(r.finish_reason == "length" for r in ahead)
        e = llm.engine
        llm._stepper.sampler = Sampler(params, e.device)
        loop = GenerationLoop(OneByOne(llm._stepper), set(llm.stop_token_ids) | set(stops), e.max_batch, e.max_seq_len,
                              e.cache.max_tokens)
        plain_order = loop.run(prompts, 12)
        assert [(r.tokens, r.finish_reason) for r in ahead] == [(r.tokens, r.finish_reason) for r in plain_order]
        assert loop.stats.decode_steps <= llm.last_stats.decode_steps
        assert e.cache.slots.n_free == e.cache.n_slots


def test_command_line(model_folders):
    f = model_folders["A"]
    prompts = prompts_for("A", [6, 3], seed=54)
    arg = ";".join(",".join(map(str, p)) for p in prompts)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "toyinfer"), "--model_dir", f, "--max_seq_len", "128",
           "--dtype", "float32", "--temperature", "0", "--prompt_ids", arg, "--max_new_tokens", "6",
           "--ignore_eos", "1", "--detail_time", "1", "--enable_cuda_graph", "1"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    w, cfg = _plain(f)
    assert [l["tokens"] for l in lines] == [plain.generate(w, cfg, p, 6) for p in prompts]
    assert "[perf]" in r.stderr and "[detail]" in r.stderr
    # token-by-token prompts give the same tokens
    r2 = subprocess.run(cmd + ["--use_dedicated_prefill", "0"], capture_output=True, text=True, timeout=300)
    assert r2.returncode == 0, r2.stderr
    assert [json.loads(l)["tokens"] for l in r2.stdout.splitlines() if l.startswith("{")] == [l["tokens"] for l in lines]


def test_command_line_with_random_weights(tmp_path):
    """--random takes a config.json alone; the same seed draws the same weights, so two runs
    print the same tokens."""
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY["B"]))
    cmd = [sys.executable, os.path.join(ROOT, "bin", "toyinfer"), "--random", str(cfg_path), "--seed", "5", "--max_seq_len", "128",
           "--dtype", "float32", "--temperature", "0", "--prompt_ids", "3,1,4,1,5;9,2,6", "--max_new_tokens", "5", "--ignore_eos", "1"]
    runs = []
    for _ in range(2):
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr
        runs.append([json.loads(l)["tokens"] for l in r.stdout.splitlines() if l.startswith("{")])
    assert runs[0] == runs[1] and [len(t) for t in runs[0]] == [5, 5]


@pytest.mark.parametrize("graph", [False, True])
def test_detail_time_stages_add_up_to_the_steps(model_folders, graph):
    """With detail_time every step is bracketed by CUDA events and, where a step runs as plain
    launches, so are its stages (embedding, each layer's attention block and feed-forward block,
    head).  The stages are back to back on the stream, so their device times add up to the step's
    within 10 %.  Steps replayed from a CUDA graph are timed whole; their stages read N/A."""
    from toyinfer_b200 import LLM, SamplingParams
    from toyinfer_b200.engine.cli import detail_lines
    name = "D"
    layers = TINY[name]["num_hidden_layers"]
    llm = LLM(model_folders[name], dtype="bfloat16", max_seq_len=512, max_batch=4, max_tokens=64 * 32,
              enable_cuda_graph=graph, detail_time=True)
    prompts = prompts_for(name, [300, 120, 41], seed=61)
    llm.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=3, ignore_eos=True)      # warm-up: first launches
    llm.engine.tracer.reset()
    llm.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=9, ignore_eos=True)
    rep = llm.timing_report()
    n_pre, t_pre = rep["prefill_step"]
    assert n_pre == 1 and t_pre > 0
    assert rep["prefill.layer.attn_block"][0] == layers and rep["prefill.layer.mlp_block"][0] == layers
    stages = sum(rep[k][1] for k in ("prefill.embed", "prefill.layer.attn_block", "prefill.layer.mlp_block", "prefill.head"))
    assert abs(stages - t_pre) <= 0.10 * t_pre, (stages, t_pre)
    inner = sum(rep[k][1] for k in ("prefill.mixer.qkv", "prefill.mixer.attention", "prefill.mixer.out"))
    assert inner <= rep["prefill.layer.attn_block"][1] * 1.001
    n_dec, t_dec = rep["decode_step"]
    assert n_dec == llm.last_stats.decode_steps and t_dec > 0
    assert rep["sample"][0] >= n_dec
    lines = "\n".join(detail_lines(llm.last_stats, rep, graph))
    if graph:
        assert "decode.layer.attn_block" not in rep
        assert "decode.layer.attn_block=N/A (CUDA graph enabled)" in lines
    else:
        assert rep["decode.layer.attn_block"][0] == layers * n_dec
        stages = sum(rep[k][1] for k in ("decode.embed", "decode.layer.attn_block", "decode.layer.mlp_block", "decode.head"))
        assert abs(stages - t_dec) <= 0.10 * t_dec, (stages, t_dec)
        assert "N/A" not in lines
    assert "prefill_total=" in lines and "decode_forward_total=" in lines
