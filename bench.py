#!/usr/bin/env python3
"""Measures generation on one B200 and prints one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Qwen3-4B (BASELINE.json configs[2]) with random
weights, a batch of 8 and a context of 8,192 positions.  A step is one decode step of
the whole batch.  ``value`` is decoded tokens per second over K steps timed on the
device with CUDA events (token ids chosen beforehand, no host round trip inside);
``e2e`` is the same through the Python entry point ``LLM.generate`` (host token ids in,
sampled token ids read back every step).  The line also carries a 2,048-token prefill,
the decode step's share of the memory roofline, and under ``points`` decode rates at
batch 1 and 64, the mean rates while 1, 8 and 64 sequences grow from 2,048 to the context
length (sampled at 13 lengths), 8 sequences at 32,768 positions, and 8 sequences at 8,192
with the layer sizes of Qwen3-8B.  ``fp32_check`` is the float32 engine with two layers of
the same sizes against the plain implementation of tests/plain (float64): the largest
error of the logits of a 512-token prompt's last place and of 8 decoded places.
Every decode step reads all weights (8 GB) and the live sequences' cache, far more than
the 126 MB L2, so nothing is flushed between steps.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_4B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 36, "hidden_size": 2560,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728,
    "vocab_size": 151936, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "max_position_embeddings": 40960,
    "tie_word_embeddings": True,
}
QWEN3_8B = dict(QWEN3_4B, hidden_size=4096, intermediate_size=12288, tie_word_embeddings=False)
QWEN3_32B = dict(QWEN3_4B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600,
                 tie_word_embeddings=False)
FULL_LAYERS = 36
CONTEXT = 8192
LONG_CONTEXT = 32768
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    try:
        with open(path) as f:
            m = json.load(f)
        for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if k in m:
                out[k] = float(m[k])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        def pump():
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                mhz.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def flops_prefill(cfg, T):
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    linear = 2.0 * T * L * (H * (q + 2 * kv) + q * H + 3 * H * I)
    attn = L * 4.0 * q * T * (T + 1) / 2          # QK^T and PV over the causal half
    return linear + attn + 2.0 * H * V            # one row of the head


def bytes_decode(cfg, batch, context, elem=2):
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    weights = L * (H * (q + 2 * kv) + q * H + 3 * H * I + 2 * H + 2 * cfg["head_dim"]) + H + V * H
    if not cfg.get("tie_word_embeddings", False):
        weights += 0  # the embedding table itself is only gathered from (batch rows)
    cache = 2.0 * L * kv * context * batch
    return (weights + cache) * elem


def random_tokens(n, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def time_decode(engine, batch, context, steps, warmup, seed=0):
    """Prefills ``batch`` prompts so that warm-up plus timed steps end at ``context``
    positions, then times ``steps`` decode steps on the device.  Returns (ms per step,
    kernels launched per step)."""
    import torch
    import toyinfer_b200.kernels as K
    vocab = engine.spec.vocab_size
    prompt_len = context - steps - warmup
    slots = [engine.new_sequence() for _ in range(batch)]
    try:
        # prompts run in groups so that the step's activations stay small; all start together
        engine.step([(s, random_tokens(prompt_len, vocab, seed + i)) for i, s in enumerate(slots)], [[] for _ in slots])
        toks = [random_tokens(steps + warmup, vocab, seed + 1000 + i) for i in range(batch)]
        for t in range(warmup):
            engine.step([(s, [toks[i][t]]) for i, s in enumerate(slots)], None)
        torch.cuda.synchronize()
        per_step = engine.launches_per_step(batch)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for t in range(warmup, warmup + steps):
            engine.step([(s, [toks[i][t]]) for i, s in enumerate(slots)], None)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps, per_step
    finally:
        for s in slots:
            engine.end_sequence(s)


def time_decode_range(engine, batch, start, end, seed=0):
    """Mean decode step time while ``batch`` sequences grow from ``start`` to ``end`` positions
    (tokens per second = batch / mean).  Token ids are chosen beforehand; timed on the device."""
    import torch
    vocab = engine.spec.vocab_size
    slots = [engine.new_sequence() for _ in range(batch)]
    try:
        engine.step([(s, random_tokens(start, vocab, seed + i)) for i, s in enumerate(slots)], [[] for _ in slots])
        steps = end - start
        toks = [random_tokens(steps, vocab, seed + 2000 + i) for i in range(batch)]
        for t in range(4):                          # warm-up (counts towards the lengths, not the time)
            engine.step([(s, [toks[i][t]]) for i, s in enumerate(slots)], None)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for t in range(4, steps):
            engine.step([(s, [toks[i][t]]) for i, s in enumerate(slots)], None)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (steps - 4)
    finally:
        for s in slots:
            engine.end_sequence(s)


def time_decode_sampled_range(engine, batch, lo, hi, points=13, steps=16, warm=32, seed=0):
    """Mean decode step time while ``batch`` sequences grow from ``lo`` to ``hi`` positions, sampled:
    at ``points`` evenly spaced lengths the step is timed over ``steps`` steps that end there (after
    ``warm`` untimed ones); between the samples the sequences are brought forward by whole pieces
    of tokens (a step that continues every sequence by several hundred tokens).  The mean weighs
    the two ends half (trapezoid rule): step time is close to linear in the length.  The warm-up is
    long on purpose: for some tens of milliseconds after a many-token step the decode steps run up to
    a tenth slower (the clocks come back slowly from the tensor cores' load), whichever kernels the
    many-token step used; with 3 warm-up steps the figure measured that step's intensity instead."""
    import torch
    vocab = engine.spec.vocab_size
    slots = [engine.new_sequence() for _ in range(batch)]
    times = []
    try:
        cur = 0
        for j in range(points):
            target = lo + (hi - lo) * j // (points - 1)
            upto = target - steps - warm
            engine.step([(s, random_tokens(upto - cur, vocab, seed + 31 * j + i)) for i, s in enumerate(slots)], [[] for _ in slots])
            cur = upto
            toks = [random_tokens(steps + warm, vocab, seed + 4000 + 31 * j + i) for i in range(batch)]
            for t in range(warm):
                engine.step([(s, [toks[i][t]]) for i, s in enumerate(slots)], None)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for t in range(warm, warm + steps):
                engine.step([(s, [toks[i][t]]) for i, s in enumerate(slots)], None)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) / steps)
            cur = target
        w = [0.5] + [1.0] * (points - 2) + [0.5]
        return sum(x * y for x, y in zip(w, times)) / sum(w)
    finally:
        for s in slots:
            engine.end_sequence(s)


def fp32_check():
    """The float32 engine (every kernel in true 32-bit) with two layers of the benchmark's sizes
    against the plain implementation in float64, which gets the same tensors: a 512-token prompt,
    then 8 tokens one by one.  The bound is the tests': |got - want| <= 1e-5 + 1e-4 |want|."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from plain import qwen3_plain as plain
    from toyinfer_b200 import models  # noqa: F401
    from toyinfer_b200.config import Qwen3Config, resolve_architecture
    from toyinfer_b200.engine import Engine
    from toyinfer_b200.parts.model import DecoderModel
    from toyinfer_b200.weights import random_parameters
    import toyinfer_b200.kernels as K
    cfg = dict(QWEN3_4B, num_hidden_layers=2)
    prompt, dec = 512, 8
    spec = resolve_architecture("Qwen3ForCausalLM").describe(Qwen3Config.from_dict(dict(cfg)))
    model = DecoderModel(spec, torch.float32, "cuda")
    weights = random_parameters(model.param_specs(), 5, torch.bfloat16, "cuda")
    model.bind({k: v.float() for k, v in weights.items()})
    eng = Engine(model, max_tokens=1024, max_batch=1, max_seq_len=1024)
    ids = random_tokens(prompt + dec, cfg["vocab_size"], 55)
    slot = eng.new_sequence()
    got = [eng.step([(slot, ids[:prompt])], None).clone()]
    for t in range(prompt, prompt + dec):
        got.append(eng.step([(slot, [ids[t]])], None).clone())
    K.check_status()
    got = torch.cat(got).double()
    want = plain.forward(weights, cfg, ids, None, rows=list(range(prompt - 1, prompt + dec))).to(got.device)
    err = (got - want).abs()
    over = (err / (1e-5 + 1e-4 * want.abs())).max().item()
    out = {"layers": 2, "prompt": prompt, "decoded": dec, "logits": int(got.numel()), "max_abs_err": float(f"{err.max().item():.3e}"),
           "max_abs_logit": round(want.abs().max().item(), 3), "rtol": 1e-4, "atol": 1e-5, "worst_err_over_bound": round(over, 3),
           "ok": bool(over <= 1.0), "against": "tests/plain/qwen3_plain.py in float64"}
    eng.end_sequence(slot)
    del eng, model, weights, got, want, err
    torch.cuda.empty_cache()
    return out


def time_prefill(engine, tokens, reps=3):
    import torch
    vocab = engine.spec.vocab_size
    best = None
    for r in range(reps + 1):
        slot = engine.new_sequence()
        ids = random_tokens(tokens, vocab, 77 + r)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([(slot, ids)], None)
        stop.record()
        torch.cuda.synchronize()
        engine.end_sequence(slot)
        ms = start.elapsed_time(stop)
        if r > 0:                      # the first run warms up
            best = ms if best is None else min(best, ms)
    return best


def run_ours(args):
    import torch
    from toyinfer_b200 import LLM, SamplingParams
    import toyinfer_b200.kernels as K

    pk = peaks()
    cfg = dict(QWEN3_4B)
    cfg["num_hidden_layers"] = args.layers
    batch, ctx = args.batch, args.context
    K.library()
    check = None if args.skip_points else fp32_check()
    big = max(batch, 64 if not args.skip_points else batch)
    max_tokens = max(batch * (ctx + 64), (64 * (ctx + 64)) if not args.skip_points else 0)
    limit = ctx if args.skip_points else max(ctx, LONG_CONTEXT)
    llm = LLM(config=cfg, seed=0, dtype="bfloat16", max_seq_len=limit, max_batch=big, max_tokens=max_tokens)
    engine = llm.engine

    sampler = ClockSampler()
    sampler.start()
    ms_step, per_step = time_decode(engine, batch, ctx, args.steps, args.warmup)
    clocks = sampler.stop()
    value = batch * 1000.0 / ms_step
    mean_ctx = ctx - args.steps / 2.0
    gbs = bytes_decode(cfg, batch, mean_ctx) / (ms_step * 1e-3) / 1e9

    # end to end through the entry point: host ids in, sampled ids back every step
    # (the first steps after the long prompts run at the clocks the prompts left behind, for
    # some tens of milliseconds; enough steps are generated that this does not decide the figure)
    e2e_steps = min(max(args.steps, 256), ctx // 4)
    prompts = [random_tokens(ctx - e2e_steps - 1, cfg["vocab_size"], 500 + i) for i in range(batch)]
    llm.generate(prompts[:1], SamplingParams(temperature=0.0), max_new_tokens=2, ignore_eos=True)     # warm-up
    torch.cuda.synchronize()
    llm.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=e2e_steps + 1, ignore_eos=True)
    st = llm.last_stats
    e2e_value = batch * st.decode_steps / st.decode_seconds if st.decode_seconds > 0 else None
    meta_bytes = engine.decode_metadata_bytes(batch)

    out = {
        "metric": "decode tokens/s", "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "impl": "ours",
        "config": {
            "model": "Qwen3-4B shape", "layers": args.layers, "layers_of_named_config": FULL_LAYERS,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "tied": True, "global_batch": batch, "seq_len": ctx, "context": ctx, "prefill_tokens": PREFILL_TOKENS,
            "points_context": PREFILL_TOKENS, "parallelism": "single GPU", "l2": "inputs larger than L2, no flush",
            "cuda_graph": True, "peaks": pk["source"], "range_points": "13 lengths from 2048 to context, 16 steps each after 32 untimed",
        },
        "e2e": {"value": round(e2e_value, 2) if e2e_value else None, "unit": "tokens/s",
                "steps": st.decode_steps, "h2d_bytes_per_step": meta_bytes, "d2h_bytes_per_step": batch * 4},
        "gpu_launches": per_step * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm_gbs"], 4)},
    }

    ms_pre = time_prefill(engine, PREFILL_TOKENS)
    fl = flops_prefill(cfg, PREFILL_TOKENS)
    out["prefill"] = {"value": round(PREFILL_TOKENS * 1000.0 / ms_pre, 1), "tokens": PREFILL_TOKENS,
                      "ms": round(ms_pre, 3), "frac": round(fl / (ms_pre * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    if args.range:
        ms_r = time_decode_range(engine, batch, PREFILL_TOKENS, ctx)
        out["range"] = {"from": PREFILL_TOKENS, "to": ctx, "batch": batch, "ms_per_step": round(ms_r, 4),
                        "value": round(batch * 1000.0 / ms_r, 2), "unit": "tokens/s"}
    if not args.skip_points:
        pts = {}
        # (32 untimed steps at least: one sequence's steps are short enough to feel the clocks coming back from
        # the prompt step before them, see time_decode_sampled_range; 452 against 475 tokens/s with 8)
        warm = max(args.warmup, 32)
        for b in (1, 64):
            ms_b, _ = time_decode(engine, b, PREFILL_TOKENS + args.steps + warm, args.steps, warm, seed=b)
            pts[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 2)
        # tokens per second averaged over the lengths from the prompt's 2,048 positions to the context
        for b in (1, 8, 64):
            ms_b = time_decode_sampled_range(engine, b, PREFILL_TOKENS, ctx, seed=10 * b)
            pts[f"range_b{b}"] = round(b * 1000.0 / ms_b, 2)
        ms_l, _ = time_decode(engine, 8, LONG_CONTEXT, args.steps, args.warmup, seed=3)
        pts[f"decode_b8_ctx{LONG_CONTEXT}"] = round(8 * 1000.0 / ms_l, 2)
        pts[f"hbm_frac_b8_ctx{LONG_CONTEXT}"] = round(bytes_decode(cfg, 8, LONG_CONTEXT - args.steps / 2.0) / (ms_l * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        del engine
        llm = None
        torch.cuda.empty_cache()
        # the same step with the layer sizes of Qwen3-8B (hidden 4,096, intermediate 12,288, untied head)
        llm8 = LLM(config=dict(QWEN3_8B), seed=0, dtype="bfloat16", max_seq_len=ctx, max_batch=8, max_tokens=8 * (ctx + 64))
        ms_8, _ = time_decode(llm8.engine, 8, ctx, args.steps, args.warmup, seed=4)
        pts["shape8b_decode_b8"] = round(8 * 1000.0 / ms_8, 2)
        pts["shape8b_hbm_frac_b8"] = round(bytes_decode(QWEN3_8B, 8, ctx - args.steps / 2.0) / (ms_8 * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        out["points"] = pts
        out["fp32_check"] = check
    return out


def run_workload(name: str):
    """The two larger workloads that BASELINE.json describes, end to end through ``LLM.generate``
    (host ids in, sampled ids out every step), random weights drawn on the device:
    8b: 16 prompts of lengths uniform in [64, 4096], 256 greedy tokens each;
    32b: 8 prompts of 2,048 tokens, 512 tokens each at temperature 0.7 with a fixed seed."""
    import torch
    from toyinfer_b200 import LLM, SamplingParams
    if name == "8b":
        cfg, n, new = QWEN3_8B, 16, 256
        g = torch.Generator().manual_seed(8)
        lens = torch.randint(64, 4097, (n,), generator=g).tolist()
        params = SamplingParams(temperature=0.0)
    else:
        cfg, n, new = QWEN3_32B, 8, 512
        lens = [2048] * n
        params = SamplingParams(temperature=0.7, top_k=0, top_p=1.0, seed=32)
    ctx = max(lens) + new
    t0 = time.perf_counter()
    llm = LLM(config=cfg, seed=0, dtype="bfloat16", max_seq_len=ctx, max_batch=n, max_tokens=sum((l + new + 63) // 64 * 64 for l in lens))
    t_build = time.perf_counter() - t0
    prompts = [random_tokens(l, cfg["vocab_size"], 900 + i) for i, l in enumerate(lens)]
    llm.generate(prompts[:1], params, max_new_tokens=2, ignore_eos=True)       # warm-up
    torch.cuda.synchronize()
    out = llm.generate(prompts, params, max_new_tokens=new, ignore_eos=True)
    st = llm.last_stats
    assert all(len(r.tokens) == new for r in out)
    return {"workload": name, "model": f"Qwen3-{name.upper()} shape, random weights, bfloat16", "layers": cfg["num_hidden_layers"],
            "sequences": n, "prompt_tokens": st.prompt_tokens, "new_tokens_each": new,
            "prefill_tokens_per_s": round(st.prompt_tokens / st.prefill_seconds, 1),
            "decode_tokens_per_s": round(n * st.decode_steps / st.decode_seconds, 1),
            "ms_per_decode_step": round(1e3 * st.decode_seconds / st.decode_steps, 3),
            "weights_gb": round(2 * sum(math.prod(sp.shape) for sp in llm.engine.model.param_specs().values()) / 1e9, 1),
            "build_seconds": round(t_build, 1), "through": "LLM.generate"}


def run_prompt_steps(lengths, layers: int):
    """One prompt of each given length through ``Engine.step`` on the benchmark model, host ids in,
    logits of the last place out: the mean of five steps after three untimed ones (a shape that comes
    back runs from a captured graph from its third time on, where the engine captures prompt steps).
    One JSON line per length."""
    import torch
    from toyinfer_b200 import LLM
    cfg = dict(QWEN3_4B)
    cfg["num_hidden_layers"] = layers
    limit = max(max(lengths) + 64, 4096)
    llm = LLM(config=cfg, seed=0, dtype="bfloat16", max_seq_len=limit, max_batch=8, max_tokens=2 * limit)
    eng = llm.engine
    for T in lengths:
        toks = random_tokens(T, cfg["vocab_size"], 1)

        def once():
            slot = eng.new_sequence()
            eng.step([(slot, toks)], None)
            eng.end_sequence(slot)

        for _ in range(3):
            once()
        torch.cuda.synchronize()
        replays = eng.graph_replays
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            once()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / 5
        print(json.dumps({"prompt_tokens": T, "layers": layers, "ms": round(ms, 3), "tokens_per_s": round(T / ms * 1e3, 1),
                          "captured": eng.graph_replays - replays == 5}), flush=True)


def run_mma_issue():
    """Cycles per tcgen05 MMA of 128 x N x 16 as one issuing thread per block sees them, with the thread
    chosen by ``lane == 0`` and by ``elect.sync`` in a warp-uniform branch, one and two blocks per SM
    (csrc/measure/mma_issue.cu).  One JSON line per case."""
    import ctypes
    import torch
    from toyinfer_b200.csrc.build import build
    lib = ctypes.CDLL(build(measure=True))       # the measurement kernels have a library of their own
    lib.ti_bench_mma_issue.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p] * 3
    lib.ti_last_error.restype = ctypes.c_char_p
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    names = {0: "A and B in shared memory, K-major", 1: "A in tensor memory, B K-major",
             2: "A in tensor memory, B MN-major", 3: "A in shared memory, B MN-major"}
    for per_sm in (1, 2):
        for n, mode in ((64, 0), (64, 1), (128, 0), (128, 1), (128, 2), (128, 3), (256, 0)):
            row = {"kernel": "mma_issue", "n": n, "operands": names[mode], "blocks_per_sm": per_sm, "mma_cycles": 128 * n * 16 * 2 // 8192}
            for elect in (0, 1):
                cyc, iss = ctypes.c_double(), ctypes.c_double()
                if lib.ti_bench_mma_issue(n, mode, elect, 64, sms * per_sm, ctypes.byref(cyc), ctypes.byref(iss), stream) != 0:
                    raise SystemExit(lib.ti_last_error().decode())
                row["elected" if elect else "lane0"] = round(cyc.value, 1)
            print(json.dumps(row), flush=True)


# ---------------------------------------------------------------------------
# one kernel at a time, at the sizes of one layer of the benchmark model
# ---------------------------------------------------------------------------
def run_kernel(name: str, reps: int, eager: bool = False):
    """Times one kernel on a small case and reports its rate against the roofline.  Launches run
    back to back (replayed from a CUDA graph) over several sets of operands that together exceed
    the L2 (126 MB), so every launch reads from memory; the time is the CUDA-event total divided
    by the launches.  Small enough to sit under ncu."""
    import math
    import torch
    import toyinfer_b200.kernels as K
    from toyinfer_b200.cache.manager import KVView
    from toyinfer_b200.engine.batch import BatchBuffers, fill_batch

    pk = peaks()
    dev = "cuda"
    if name == "mma_issue":
        return run_mma_issue()
    g = torch.Generator(device=dev).manual_seed(0)
    H, I = 2560, 9728

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(torch.bfloat16)

    def make():
        if name.startswith("gemm:"):                     # gemm:M,N,K or gemm:M,N,K,BN,SPLITS (tile width and splits forced)
            M, N, Kd, *force = (int(v) for v in name[5:].split(","))
            if force:
                from toyinfer_b200.kernels import gemm
                gemm.set_tile_force(force[0], force[1] if len(force) > 1 else 0)
            x, w = rnd(M, Kd), rnd(N, Kd, scale=0.02)
            return (lambda: K.linear(x, w)), (N * Kd + M * Kd + M * N) * 2, 2.0 * M * N * Kd
        if name in ("gemm_decode", "gemm_decode_b64", "gemm_prefill", "gemm_head", "gemm_down", "gemm_qkv", "gemm_o"):
            M = {"gemm_decode_b64": 64, "gemm_prefill": 2048}.get(name, 8)
            N, Kd = {"gemm_head": (151936, H), "gemm_down": (H, I), "gemm_qkv": (6144, H), "gemm_o": (H, 4096)}.get(name, (2 * I, H))
            x, w = rnd(M, Kd), rnd(N, Kd, scale=0.02)
            return (lambda: K.linear(x, w)), (N * Kd + M * Kd + M * N) * 2, 2.0 * M * N * Kd
        if name in ("attn_decode", "attn_decode_b64", "attn_decode_b1"):
            B, ctx = {"attn_decode": (8, 8192), "attn_decode_b64": (64, 2048), "attn_decode_b1": (1, 2048)}[name]
            nh, nkv, hd = 32, 8, 128
            pages = B * ctx // 64
            table = (torch.arange(pages, dtype=torch.int32, device=dev).view(B, ctx // 64) + 1)
            table = torch.cat([table, torch.zeros(1, ctx // 64, dtype=torch.int32, device=dev)]).contiguous()
            mem = KVView(rnd(pages + 1, nkv, 64, hd), rnd(pages + 1, nkv, 64, hd), table, nkv, hd, 0, 0)
            batch = fill_batch(BatchBuffers(B, B, dev), "extend", list(range(B)), [ctx - 1] * B, [[0]] * B, B, ctx)
            q = rnd(B, nh, hd)
            return (lambda: K.attention_decode(q, mem, 1 / math.sqrt(hd), 0, batch)), 2 * B * ctx * nkv * hd * 2, 4.0 * B * ctx * nh * hd
        if name.startswith("add_rmsnorm"):                # add_rmsnorm or add_rmsnorm:TOKENS
            T = int(name.split(":")[1]) if ":" in name else PREFILL_TOKENS
            h, d, w = rnd(T, H), rnd(T, H, scale=0.01), rnd(H)
            return (lambda: K.add_rmsnorm(h, d, w, 1e-6)), 4 * T * H * 2, 0.0
        if name.startswith("rope_store"):                 # rope_store or rope_store:TOKENS
            from toyinfer_b200.parts.rope import rotary_tables
            T, nh, nkv, hd = (int(name.split(":")[1]) if ":" in name else PREFILL_TOKENS), 32, 8, 128
            pages = (T + 63) // 64
            table = torch.zeros(2, pages, dtype=torch.int32, device=dev)
            table[0] = torch.arange(1, pages + 1, dtype=torch.int32, device=dev)
            mem = KVView(rnd(pages + 1, nkv, 64, hd), rnd(pages + 1, nkv, 64, hd), table, nkv, hd, 0, 0)
            qkv = rnd(T, (nh + 2 * nkv) * hd)
            q = qkv[:, :nh * hd].view(T, nh, hd)
            k = qkv[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
            v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)
            qw, kw = rnd(hd), rnd(hd)
            cos, sin = rotary_tables(hd, 1e6, T + 64)
            tables = (cos.to(dev), sin.to(dev), hd)
            batch = fill_batch(BatchBuffers(1, T, dev), "start", [0], [0], [[0] * T], 1, T)
            # q and k read and written in place, v read, k and v written to the pages
            return (lambda: K.qk_norm_rope_store(q, k, v, qw, kw, 1e-6, tables, batch, mem)), \
                (2 * nh + 2 * nkv + nkv + 2 * nkv) * T * hd * 2, 0.0
        if name.startswith("attn_prefill"):               # attn_prefill or attn_prefill:TOKENS
            T, nh, nkv, hd = (int(name.split(":")[1]) if ":" in name else PREFILL_TOKENS), 32, 8, 128
            qkv = rnd(T, (nh + 2 * nkv) * hd)
            q = qkv[:, :nh * hd].view(T, nh, hd)
            k = qkv[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
            v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)
            batch = fill_batch(BatchBuffers(1, T, dev), "start", [0], [0], [[0] * T], 1, T)
            return (lambda: K.attention_prefill(q, k, v, 1 / math.sqrt(hd), 0, batch)), qkv.numel() * 2 + T * nh * hd * 2, \
                4.0 * nh * hd * T * (T + 1) / 2
        if name.startswith("attn_chunk"):                 # attn_chunk or attn_chunk:CACHED,NEW[,HEAD_DIM]
            sizes = [int(v) for v in name.split(":")[1].split(",")] if ":" in name else [2048, 2048]
            cached, new = sizes[:2]
            nh, nkv, hd = 32, 8, (sizes[2] if len(sizes) > 2 else 128)
            pages = (cached + new + 63) // 64
            table = torch.zeros(2, pages, dtype=torch.int32, device=dev)
            table[0] = torch.arange(1, pages + 1, dtype=torch.int32, device=dev)
            mem = KVView(rnd(pages + 1, nkv, 64, hd), rnd(pages + 1, nkv, 64, hd), table, nkv, hd, 0, 0)
            qkv = rnd(new, (nh + 2 * nkv) * hd)
            q = qkv[:, :nh * hd].view(new, nh, hd)
            k = qkv[:, nh * hd:(nh + nkv) * hd].view(new, nkv, hd)
            v = qkv[:, (nh + nkv) * hd:].view(new, nkv, hd)
            batch = fill_batch(BatchBuffers(1, new, dev), "mixed", [0], [cached], [[0] * new], 1, cached + new)
            return (lambda: K.attention_chunk(q, k, v, mem, 1 / math.sqrt(hd), 0, batch)), \
                qkv.numel() * 2 + new * nh * hd * 2 + 2 * cached * nkv * hd * 2, 4.0 * nh * hd * new * (cached + (new + 1) / 2)
        raise SystemExit(f"unknown kernel case {name!r}")

    fn, nbytes, flops = make()
    sets = [fn]
    while len(sets) * nbytes < 400e6 and len(sets) < 16:
        sets.append(make()[0])
    for f in sets:
        f()
    torch.cuda.synchronize()
    # one pass over the sets captured into a CUDA graph, as decode steps are in serving: the
    # host's launch rate (tens of microseconds per call from Python) stays out of the number
    if eager:                      # plain launches (for a profiler that wants to see each one)
        class _Eager:
            def replay(self):
                for f in sets:
                    f()
        graph = _Eager()
    else:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for f in sets:
                f()
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    K.check_status()
    ms = a.elapsed_time(b) / (reps * len(sets))
    return {"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "tflops": round(flops / ms / 1e9, 1),
            "hbm_frac": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4), "tensor_frac": round(flops / ms / 1e9 / pk["bf16_tflops"], 4),
            "peaks": pk["source"], "launches": reps * len(sets), "operand_sets": len(sets)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the named configuration (reported)")
    ap.add_argument("--skip-points", action="store_true", help="leave out the batch 1 and 64 points")
    ap.add_argument("--range", action="store_true",
                    help="also the mean decode rate while the batch grows from 2,048 positions to --context (some 20 s more)")
    ap.add_argument("--kernel", default="", help="time one kernel alone instead: gemm_decode, gemm_decode_b64, gemm_down, "
                    "gemm_qkv, gemm_o, gemm_head, gemm_prefill, gemm:M,N,K[,BN,SPLITS], attn_decode, attn_decode_b64, attn_decode_b1, "
                    "attn_prefill[:TOKENS], attn_chunk[:CACHED,NEW[,HEAD_DIM]], add_rmsnorm[:TOKENS], rope_store[:TOKENS], mma_issue; "
                    "ref:all or ref:<case> times the reference's kernel recompiled for sm_100a beside this library's")
    ap.add_argument("--workload", default="", choices=["", "8b", "32b"],
                    help="run one of the larger described workloads end to end instead (8B or 32B shape)")
    ap.add_argument("--prompt-steps", default="", help="time one prompt step of each of these lengths instead (comma-separated), "
                    "with --layers layers")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--eager", action="store_true", help="with --kernel: plain launches instead of a graph replay")
    args = ap.parse_args()
    if args.kernel.startswith("ref:"):
        # the reference's own kernels, recompiled for sm_100a, beside this library's (baseline/ref_kernels.py)
        from baseline import ref_kernels
        names = ref_kernels.CASES if args.kernel == "ref:all" else [args.kernel[4:]]
        for n in names:
            sampler = ClockSampler()
            sampler.start()
            row = ref_kernels.run(n, args.reps)
            row["clocks"] = sampler.stop()
            print(json.dumps(row), flush=True)
        return 0
    if args.kernel:
        result = run_kernel(args.kernel, args.reps, args.eager)
        if result is not None:          # mma_issue prints its own lines
            print(json.dumps(result))
        return 0
    if args.workload:
        print(json.dumps(run_workload(args.workload)))
        return 0
    if args.prompt_steps:
        run_prompt_steps([int(v) for v in args.prompt_steps.split(",")], args.layers)
        return 0
    if args.impl == "reference":
        print(json.dumps({"impl": "reference",
                          "unavailable": "wiketool/ToyInfer has no setup.py or pyproject.toml (pip: 'not installable'); it is a "
                                         "CMake program whose third_party sources are absent and that builds for sm_89 only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
