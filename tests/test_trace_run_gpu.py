"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits files compared
with the plain implementation; whole requests, the last 32 tokens one by one, unequal
batches with early ends and reused slots, and a request fed in pieces beside one that
goes on token by token."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, TINY, prompts_for
from helpers import assert_logits_close, plain_logits

pytestmark = pytest.mark.gpu


def run_trace(folder, dtype, steps, out_dir, max_tokens=2048):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for s in steps:
        p.stdin.write(json.dumps(s) + "\n")
        p.stdin.flush()
        line = p.stdout.readline().strip()
        assert line == f"done {s['step']}", line
    p.stdin.close()
    assert p.wait(timeout=120) == 0


def read_step(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_trace_whole_then_one_by_one_then_batches(model_folders, tmp_path, name, dtype):
    folder, V = model_folders[name], TINY[name]["vocab_size"]
    a, b, c, d = prompts_for(name, [90, 150 if name == "C" else 100, 3, 41], seed=30)
    steps, checks = [], []
    # request a: whole, all places wanted, ended at once
    steps.append({"step": 0, "entries": [{"id": "a", "tokens": a, "want": list(range(len(a)))}], "end": ["a"]})
    checks.append((0, [(a, list(range(len(a))))]))
    # request b: whole prefix, then the last 32 tokens one by one
    head = len(b) - 32
    steps.append({"step": 1, "entries": [{"id": "b", "tokens": b[:head], "want": [head - 1]}], "end": []})
    checks.append((1, [(b, [head - 1])]))
    for t in range(head, len(b)):
        last = t == len(b) - 1
        steps.append({"step": len(steps), "entries": [{"id": "b", "tokens": [b[t]], "want": [0]}],
                      "end": ["b"] if last else []})
        checks.append((len(steps) - 1, [(b, [t])]))
    # a batch of three unequal requests that reuse the slots; c ends first, then d
    n0 = len(steps)
    pa, pc, pd = len(a) - 6, len(c) - 2, len(d) - 4
    steps.append({"step": n0, "entries": [{"id": "a2", "tokens": a[:pa], "want": [pa - 1]},
                                          {"id": "c", "tokens": c[:pc], "want": []},
                                          {"id": "d", "tokens": d[:pd], "want": [0, pd - 1]}], "end": []})
    checks.append((n0, [(a, [pa - 1]), (d, [0, pd - 1])]))
    for t in range(6):
        entries, chk, end = [{"id": "a2", "tokens": [a[pa + t]], "want": [0]}], [(a, [pa + t])], []
        if t < 2:
            entries.append({"id": "c", "tokens": [c[pc + t]], "want": [0]})
            chk.append((c, [pc + t]))
            if t == 1:
                end.append("c")
        if t < 4:
            entries.append({"id": "d", "tokens": [d[pd + t]], "want": [0]})
            chk.append((d, [pd + t]))
            if t == 3:
                end.append("d")
        if t == 5:
            end.append("a2")
        steps.append({"step": n0 + 1 + t, "entries": entries, "end": end})
        checks.append((n0 + 1 + t, chk))
    # request e in pieces of 20, 64 and the rest, while f starts with the second piece and then
    # goes on one token at a time
    e, f = prompts_for(name, [len(b), 30], seed=31)
    n1 = len(steps)
    steps.append({"step": n1, "entries": [{"id": "e", "tokens": e[:20], "want": [19]}], "end": []})
    checks.append((n1, [(e, [19])]))
    steps.append({"step": n1 + 1, "entries": [{"id": "e", "tokens": e[20:84], "want": [0, 63]},
                                              {"id": "f", "tokens": f[:28], "want": [27]}], "end": []})
    checks.append((n1 + 1, [(e, [20, 83]), (f, [27])]))
    steps.append({"step": n1 + 2, "entries": [{"id": "f", "tokens": [f[28]], "want": [0]},
                                              {"id": "e", "tokens": e[84:], "want": [len(e) - 85]}], "end": ["e"]})
    checks.append((n1 + 2, [(f, [28]), (e, [len(e) - 1])]))
    steps.append({"step": n1 + 3, "entries": [{"id": "f", "tokens": [f[29]], "want": [0]}], "end": ["f"]})
    checks.append((n1 + 3, [(f, [29])]))
    out = str(tmp_path / "out")
    run_trace(folder, dtype, steps, out, max_tokens=64 * 6)
    for step, parts in checks:
        got = read_step(out, step, V)
        want = torch.cat([plain_logits(folder, ids, dtype)[places] for ids, places in parts])
        assert_logits_close(got, want, dtype, f"{name} step {step}")
