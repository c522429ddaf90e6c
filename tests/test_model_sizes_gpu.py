"""Real Qwen3 layer sizes with random weights against the plain implementation: two layers of
the 4B shape (hidden 2560, 32 heads over 8 kv heads of 128, intermediate 9728, vocabulary
151936) and one layer of the 32B shape (64 heads over 8 kv heads, hidden 5120).  The plain
implementation's elementary operations run on the GPU in float64 here (on the CPU they would
take minutes at this size); it gets the very tensors the engines are built from.

The float32 engine must match it at rtol 1e-4 (the form of the reference's own kernel tests,
tests/test_helpers.h:70-72: |got - want| <= atol + rtol |want|), the bfloat16 engine (tcgen05
matrix products and attention, TMA, CUDA graphs) the plain implementation rounded where bfloat16
is stored, at the bound of helpers.assert_logits_close.  Every way of cutting the work is run:
whole prompts, the last 32 tokens one by one, unequal batches with early ends in a cache small
enough that slots and pages come back, and a prompt fed in pieces beside decoding sequences."""
from __future__ import annotations

import pytest
import torch

from helpers import assert_logits_close, rounding_of
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

CFG_4B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 2560,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728,
    "vocab_size": 151936, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "max_position_embeddings": 40960,
    "tie_word_embeddings": True,
}
# one layer of the 32B shape: 8 query heads per kv head, untied head
CFG_32B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 5120,
    "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 25600,
    "vocab_size": 32000, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "max_position_embeddings": 40960,
    "tie_word_embeddings": False,
}
CFGS = {"4B-shape": CFG_4B, "32B-shape": CFG_32B}
DTYPES = ["float32", "bfloat16"]


class Sized:
    """The weights of one shape (bfloat16 values, on the GPU), an engine per precision built from
    them, and the plain implementation's logits of a sequence's wanted places."""

    def __init__(self, cfg):
        from toyinfer_b200 import models  # noqa: F401
        from toyinfer_b200.config import Qwen3Config, resolve_architecture
        from toyinfer_b200.parts.model import DecoderModel
        from toyinfer_b200.weights import random_parameters
        self.cfg = cfg
        arch = resolve_architecture("Qwen3ForCausalLM")
        self.spec = arch.describe(Qwen3Config.from_dict(dict(cfg)))
        probe = DecoderModel(self.spec, torch.bfloat16, "cuda")
        self.weights = random_parameters(probe.param_specs(), 123, torch.bfloat16, "cuda")
        self._engines = {}
        self._plain = {}

    def engine(self, dtype, **kw):
        from toyinfer_b200.engine import Engine
        from toyinfer_b200.parts.model import DecoderModel
        dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
        if dtype not in self._engines:
            model = DecoderModel(self.spec, dt, "cuda")
            model.bind({k: v.to(dt) for k, v in self.weights.items()})
            self._engines[dtype] = model
        kw.setdefault("max_tokens", 64 * 64)
        kw.setdefault("max_batch", 4)
        kw.setdefault("max_seq_len", 4096)
        return Engine(self._engines[dtype], **kw)

    def want(self, ids, rows, dtype):
        key = (tuple(ids), tuple(rows), dtype)
        if key not in self._plain:
            self._plain[key] = plain.forward(self.weights, self.cfg, ids, rounding_of(dtype), rows=rows).cpu()
        return self._plain[key]


@pytest.fixture(scope="module", params=list(CFGS))
def sized(request):
    s = Sized(CFGS[request.param])
    yield s
    del s
    torch.cuda.empty_cache()


def ids_for(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompts_and_the_last_32_one_by_one(sized, dtype):
    import toyinfer_b200.kernels as K
    eng = sized.engine(dtype)
    for n in (1, 65, 300):
        ids = ids_for(sized.cfg, [n], seed=n)[0]
        rows = sorted({0, n // 2, n - 1})
        slot = eng.new_sequence()
        got = eng.step([(slot, ids)], [rows])
        assert_logits_close(got, sized.want(ids, rows, dtype), dtype, f"whole prompt of {n}")
        eng.end_sequence(slot)
    n = 200
    ids = ids_for(sized.cfg, [n], seed=7)[0]
    rows = list(range(n - 33, n))
    slot = eng.new_sequence()
    got = [eng.step([(slot, ids[:n - 32])], [[n - 33]]).clone()]
    for t in range(n - 32, n):
        got.append(eng.step([(slot, [ids[t]])], [[0]]).clone())
    K.check_status()
    assert_logits_close(torch.cat(got), sized.want(ids, rows, dtype), dtype, "the last 32 one by one")
    if dtype == "bfloat16":
        assert eng.graph_replays >= 30


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_one_after_another(sized, dtype):
    """Prompts of 700, 129 and 1 tokens, then decoding with early ends; then a second batch in the
    same slots and pages (the cache holds 24 pages: both batches together would not fit)."""
    import toyinfer_b200.kernels as K
    eng = sized.engine(dtype, max_tokens=64 * 24, max_batch=4)
    for r, (lens, dec) in enumerate((([700, 129, 1], [6, 2, 4]), ([1100, 40], [3, 5]))):
        seqs = ids_for(sized.cfg, [n + d for n, d in zip(lens, dec)], seed=20 + r)
        rows = [list(range(n - 1, n + d)) for n, d in zip(lens, dec)]
        want = [sized.want(s, rw, dtype) for s, rw in zip(seqs, rows)]
        slots = [eng.new_sequence() for _ in seqs]
        logits = eng.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)], None).clone()
        for i in range(len(seqs)):
            assert_logits_close(logits[i], want[i][0], dtype, f"batch {r} prompt {i}")
        live, t = list(range(len(seqs))), 0
        while live:
            logits = eng.step([(slots[i], [seqs[i][lens[i] + t]]) for i in live], None).clone()
            for row, i in enumerate(live):
                assert_logits_close(logits[row], want[i][1 + t], dtype, f"batch {r} sequence {i} step {t}")
            t += 1
            for i in [i for i in live if t >= dec[i]]:
                eng.end_sequence(slots[i])
            live = [i for i in live if t < dec[i]]
        K.check_status()
        assert eng.cache.slots.n_free == eng.cache.n_slots
        assert all(g.pool.n_free == g.pool.n_pages for g in eng.cache.kv_groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_in_pieces_beside_decoding_sequences(sized, dtype):
    import toyinfer_b200.kernels as K
    eng = sized.engine(dtype)
    a, b = ids_for(sized.cfg, [500, 90], seed=31)
    cuts = [0, 7, 71, 72, 400, 500]
    wa = sized.want(a, [c - 1 for c in cuts[1:]], dtype)
    wb = sized.want(b, list(range(79, 79 + len(cuts) - 1)), dtype)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    eng.step([(sb, b[:79])], [[]])
    for i, (lo, hi) in enumerate(zip(cuts, cuts[1:])):
        out = eng.step([(sa, a[lo:hi]), (sb, [b[79 + i]])], None).clone()
        assert_logits_close(out[0], wa[i], dtype, f"piece {lo}:{hi}")
        assert_logits_close(out[1], wb[i], dtype, f"the decoding sequence beside piece {lo}:{hi}")
    K.check_status()
