"""The library's engine, cache and batching driven on the CPU (kernels replaced by the
torch stand-ins of tests/cpu_kernels.py) against the plain implementation: whole
prompts, the last tokens one by one, and unequal batches one after another."""
from __future__ import annotations

import pytest
import torch

import cpu_kernels
from conftest import TINY, prompts_for
from plain import qwen3_plain as plain
from toyinfer_b200.engine import Engine


@pytest.fixture()
def cpu_engine(monkeypatch, model_folders):
    cpu_kernels.install(monkeypatch)

    def make(name, **kw):
        kw.setdefault("max_tokens", 2048)
        kw.setdefault("max_batch", 8)
        return Engine.from_folder(model_folders[name], dtype="float32", device="cpu", **kw)

    return make


def _plain_logits(folder, ids):
    return plain.forward(plain.read_weights(folder), plain.read_config(folder), ids).float()


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompt_matches_plain(cpu_engine, model_folders, name):
    eng = cpu_engine(name)
    ids = prompts_for(name, [90 if name == "C" else 37])[0]
    slot = eng.new_sequence()
    got = eng.step([(slot, ids)], [list(range(len(ids)))])
    want = _plain_logits(model_folders[name], ids)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
    eng.end_sequence(slot)


@pytest.mark.parametrize("seed", [1, 2])
@pytest.mark.parametrize("name", ["B", "C"])
def test_random_schedules(cpu_engine, model_folders, name, seed):
    """Requests come and go as a random schedule decides (helpers.run_random_schedule), in a cache
    so small that slots and pages come around again: every position's logits are those of its
    sequence alone and whole."""
    import random
    from helpers import run_random_schedule
    rng = random.Random(77 * seed + ord(name))
    longest = {"B": 150, "C": 200}[name]
    eng = cpu_engine(name, max_batch=3, max_tokens=3 * (longest + 64))
    lens = [rng.choice([1, 2, 63, 64, 65, rng.randint(66, longest)]) for _ in range(5)]
    ids = prompts_for(name, lens, seed=50 + seed)
    got = run_random_schedule(eng, ids, rng, max_live=3)
    for r, x in enumerate(ids):
        torch.testing.assert_close(got[r], _plain_logits(model_folders[name], x), rtol=1e-4, atol=1e-5,
                                   msg=lambda m: f"{name} request {r} of {lens[r]} tokens, seed {seed}: {m}")


@pytest.mark.parametrize("name", ["A", "C"])
def test_last_tokens_one_by_one(cpu_engine, model_folders, name):
    eng = cpu_engine(name)
    n = 150 if name == "C" else 60
    ids = prompts_for(name, [n], seed=1)[0]
    want = _plain_logits(model_folders[name], ids)
    slot = eng.new_sequence()
    head = n - 32
    got = [eng.step([(slot, ids[:head])], [[head - 1]])]
    for t in range(head, n):
        got.append(eng.step([(slot, [ids[t]])], [[0]]).clone())
    got = torch.cat(got)
    torch.testing.assert_close(got, want[head - 1:], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_a_prompt_cut_into_pieces(cpu_engine, model_folders, name):
    """A sequence fed 7, 64, 1 tokens, then the rest, then 16 + 16 more: every place's logits are
    those of the whole sequence.  In C the pieces are longer than the window's ring has slack."""
    eng = cpu_engine(name)
    n = 230 if name == "C" else 120
    ids = prompts_for(name, [n], seed=2)[0]
    want = _plain_logits(model_folders[name], ids)
    slot = eng.new_sequence()
    cuts = [0, 7, 71, 72, n - 32, n - 16, n]
    got = []
    for a, b in zip(cuts, cuts[1:]):
        got.append(eng.step([(slot, ids[a:b])], [list(range(b - a))]).clone())
        assert eng.length(slot) == b
    torch.testing.assert_close(torch.cat(got), want, rtol=1e-4, atol=1e-5)
    eng.end_sequence(slot)


@pytest.mark.parametrize("name", ["A", "C"])
def test_a_prompt_joins_sequences_that_decode(cpu_engine, model_folders, name):
    """Two sequences decode; a third starts beside them with its whole prompt in the same step, and
    one of the first two goes on by five tokens at once in the step after."""
    eng = cpu_engine(name)
    a, b, c = prompts_for(name, [90, 45, 70], seed=5)
    wa, wb, wc = (_plain_logits(model_folders[name], x) for x in (a, b, c))
    sa, sb = eng.new_sequence(), eng.new_sequence()
    eng.step([(sa, a[:80]), (sb, b[:30])], [[], []])
    out = eng.step([(sa, [a[80]]), (sb, [b[30]])], None)
    torch.testing.assert_close(out, torch.stack([wa[80], wb[30]]), rtol=1e-4, atol=1e-5)
    sc = eng.new_sequence()
    out = eng.step([(sa, [a[81]]), (sc, c[:60]), (sb, [b[31]])], [[0], [0, 59], [0]])
    torch.testing.assert_close(out, torch.stack([wa[81], wc[0], wc[59], wb[31]]), rtol=1e-4, atol=1e-5)
    out = eng.step([(sa, a[82:87]), (sc, [c[60]]), (sb, [b[32]])], [[4], [0], [0]])
    torch.testing.assert_close(out, torch.stack([wa[86], wc[60], wb[32]]), rtol=1e-4, atol=1e-5)
    out = eng.step([(sa, [a[87]]), (sc, [c[61]]), (sb, [b[33]])], None)
    torch.testing.assert_close(out, torch.stack([wa[87], wc[61], wb[33]]), rtol=1e-4, atol=1e-5)


def test_unequal_batches_reuse_slots(cpu_engine, model_folders):
    name = "C"
    eng = cpu_engine(name, max_tokens=64 * 8)
    for round_ in range(3):
        lens = [70, 3, 130, 41][: 4 - round_ % 2]
        dec = [5, 9, 2, 7]
        seqs = prompts_for(name, [n + d for n, d in zip(lens, dec)], seed=10 + round_)
        want = [_plain_logits(model_folders[name], s) for s in seqs]
        slots = [eng.new_sequence() for _ in seqs]
        logits = eng.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)], None)
        for i, n in enumerate(lens):
            torch.testing.assert_close(logits[i], want[i][n - 1], rtol=1e-4, atol=1e-5)
        live = list(range(len(seqs)))
        t = 0
        while live:
            logits = eng.step([(slots[i], [seqs[i][lens[i] + t]]) for i in live], None)
            for r, i in enumerate(live):
                torch.testing.assert_close(logits[r], want[i][lens[i] + t], rtol=1e-4, atol=1e-5)
            t += 1
            for i in [i for i in live if t >= dec[i]]:
                eng.end_sequence(slots[i])
            live = [i for i in live if t < dec[i]]
        assert eng.cache.slots.n_free == eng.cache.n_slots
        for g in eng.cache.kv_groups:
            assert g.pool.n_free == g.pool.n_pages


def test_a_layers_keys_and_values_are_let_go_after_their_last_user(cpu_engine, monkeypatch):
    """What a schedule entry leaves for entries that borrow its memory (this step's keys and
    values) must not outlive its last user: kept until the step's end it pins every layer's
    projection buffer (at 260,000 prompt tokens that was 3 GB per layer)."""
    from toyinfer_b200.parts.attention import GQAAttention
    eng = cpu_engine("B")
    seen = []
    inner = GQAAttention.forward

    def forward(self, x, batch, mem, shared):
        assert all(not d for d in seen), "an earlier entry's keys and values are still held"
        seen.append(shared)
        return inner(self, x, batch, mem, shared)

    monkeypatch.setattr(GQAAttention, "forward", forward)
    slot = eng.new_sequence()
    eng.step([(slot, prompts_for("B", [9])[0])], None)
    assert len(seen) == TINY["B"]["num_hidden_layers"] and all(not d for d in seen)
    eng.end_sequence(slot)


def test_a_norm_left_to_the_readers_product_changes_no_result(cpu_engine, model_folders, monkeypatch):
    """Single-token steps with the norm handed on as a kernels.PendingNorm (the sum h + delta then
    lands in a new tensor, and the block must go on with that one) give the logits of plain steps."""
    import toyinfer_b200.kernels as K
    name = "B"
    ids = prompts_for(name, [40], seed=3)[0]

    def run(eng):
        slot = eng.new_sequence()
        got = [eng.step([(slot, ids[:8])], [[7]])]
        for t in range(8, len(ids)):
            got.append(eng.step([(slot, [ids[t]])], [[0]]).clone())
        eng.end_sequence(slot)
        return torch.cat(got)

    plain_steps = run(cpu_engine(name))
    made = []

    def pending_norm(h, delta, weight, eps):
        if h.shape[0] != 1:
            return None
        made.append(1)
        return cpu_kernels.PendingOutOfPlace(h, delta, weight, eps)

    monkeypatch.setattr(K, "pending_norm", pending_norm)
    pending_steps = run(cpu_engine(name))
    assert len(made) == 2 * TINY[name]["num_hidden_layers"] * (len(ids) - 8)      # both norms of every layer, every single-token step
    assert torch.equal(pending_steps, plain_steps)
    want = _plain_logits(model_folders[name], ids)
    torch.testing.assert_close(pending_steps, want[7:], rtol=1e-4, atol=1e-5)


def test_other_ends_of_a_model(cpu_engine, model_folders, monkeypatch):
    """A description with an embedding multiplier, a logit scale and soft cap, and no final norm is
    built from the shipped embedding and head parts (nothing in the library is edited) and follows
    the same layers computed plainly with those ends."""
    import math
    from toyinfer_b200.config.registry import load_config
    from toyinfer_b200.parts import PartSpec
    from toyinfer_b200.parts.model import DecoderModel
    from toyinfer_b200.weights import load_parameters
    cpu_engine("A")          # installs the CPU stand-ins
    folder = model_folders["B"]
    arch, cfg = load_config(folder)
    spec = arch.describe(cfg)
    scale, lscale, cap = math.sqrt(cfg.hidden_size), 0.5, 3.0
    spec.embedding = PartSpec("token_table", {"vocab_size": cfg.vocab_size, "scale": scale})
    spec.head = PartSpec("linear", {"vocab_size": cfg.vocab_size, "norm": None, "tied": False, "scale": lscale, "softcap": cap})
    model = DecoderModel(spec, torch.float32, "cpu")
    assert "model.norm.weight" not in model.param_specs()
    model.bind(load_parameters(model.param_specs(), folder, torch.float32, model.device, ignorable=("model.norm.weight",)))
    eng = Engine(model, max_tokens=512, max_batch=2)
    ids = prompts_for("B", [23], seed=12)[0]
    slot = eng.new_sequence()
    got = torch.cat([eng.step([(slot, ids[:20])], [list(range(20))]), eng.step([(slot, ids[20:])], [[0, 1, 2]])])
    w, c = plain.read_weights(folder), plain.read_config(folder)
    h = plain.embedding(w["model.embed_tokens.weight"], ids) * scale
    for layer in range(c["num_hidden_layers"]):
        h = plain.decoder_layer(h, w, c, layer)
    logits = plain.linear(h, w["lm_head.weight"]) * lscale
    want = cap * torch.tanh(logits / cap)
    torch.testing.assert_close(got.double(), want, rtol=1e-4, atol=1e-5)


def test_sizes_no_kernel_takes_are_refused_when_the_model_is_built():
    """Before any weight is read: heads of 6 elements (the attention kernels want a multiple of 4)
    and 40 query heads of 128 per kv head in float32 (beyond the CUDA-core decode kernel)."""
    from toyinfer_b200 import models  # noqa: F401
    from toyinfer_b200.config import Qwen3Config, resolve_architecture
    from toyinfer_b200.kernels import KernelError
    from toyinfer_b200.parts.model import DecoderModel
    arch = resolve_architecture("Qwen3ForCausalLM")
    cfg = dict(TINY["A"], head_dim=6)
    with pytest.raises(KernelError, match="head size 6"):
        DecoderModel(arch.describe(Qwen3Config.from_dict(cfg)), torch.float32, "cpu")
    cfg = dict(TINY["A"], head_dim=128, num_attention_heads=40, num_key_value_heads=1)
    with pytest.raises(KernelError, match="40 query heads per kv head"):
        DecoderModel(arch.describe(Qwen3Config.from_dict(cfg)), torch.float32, "cpu")
    DecoderModel(arch.describe(Qwen3Config.from_dict(cfg)), torch.bfloat16, "cpu")       # the tensor-core kernels take it


def test_default_cache_size_asks_the_cache_for_bytes_per_token():
    from toyinfer_b200.cache import bytes_per_token
    from toyinfer_b200.parts import KVRequest, StateRequest
    reqs = [KVRequest(2, 16), None, KVRequest(8, 128, window=64), StateRequest((5,), torch.float32)]
    assert bytes_per_token(reqs, torch.bfloat16) == 2 * 2 * 16 * 2 + 2 * 8 * 128 * 2
    assert bytes_per_token(reqs, torch.float32) == 2 * (2 * 2 * 16 * 2 + 2 * 8 * 128 * 2)
    assert bytes_per_token([None, StateRequest((5,))], torch.float32) == 0


def test_decode_attention_merges_as_clusters_only_when_all_find_room(monkeypatch):
    """The plan of a decode step's attention: splits of two pages merged inside clusters when the
    device holds all clusters at once with some to spare, else splits of four pages merged through
    scratch memory; the same answer for the same padded batch and planned length."""
    from toyinfer_b200.kernels import attention
    room = {16: 14, 9: 30, 8: 33, 4: 71, 2: 148}
    monkeypatch.setattr(attention, "cluster_room", lambda hd, fused, splits: room.get(splits, 296 // splits))
    monkeypatch.setattr(attention, "_combine_late", lambda n_seq: n_seq <= 16)
    plan = lambda n_seq, length, tc=True: attention.decode_plan(n_seq, 32, 8, 128, length, 64, 148, tc, True)
    assert plan(1, 2112) == (16, 2)          # 8 clusters of 16, room for 14
    assert plan(2, 2112) == (9, 1)           # 16 clusters of 16 do not fit: nine splits of four pages
    assert plan(4, 2112) == (9, 1)           # 32 clusters of 9, room for 30
    assert plan(8, 2112) == (4, 2)           # 64 of 4, room for 71
    assert plan(8, 100) == (1, 1)            # two pages: nothing to split
    assert plan(32, 2112) == (1, 0)          # a block per SM without splits
    assert plan(1, 2112, tc=False) == (9, 1)   # the CUDA-core kernel knows no clusters
    monkeypatch.setattr(attention, "force_merge_mode", 2)
    assert plan(2, 2112) == (16, 2)
    monkeypatch.setattr(attention, "force_merge_mode", 0)
    assert plan(1, 2112) == (9, 0)


def test_decode_attention_splits_the_keys_of_a_batch_that_would_leave_a_thin_second_round(monkeypatch):
    """A padded batch whose real sequences give a few more long blocks than run at once (two per SM) has
    its keys split after all; batches that fit one round, or fill two, are left whole."""
    from toyinfer_b200.kernels import attention
    splits = lambda n_live, length, n_seq=64: attention.decode_splits(n_seq, 8, length, 64, 148, n_live=n_live)
    assert [splits(n, 8192) for n in (32, 37, 38, 44, 45, 48, 53, 54, 64)] == [1, 1, 4, 4, 2, 2, 2, 1, 1]
    assert [splits(n, 2048) for n in (37, 38, 48, 53, 54, 64)] == [1, 2, 2, 2, 1, 1]
    assert splits(40, 100) == 1                                  # two pages: nothing to split
    assert attention.decode_splits(64, 8, 8192, 64, 148) == 1    # asked without the number of real sequences
    assert splits(8, 8192, n_seq=8) == 4                         # a batch that fits: as before
    places = {128: 296, 64: 592}
    monkeypatch.setattr(attention, "cluster_room", lambda hd, fused, splits: places[hd] // splits)
    plan = lambda n_live, hd=128: attention.decode_plan(64, 32, 8, hd, 8192, 64, 148, True, True, n_live)
    assert plan(64) == (1, 0) and plan(40) == (4, 0)             # merged through scratch memory: no room for 512 clusters
    assert plan(40, hd=64) == (1, 0)                             # smaller blocks, four per SM: 320 of them run at once


def test_spare_token_rows_of_a_step_of_fixed_size_change_nothing(cpu_engine, model_folders):
    """The form of a captured prompt step: more token rows than the sequences hold.  The spare rows stand at
    position 0 of a stand-in sequence in the scratch slot; the sequences' logits and what they leave in
    the cache are those of the plain implementation."""
    from toyinfer_b200.engine.batch import BatchBuffers, fill_batch
    name = "B"
    eng = cpu_engine(name)
    seqs = prompts_for(name, [21, 8, 34], seed=9)
    heads = [s[:-1] for s in seqs]
    slots = [eng.new_sequence() for _ in seqs]
    for s, ids in zip(slots, heads):
        eng.cache.reserve(s, len(ids))
    eng.cache.flush()
    buf = BatchBuffers(len(seqs) + 1, 128, "cpu")
    batch = fill_batch(buf, "start", slots, [0] * 3, heads, eng.cache.scratch_slot, eng.max_seq_len, total_tok=128, new_bound=64)
    used = sum(len(h) for h in heads)
    assert (batch.n_seq, batch.n_tok, batch.n_real_tok, batch.max_new) == (3, 128, used, 64)
    assert batch.seq_slot.tolist() == slots + [eng.cache.scratch_slot] and batch.seq_new.tolist() == [20, 7, 33, 0]
    assert batch.tok_seq[used:].tolist() == [3] * (128 - used) and batch.tok_pos[used:].tolist() == [0] * (128 - used)
    assert batch.cu_new.tolist() == [0, 20, 27, 60, 60]
    h, delta = eng.model.forward_hidden(batch, eng.memories)
    got = eng.model.logits(h, delta, batch.cu_new[1:4] - 1)
    for s, ids in zip(slots, heads):
        eng.cache.commit(s, len(ids))
    for i, ids in enumerate(seqs):
        want = _plain_logits(model_folders[name], ids)
        torch.testing.assert_close(got[i], want[-2], rtol=1e-4, atol=1e-5)
        nxt = eng.step([(slots[i], [ids[-1]])], None)         # reads what the padded step stored
        torch.testing.assert_close(nxt[0], want[-1], rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError):                            # spare rows need room for the stand-in sequence
        fill_batch(BatchBuffers(3, 128, "cpu"), "start", slots, [0] * 3, heads, eng.cache.scratch_slot, eng.max_seq_len, total_tok=128)
