"""The engine on the GPU against the plain implementation, in float32 and bfloat16:
each request alone and whole; with the last 32 tokens one by one; in batches of unequal
lengths whose shorter requests end earlier, batch after batch so that slots are used
again; long decoding; the first tokens of a sequence; a prompt cut into pieces; a prompt
that starts beside sequences that decode; graph replay against eager steps.

Configurations A, B and C have heads of 16, 32 and 48 (the CUDA-core attention kernels in
both precisions); D (heads of 128) and E (heads of 64, a window equal to its ring) put the
bfloat16 tensor-core attention kernels under the same schedules."""
from __future__ import annotations

import pytest
import torch

from conftest import TINY, prompts_for
from helpers import assert_logits_close, plain_logits

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C", "D", "E"]
WINDOWED = ("C", "E")


def make_engine(folder, dtype, **kw):
    from toyinfer_b200.engine import Engine
    kw.setdefault("max_tokens", 4096)
    kw.setdefault("max_batch", 8)
    return Engine.from_folder(folder, dtype=dtype, device="cuda", **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(model_folders, name, dtype):
    eng = make_engine(model_folders[name], dtype)
    lens = [1, 2, 17, 64, 65, 100] if name not in WINDOWED else [1, 40, 41, 130, 200]
    for i, ids in enumerate(prompts_for(name, lens, seed=3)):
        slot = eng.new_sequence()
        got = eng.step([(slot, ids)], [list(range(len(ids)))])
        assert_logits_close(got, plain_logits(model_folders[name], ids, dtype), dtype, f"{name} len {len(ids)}")
        eng.end_sequence(slot)


@pytest.mark.parametrize("graph", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(model_folders, name, dtype, graph):
    eng = make_engine(model_folders[name], dtype, use_cuda_graph=graph)
    n = {"A": 100, "B": 77, "C": 190, "D": 150, "E": 200}[name]
    ids = prompts_for(name, [n], seed=4)[0]
    want = plain_logits(model_folders[name], ids, dtype)
    slot = eng.new_sequence()
    head = n - 32
    got = [eng.step([(slot, ids[:head])], [[head - 1]]).clone()]
    for t in range(head, n):
        got.append(eng.step([(slot, [ids[t]])], [[0]]).clone())
    assert_logits_close(torch.cat(got), want[head - 1:], dtype, f"{name} one by one")
    if graph:
        assert eng.graph_replays >= 30


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens_token_by_token(model_folders, name, dtype):
    """A sequence fed from its very first token through single-token steps."""
    eng = make_engine(model_folders[name], dtype)
    ids = prompts_for(name, [70], seed=5)[0]
    want = plain_logits(model_folders[name], ids, dtype)
    slot = eng.new_sequence()
    got = [eng.step([(slot, [t])], [[0]]).clone() for t in ids]
    assert_logits_close(torch.cat(got), want, dtype, f"{name} from the first token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_one_after_another(model_folders, name, dtype):
    # a cache of 8 pages: three batches can only run if pages and slots come back
    eng = make_engine(model_folders[name], dtype, max_tokens=64 * 8, max_batch=4)
    plans = [([5, 9, 2], [8, 8, 8]), ([17, 1, 40, 8], [12, 3, 7, 1]), ([70, 3, 100], [4, 20, 9])]
    for r, (lens, dec) in enumerate(plans):
        seqs = prompts_for(name, [n + d for n, d in zip(lens, dec)], seed=20 + r)
        want = [plain_logits(model_folders[name], s, dtype) for s in seqs]
        slots = [eng.new_sequence() for _ in seqs]
        logits = eng.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)], None).clone()
        for i, n in enumerate(lens):
            assert_logits_close(logits[i], want[i][n - 1], dtype, f"{name} batch {r} prompt {i}")
        live, t = list(range(len(seqs))), 0
        while live:
            logits = eng.step([(slots[i], [seqs[i][lens[i] + t]]) for i in live], None).clone()
            for row, i in enumerate(live):
                assert_logits_close(logits[row], want[i][lens[i] + t], dtype, f"{name} batch {r} seq {i} step {t}")
            t += 1
            for i in [i for i in live if t >= dec[i]]:
                eng.end_sequence(slots[i])
            live = [i for i in live if t < dec[i]]
        assert eng.cache.slots.n_free == eng.cache.n_slots
        assert all(g.pool.n_free == g.pool.n_pages for g in eng.cache.kv_groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_a_prompt_cut_into_pieces(model_folders, name, dtype):
    """A sequence fed 7, 64, 1 tokens, a long piece, then 16 + 16 more: every place's logits are
    those of the whole sequence.  With a window the pieces are longer than its ring has slack."""
    eng = make_engine(model_folders[name], dtype)
    n = {"A": 120, "B": 200, "C": 300, "D": 400, "E": 330}[name]
    ids = prompts_for(name, [n], seed=8)[0]
    want = plain_logits(model_folders[name], ids, dtype)
    slot = eng.new_sequence()
    cuts = [0, 7, 71, 72, n - 32, n - 16, n]
    got = []
    for a, b in zip(cuts, cuts[1:]):
        got.append(eng.step([(slot, ids[a:b])], [list(range(b - a))]).clone())
        assert eng.length(slot) == b
    assert_logits_close(torch.cat(got), want, dtype, f"{name} in pieces")
    # and the same again in the slot's next use, cut elsewhere
    eng.end_sequence(slot)
    slot = eng.new_sequence()
    got = [eng.step([(slot, ids[a:b])], [list(range(b - a))]).clone() for a, b in ((0, 65), (65, 66), (66, n))]
    assert_logits_close(torch.cat(got), want, dtype, f"{name} in pieces, second use of the slot")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_a_prompt_joins_sequences_that_decode(model_folders, name, dtype):
    """Two sequences decode; a third starts beside them with its whole prompt in the same step;
    then one of the first two goes on by five tokens at once while the others go on by one."""
    eng = make_engine(model_folders[name], dtype)
    la = 110 if name == "A" else 150          # A holds 128 positions
    h = la - 20
    a, b, c = prompts_for(name, [la, 45, 100], seed=9)
    wa, wb, wc = (plain_logits(model_folders[name], x, dtype) for x in (a, b, c))
    sa, sb = eng.new_sequence(), eng.new_sequence()
    eng.step([(sa, a[:h]), (sb, b[:30])], [[], []])
    out = eng.step([(sa, [a[h]]), (sb, [b[30]])], None).clone()
    assert_logits_close(out, torch.stack([wa[h], wb[30]]), dtype, f"{name} before the join")
    sc = eng.new_sequence()
    out = eng.step([(sa, [a[h + 1]]), (sc, c[:80]), (sb, [b[31]])], [[0], [0, 79], [0]]).clone()
    assert_logits_close(out, torch.stack([wa[h + 1], wc[0], wc[79], wb[31]]), dtype, f"{name} the join")
    out = eng.step([(sa, a[h + 2:h + 7]), (sc, [c[80]]), (sb, [b[32]])], [[4], [0], [0]]).clone()
    assert_logits_close(out, torch.stack([wa[h + 6], wc[80], wb[32]]), dtype, f"{name} five at once")
    out = eng.step([(sa, [a[h + 7]]), (sc, [c[81]]), (sb, [b[33]])], None).clone()
    assert_logits_close(out, torch.stack([wa[h + 7], wc[81], wb[33]]), dtype, f"{name} after the join")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["C", "E"])
def test_long_decoding(model_folders, name, dtype):
    """More than 200 single-token steps after a short prompt (ring wrapped three times; in E
    the ring has no slack: the newest position overwrites the one that just left the window)."""
    eng = make_engine(model_folders[name], dtype)
    ids = prompts_for(name, [300], seed=6)[0]
    want = plain_logits(model_folders[name], ids, dtype)
    slot = eng.new_sequence()
    got = [eng.step([(slot, ids[:9])], [[8]]).clone()]
    for t in range(9, 300):
        got.append(eng.step([(slot, [ids[t]])], [[0]]).clone())
    assert_logits_close(torch.cat(got), want[8:], dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_across_a_length_class(tmp_path, dtype):
    """Decode steps are captured per class of sequence lengths (powers of two from 1,024): a
    sequence that grows from 1,000 to 1,050 positions moves from one captured step to the next,
    with another sequence of 30 positions beside it; both must follow the plain implementation."""
    from toyinfer_b200.weights import write_model_folder
    cfg = dict(TINY["A"], max_position_embeddings=2304)
    folder = write_model_folder(cfg, 17, str(tmp_path / "long"))
    eng = make_engine(folder, dtype, max_tokens=4096, max_batch=2)
    g = torch.Generator().manual_seed(4)
    long_ids = torch.randint(0, cfg["vocab_size"], (1050,), generator=g).tolist()
    short_ids = torch.randint(0, cfg["vocab_size"], (80,), generator=g).tolist()
    want_long, want_short = plain_logits(folder, long_ids, dtype), plain_logits(folder, short_ids, dtype)
    a, b = eng.new_sequence(), eng.new_sequence()
    eng.step([(a, long_ids[:1000]), (b, short_ids[:30])], [[], []])
    got_a, got_b = [], []
    for t in range(50):
        out = eng.step([(a, [long_ids[1000 + t]]), (b, [short_ids[30 + t]])], [[0], [0]])
        got_a.append(out[0:1].clone())
        got_b.append(out[1:2].clone())
    assert len(eng._graphs) == 2        # the keys of 1,024 and of 2,048 positions are split differently here
    assert_logits_close(torch.cat(got_a), want_long[1000:1050], dtype, "across a length class, long")
    assert_logits_close(torch.cat(got_b), want_short[30:80], dtype, "across a length class, short")


def test_length_classes_with_the_same_launches_share_a_captured_step(tmp_path):
    """Where nothing in the model's launches tells two classes of lengths apart (heads of 128 in
    bfloat16: sixteen splits of the keys from 2,048 positions on), a sequence that grows past the
    class's end keeps replaying the same captured step, and stays right."""
    from toyinfer_b200.weights import write_model_folder
    dtype = "bfloat16"
    cfg = dict(TINY["D"], max_position_embeddings=4608)
    folder = write_model_folder(cfg, 19, str(tmp_path / "longer"))
    eng = make_engine(folder, dtype, max_tokens=8192, max_batch=2)
    assert eng.model.launch_plan(2, 2048) == eng.model.launch_plan(2, 4096) != eng.model.launch_plan(2, 1024)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg["vocab_size"], (2070,), generator=g).tolist()
    want = plain_logits(folder, ids, dtype)
    a = eng.new_sequence()
    eng.step([(a, ids[:2030])], [[]])
    got = [eng.step([(a, [ids[2030 + t]])], [[0]]).clone() for t in range(40)]
    assert len(eng._graphs) == 1 and eng.graph_replays >= 38
    assert_logits_close(torch.cat(got), want[2030:2070], dtype, "across two length classes with one captured step")


def test_a_partly_filled_batch_splits_its_keys_and_a_full_one_does_not(model_folders, monkeypatch):
    """The decode attention's plan looks at how many sequences of the padded batch are real: five of eight
    on a device of (here pretended) four SMs would leave a thin second round of blocks and are split
    two ways, eight of eight are not; two captured steps for one batch size, the plain implementation's
    logits from both, also when the batch shrinks from one to the other."""
    from toyinfer_b200.kernels import attention, gemm
    monkeypatch.setattr(attention, "sm_count", lambda device: 4)
    monkeypatch.setattr(gemm, "sm_count", lambda device: 4)
    monkeypatch.setattr(attention, "cluster_room", lambda hd, fused, splits: 8 // splits)      # two blocks on each of them
    name, dtype = "D", "bfloat16"
    eng = make_engine(model_folders[name], dtype, max_batch=8, max_tokens=64 * 40)
    assert eng.model.launch_plan(8, 1024, 5)[0][0] == 2 and eng.model.launch_plan(8, 1024, 8)[0][0] == 1
    lens = [70, 9, 130, 33, 64, 5, 90, 17]
    seqs = prompts_for(name, [n + 6 for n in lens], seed=80)
    want = [plain_logits(model_folders[name], s, dtype) for s in seqs]
    slots = [eng.new_sequence() for _ in seqs]
    eng.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)], [[] for _ in seqs])
    live = list(range(8))
    for t in range(6):
        if t == 3:                                   # three sequences end: five of eight go on
            for i in (1, 4, 6):
                eng.end_sequence(slots[i])
            live = [i for i in live if i not in (1, 4, 6)]
        logits = eng.step([(slots[i], [seqs[i][lens[i] + t]]) for i in live], None).clone()
        for row, i in enumerate(live):
            assert_logits_close(logits[row], want[i][lens[i] + t], dtype, f"sequence {i} step {t} of {len(live)} live")
    assert len(eng._graphs) == 2 and eng.graph_replays >= 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_and_company_change_nothing(model_folders, dtype):
    """A request's logits are the same alone, in a batch of 3 (padded to 4 by the graph's
    bucket) and in a batch of 5 (padded to 8), beyond rounding."""
    name = "B"
    seqs = prompts_for(name, [30, 11, 50, 6, 19], seed=7)
    outs = []
    for group in ([0], [0, 1, 2], [0, 1, 2, 3, 4]):
        eng = make_engine(model_folders[name], dtype)
        slots = [eng.new_sequence() for _ in group]
        a = eng.step([(s, seqs[i][:-4]) for s, i in zip(slots, group)], None)[0].clone()
        rows = [a]
        for t in range(4, 0, -1):
            rows.append(eng.step([(s, [seqs[i][-t]]) for s, i in zip(slots, group)], None)[0].clone())
        outs.append(torch.stack(rows))
    want = plain_logits(model_folders[name], seqs[0], dtype)[-5:]
    for o in outs:
        assert_logits_close(o, want, dtype, "company")
    if dtype == "float32":
        torch.testing.assert_close(outs[0], outs[2], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_shapes_that_come_back_run_from_a_captured_step(model_folders, name, dtype):
    """Batches of prompts whose rounded shape is the same: the first runs as it is, the second is
    captured, the others are replayed.  Each prompt's logits and the tokens decoded after it (they read
    what the prompt step left in the cache) are the plain implementation's, and slots are used again."""
    eng = make_engine(model_folders[name], dtype, max_tokens=64 * 12, max_batch=4)
    assert eng.prompt_graph_tokens > 0
    # three sequences and 65-128 tokens each time (128 token rows), the longest prompt 33-64
    rounds = [[40, 9, 33], [64, 1, 20], [35, 35, 35], [50, 2, 60], [33, 33, 1]]
    for r, lens in enumerate(rounds):
        seqs = prompts_for(name, [n + 3 for n in lens], seed=40 + r)
        want = [plain_logits(model_folders[name], s, dtype) for s in seqs]
        slots = [eng.new_sequence() for _ in seqs]
        logits = eng.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)], None).clone()
        for i, n in enumerate(lens):
            assert_logits_close(logits[i], want[i][n - 1], dtype, f"{name} round {r} prompt {i}")
        for t in range(3):
            logits = eng.step([(sl, [s[n + t]]) for sl, s, n in zip(slots, seqs, lens)], None).clone()
            for i, n in enumerate(lens):
                assert_logits_close(logits[i], want[i][n + t], dtype, f"{name} round {r} seq {i} step {t}")
        for sl in slots:
            eng.end_sequence(sl)
    assert len(eng._prompt_graphs) == 1
    assert eng.graph_replays >= 3 + 5 * 2          # prompt rounds 2-4, and every round's decode steps but its first
    # other wanted places than each prompt's last are not the captured step's business
    slot = eng.new_sequence()
    ids = prompts_for(name, [40], seed=50)[0]
    for _ in range(3):
        got = eng.step([(slot, ids)], [[0, 39]])
        assert_logits_close(got, plain_logits(model_folders[name], ids, dtype)[[0, 39]], dtype, "two wanted places")
        eng.end_sequence(slot)
        slot = eng.new_sequence()
    assert len(eng._prompt_graphs) == 1


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_captured_prompt_step_with_and_without_spare_rows(model_folders, dtype):
    """One prompt of 33-64 tokens is one shape of 64 token rows: full, or with up to 31 rows of nobody's."""
    eng = make_engine(model_folders["D"], dtype)
    for i, n in enumerate((64, 50, 64, 33, 64)):
        ids = prompts_for("D", [n + 2], seed=70 + i)[0]
        want = plain_logits(model_folders["D"], ids, dtype)
        slot = eng.new_sequence()
        got = [eng.step([(slot, ids[:n])], None).clone()] + [eng.step([(slot, [t])], None).clone() for t in ids[n:]]
        assert_logits_close(torch.cat(got), want[n - 1:], dtype, f"prompt of {n}")
        eng.end_sequence(slot)
    assert list(eng._prompt_graphs) == [(1, 64, 64)]


def test_captured_prompt_steps_are_kept_to_a_number(model_folders):
    eng = make_engine(model_folders["B"], "bfloat16", max_tokens=64 * 12, max_batch=4)
    eng.max_prompt_graphs = 2
    for n in (10, 70, 130, 10):                # three shapes (64, 128 and 192 token rows); the first comes back
        ids = prompts_for("B", [n], seed=60)[0]
        want = plain_logits(model_folders["B"], ids, "bfloat16")[-1]
        for _ in range(3):
            slot = eng.new_sequence()
            assert_logits_close(eng.step([(slot, ids)], None)[0], want, "bfloat16", f"prompt of {n}")
            eng.end_sequence(slot)
        assert len(eng._prompt_graphs) <= 2
    assert [k[1] for k in eng._prompt_graphs] == [192, 64]


def test_step_refuses_what_it_cannot_run(model_folders):
    from toyinfer_b200.engine import StepError
    eng = make_engine(model_folders["A"], "float32")
    a, b = eng.new_sequence(), eng.new_sequence()
    eng.step([(a, [1, 2, 3])], None)
    with pytest.raises(StepError):
        eng.step([(b, [10 ** 6])], None)            # token outside the vocabulary
    with pytest.raises(StepError):
        eng.step([(a, [4]), (a, [5])], None)        # a slot twice
    with pytest.raises(StepError):
        eng.step([(a, [])], None)                   # no token
    with pytest.raises(StepError):
        eng.step([(a, [1] * 200)], None)            # beyond the model's positions
    with pytest.raises(StepError):
        eng.step([(a, None), (b, [1, 2])], None, token_source=torch.zeros(2, dtype=torch.int32, device="cuda"))
    assert eng.length(a) == 3 and eng.length(b) == 0    # nothing was changed


@pytest.mark.parametrize("seed", [1, 2, 3])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "C", "D", "E"])
def test_random_schedules(model_folders, name, dtype, seed):
    """Requests of random lengths come and go as a random schedule decides: a step takes a random
    subset of the live sequences, each with a random number of its next tokens (one, a few, a long
    piece), new sequences start beside them, finished ones give their slot and pages back, in a cache
    so small that both come around again.  Every position's logits must be those of its sequence
    alone and whole, whatever kept it company."""
    import random
    from helpers import run_random_schedule
    rng = random.Random(1000 * seed + sum(map(ord, name + dtype)))
    longest = {"B": 200, "C": 300, "D": 500, "E": 330}[name]
    eng = make_engine(model_folders[name], dtype, max_batch=4, max_tokens=4 * (longest + 64))
    lens = [rng.choice([1, 2, 17, 63, 64, 65, rng.randint(66, longest)]) for _ in range(7)]
    ids = prompts_for(name, lens, seed=40 + seed)
    got = run_random_schedule(eng, ids, rng)
    for r, x in enumerate(ids):
        assert_logits_close(got[r], plain_logits(model_folders[name], x, dtype), dtype,
                            f"{name} request {r} of {lens[r]} tokens, seed {seed}")
