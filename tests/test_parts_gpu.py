"""Each part of a model alone against the plain implementation, and the generality of
the assembly: a toy mixer with a state of its own, a toy feed-forward with routing and
another position encoding are defined here, registered, built and stepped without a
change to the library's files; a schedule that names a layer twice and lets a layer read
another layer's cache runs and matches a plain composition of the same parts."""
from __future__ import annotations

import math

import pytest
import torch

from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


def lib():
    import toyinfer_b200.kernels as K
    from toyinfer_b200 import parts
    from toyinfer_b200.cache import CacheManager
    from toyinfer_b200.engine import Engine
    from toyinfer_b200.engine.batch import BatchBuffers, fill_batch
    from toyinfer_b200.parts.model import DecoderModel, LayerSpec, ModelSpec, ScheduleEntry
    from toyinfer_b200.weights import random_parameters
    return dict(K=K, parts=parts, CacheManager=CacheManager, Engine=Engine, BatchBuffers=BatchBuffers,
                fill_batch=fill_batch, DecoderModel=DecoderModel, LayerSpec=LayerSpec, ModelSpec=ModelSpec,
                ScheduleEntry=ScheduleEntry, random_parameters=random_parameters)


def bind_random(part, seed, dtype):
    """Draws the part's tensors on the CPU (float32), binds device copies, returns the CPU ones."""
    from toyinfer_b200.weights import random_parameters
    cpu = random_parameters(part.param_specs(), seed, torch.float32, "cpu")
    if dtype == torch.bfloat16:
        cpu = {k: v.to(torch.bfloat16).float() for k, v in cpu.items()}
    part.bind({k: v.to(DEV, dtype) for k, v in cpu.items()})
    return cpu


def ctx_for(dtype, hidden, positions=None):
    from toyinfer_b200.parts import BuildContext
    c = BuildContext(dtype=dtype, device=torch.device(DEV), hidden_size=hidden)
    c.positions.update(positions or {})
    return c


def batch_for(mode, slots, starts, news, scratch):
    L = lib()
    buf = L["BatchBuffers"](len(slots), sum(news), DEV)
    return L["fill_batch"](buf, mode, slots, starts, [[0] * n for n in news], scratch, 4096)


def rmode(dtype):
    return None if dtype == torch.float32 else torch.bfloat16


def tol(dtype):
    return dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=6e-3)


DT = [torch.float32, torch.bfloat16]


# ---------------------------------------------------------------------------
# the shipped parts, one at a time
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DT)
def test_norm_part(dtype):
    from toyinfer_b200.parts import PartSpec, build_part
    n = build_part("norm", PartSpec("rmsnorm", {"size": 72, "eps": 1e-5}), ctx_for(dtype, 72), "x.")
    w = bind_random(n, 1, dtype)["x.weight"]
    g = torch.Generator().manual_seed(0)
    h = torch.randn(5, 72, generator=g).to(dtype)
    d = torch.randn(5, 72, generator=g).to(dtype)
    torch.testing.assert_close(n.forward(h.to(DEV)).cpu().double(), plain.rms_norm(h.double(), w, 1e-5, rmode(dtype)), **tol(dtype))
    hd = h.to(DEV).clone()
    y = n.add_forward(hd, d.to(DEV))
    hs = plain.rnd(h.double() + d.double(), rmode(dtype))
    torch.testing.assert_close(hd.cpu().double(), hs, **tol(dtype))
    torch.testing.assert_close(y.cpu().double(), plain.rms_norm(hs, w, 1e-5, rmode(dtype)), **tol(dtype))


def test_position_part_tables():
    from toyinfer_b200.parts import PartSpec, build_part
    p = build_part("position", PartSpec("rotary_half", {"dim": 48, "theta": 5e5, "max_positions": 300}),
                   ctx_for(torch.float32, 8), "")
    cos, sin, dim = p.rotary_tables()
    ang = plain.rope_angles(48, 5e5, range(300))
    assert dim == 48 and cos.shape == (300, 24)
    torch.testing.assert_close(cos.cpu().double(), torch.cos(ang), rtol=0, atol=1e-7)
    torch.testing.assert_close(sin.cpu().double(), torch.sin(ang), rtol=0, atol=1e-7)


@pytest.mark.parametrize("dtype", DT)
def test_feed_forward_part(dtype):
    from toyinfer_b200.parts import PartSpec, build_part
    f = build_part("feed_forward", PartSpec("swiglu", {"intermediate_size": 200}), ctx_for(dtype, 96), "m.")
    w = bind_random(f, 2, dtype)
    x = torch.randn(7, 96, generator=torch.Generator().manual_seed(3)).to(dtype)
    got = f.forward(x.to(DEV), None).cpu().double()
    r = rmode(dtype)
    gate, up = plain.linear(x.double(), w["m.gate_proj.weight"], r), plain.linear(x.double(), w["m.up_proj.weight"], r)
    want = plain.linear(plain.swiglu(gate, up, r), w["m.down_proj.weight"], r)
    torch.testing.assert_close(got, want, **tol(dtype))


@pytest.mark.parametrize("hidden,inter", [(96, 200), (2560, 1000)])
def test_norm_left_to_the_feed_forwards_product(hidden, inter):
    """One bfloat16 token: the norm part hands a pending norm on, the feed-forward's first product
    forms the input itself, and the sum h + delta comes back as the new hidden state; against the
    plain implementation, and against the same parts with the norm kernel (same bits for rows longer
    than 1,024, where both sum in the same order)."""
    import toyinfer_b200.kernels as K
    from toyinfer_b200.parts import PartSpec, build_part
    dtype = torch.bfloat16
    n = build_part("norm", PartSpec("rmsnorm", {"size": hidden, "eps": 1e-6}), ctx_for(dtype, hidden), "n.")
    f = build_part("feed_forward", PartSpec("swiglu", {"intermediate_size": inter}), ctx_for(dtype, hidden), "m.")
    wn = bind_random(n, 4, dtype)["n.weight"]
    w = bind_random(f, 5, dtype)
    g = torch.Generator().manual_seed(6)
    h = torch.randn(1, hidden, generator=g).to(dtype)
    d = (0.5 * torch.randn(1, hidden, generator=g)).to(dtype)
    assert f.takes_pending_norm
    h_dev = h.to(DEV)
    pending = n.add_pending(h_dev, d.to(DEV))
    assert isinstance(pending, K.PendingNorm)
    got = f.forward(pending, None)
    r = torch.bfloat16
    hs = plain.rnd(h.double() + d.double(), r)
    x = plain.rms_norm(hs, wn, 1e-6, r)
    gate, up = plain.linear(x, w["m.gate_proj.weight"], r), plain.linear(x, w["m.up_proj.weight"], r)
    want = plain.linear(plain.swiglu(gate, up, r), w["m.down_proj.weight"], r)
    torch.testing.assert_close(got.cpu().double(), want, **tol(dtype))
    torch.testing.assert_close(pending.hidden().cpu().double(), hs, rtol=0, atol=0)
    assert torch.equal(h_dev.cpu(), h)                       # the sum went to a new tensor
    h2 = h.to(DEV)
    apart = f.forward(n.add_forward(h2, d.to(DEV)), None)    # norm kernel, then the products
    assert torch.equal(h2, pending.hidden())
    if hidden > 1024:
        assert torch.equal(apart, got)
    else:
        torch.testing.assert_close(apart.float(), got.float(), **tol(dtype))
    # more than one token: the norm part does the work itself
    two = n.add_pending(torch.zeros(2, hidden, dtype=dtype, device=DEV), torch.zeros(2, hidden, dtype=dtype, device=DEV))
    assert isinstance(two, torch.Tensor)


def plain_attention_layer(x, w, p, nh, nkv, hd, eps, theta, window, r, positions=None, rope_fn=None):
    T = x.shape[0]
    q = plain.linear(x, w[p + "q_proj.weight"], r).view(T, nh, hd)
    k = plain.linear(x, w[p + "k_proj.weight"], r).view(T, nkv, hd)
    v = plain.linear(x, w[p + "v_proj.weight"], r).view(T, nkv, hd)
    q, k = plain.rms_norm(q, w[p + "q_norm.weight"], eps, r), plain.rms_norm(k, w[p + "k_norm.weight"], eps, r)
    if rope_fn is None:
        ang = plain.rope_angles(hd, theta, range(T))
        q, k = plain.rope(q, ang, r), plain.rope(k, ang, r)
    else:
        q, k = rope_fn(q), rope_fn(k)
    a = plain.attention(q, k, v, 1 / math.sqrt(hd), window, r)
    return plain.linear(a.reshape(T, nh * hd), w[p + "o_proj.weight"], r), (k, v)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 0), (5, 1, 48, 40), (4, 2, 64, 0)])
def test_attention_mixer_alone(dtype, nh, nkv, hd, window):
    """The mixer with memory from a cache manager: a whole prompt, then tokens one by one."""
    from toyinfer_b200.cache import CacheManager
    from toyinfer_b200.parts import PartSpec, build_part
    H, eps, theta, n, extra = 80, 1e-6, 1e4, 70, 6
    ctx = ctx_for(dtype, H)
    ctx.positions["rope"] = build_part("position", PartSpec("rotary_half", {"dim": hd, "theta": theta, "max_positions": 256}), ctx, "")
    m = build_part("mixer", PartSpec("gqa_attention", {"n_heads": nh, "n_kv_heads": nkv, "head_dim": hd,
                                                        "qk_norm_eps": eps, "position": "rope", "window": window}), ctx, "a.")
    w = bind_random(m, 4, dtype)
    cache = CacheManager([m.memory_request()], 64 * 8, 3, 256, dtype, DEV)
    x = torch.randn(n + extra, H, generator=torch.Generator().manual_seed(5)).to(dtype)
    want, _ = plain_attention_layer(x.double(), w, "a.", nh, nkv, hd, eps, theta, window, rmode(dtype))
    cache.allocate_slot()                     # slot 0 stays empty; the sequence lives in slot 1
    s = cache.allocate_slot()
    cache.reserve(s, n)
    cache.flush()
    got = m.forward(x[:n].to(DEV), batch_for("start", [s], [0], [n], cache.scratch_slot), cache.view(0), {})
    torch.testing.assert_close(got.cpu().double(), want[:n], **tol(dtype))
    cache.commit(s, n)
    for t in range(n, n + extra):
        cache.reserve(s, t + 1)
        cache.flush()
        got = m.forward(x[t:t + 1].to(DEV), batch_for("extend", [s], [t], [1], cache.scratch_slot), cache.view(0), {})
        torch.testing.assert_close(got.cpu().double(), want[t:t + 1], **tol(dtype))
        cache.commit(s, t + 1)


# ---------------------------------------------------------------------------
# toy parts defined here, not in the library
# ---------------------------------------------------------------------------
def make_toy_parts():
    import toyinfer_b200.kernels as K
    from toyinfer_b200.parts import FeedForward, Mixer, ParamSpec, PositionEncoding, StateRequest, register_part

    class DecayMixer(Mixer):
        """state <- decay * state + W x;  y = state.  A state of its own per sequence."""

        def __init__(self, ctx, prefix, decay):
            self.h, self.decay, self.name = ctx.hidden_size, float(decay), prefix + "w.weight"
            self.dtype = ctx.dtype

        def param_specs(self):
            return {self.name: ParamSpec((self.h, self.h), std=0.1)}

        def bind(self, tensors):
            self.w = tensors.pop(self.name)

        def memory_request(self):
            return StateRequest((self.h,), torch.float32)

        def forward(self, x, batch, mem, shared):
            u = K.linear(x, self.w).float()
            if batch.mode == "extend":                      # device only: works inside a captured graph
                idx = batch.seq_slot.long()
                st = mem.state.index_select(0, idx) * self.decay + u
                mem.state.index_copy_(0, idx, st)
                return st.to(self.dtype)
            out = torch.empty_like(u)
            o = 0
            for slot, n in zip(batch.host_slots, batch.host_new):
                st = mem.state[slot].clone()
                for t in range(n):
                    st = st * self.decay + u[o + t]
                    out[o + t] = st
                mem.state[slot] = st
                o += n
            return out.to(self.dtype)

    class RoutedFF(FeedForward):
        """Two experts; a router picks one per token (32-bit logits, lower index on ties)."""

        def __init__(self, ctx, prefix, inner):
            self.h, self.inner, self.p = ctx.hidden_size, inner, prefix

        def param_specs(self):
            s = {self.p + "router.weight": ParamSpec((2, self.h), std=0.5)}
            for e in range(2):
                s[f"{self.p}e{e}.up.weight"] = ParamSpec((self.inner, self.h), std=0.1)
                s[f"{self.p}e{e}.down.weight"] = ParamSpec((self.h, self.inner), std=0.1)
            return s

        def bind(self, tensors):
            self.t = {k: tensors.pop(k) for k in list(self.param_specs())}

        def forward(self, x, batch):
            logits = K.linear(x, self.t[self.p + "router.weight"], out_dtype=torch.float32)
            pick = (logits[:, 1] > logits[:, 0])
            ys = []
            for e in range(2):
                hmid = torch.relu(K.linear(x, self.t[f"{self.p}e{e}.up.weight"]).float()).to(x.dtype)
                ys.append(K.linear(hmid, self.t[f"{self.p}e{e}.down.weight"]))
            return torch.where(pick[:, None], ys[1], ys[0])

    class PairRotary(PositionEncoding):
        """Rotates neighbouring pairs (2i, 2i+1) instead of halves; no tables for the fused kernel."""

        def __init__(self, ctx, prefix, dim, theta):
            i = torch.arange(dim // 2, dtype=torch.float64)
            self.inv_freq = torch.pow(torch.tensor(theta, dtype=torch.float64), -2 * i / dim).to(ctx.device)

        def apply(self, q, k, tok_pos):
            ang = tok_pos.double()[:, None] * self.inv_freq[None, :]
            c, s = torch.cos(ang).float()[:, None, :], torch.sin(ang).float()[:, None, :]
            for t in (q, k):
                a, b = t[..., 0::2].float().clone(), t[..., 1::2].float().clone()
                t[..., 0::2] = (a * c - b * s).to(t.dtype)
                t[..., 1::2] = (b * c + a * s).to(t.dtype)

    for fam, kind, cls in (("mixer", "toy_decay", DecayMixer), ("feed_forward", "toy_routed", RoutedFF),
                           ("position", "toy_pair_rotary", PairRotary)):
        register_part(fam, kind, cls, replace=True)


def pair_rope_plain(x, theta):
    T, _, d = x.shape
    i = torch.arange(d // 2, dtype=torch.float64)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * torch.pow(torch.tensor(theta, dtype=torch.float64), -2 * i / d)
    c, s = torch.cos(ang).float().double()[:, None, :], torch.sin(ang).float().double()[:, None, :]
    out = x.clone()
    a, b = x[..., 0::2], x[..., 1::2]
    out[..., 0::2] = a * c - b * s
    out[..., 1::2] = b * c + a * s
    return out


def toy_spec(H=48, V=90):
    """Three layers: a decay mixer with a routed feed-forward, attention with the toy pair
    rotation, attention with the shipped rotation and a dense feed-forward."""
    from toyinfer_b200.parts import PartSpec
    from toyinfer_b200.parts.model import LayerSpec, ModelSpec
    norm = PartSpec("rmsnorm", {"size": H, "eps": 1e-5})
    att = lambda pos: PartSpec("gqa_attention", {"n_heads": 3, "n_kv_heads": 1, "head_dim": 16, "qk_norm_eps": 1e-5, "position": pos})
    blocks = [
        PartSpec("prenorm", {"norm": norm, "mixer": PartSpec("toy_decay", {"decay": 0.9}), "feed_forward": PartSpec("toy_routed", {"inner": 40})}),
        PartSpec("prenorm", {"norm": norm, "mixer": att("pairs"), "feed_forward": PartSpec("swiglu", {"intermediate_size": 56})}),
        PartSpec("prenorm", {"norm": norm, "mixer": att("halves"), "feed_forward": PartSpec("toy_routed", {"inner": 24})}),
    ]
    return ModelSpec(vocab_size=V, hidden_size=H, max_positions=256,
                     layers=[LayerSpec(f"model.layers.{i}.", b) for i, b in enumerate(blocks)], final_norm=norm,
                     positions={"pairs": PartSpec("toy_pair_rotary", {"dim": 16, "theta": 1e4}),
                                "halves": PartSpec("rotary_half", {"dim": 16, "theta": 1e4, "max_positions": 256})},
                     tie_head=True)


def toy_plain_forward(w, ids, H=48):
    """The same three layers from plain parts, float64, whole sequence."""
    eps = 1e-5
    h = plain.embedding(w["model.embed_tokens.weight"], ids)
    T = len(ids)

    def routed(x, p, inner):
        logits = (x @ w[p + "router.weight"].double().T).float()
        pick = logits[:, 1] > logits[:, 0]
        ys = [torch.relu(x @ w[f"{p}e{e}.up.weight"].double().T) @ w[f"{p}e{e}.down.weight"].double().T for e in range(2)]
        return torch.where(pick[:, None], ys[1], ys[0])

    # layer 0
    p = "model.layers.0."
    x = plain.rms_norm(h, w[p + "input_layernorm.weight"], eps)
    u = x @ w[p + "self_attn.w.weight"].double().T
    st, rows = torch.zeros(H, dtype=torch.float64), []
    for t in range(T):
        st = st * 0.9 + u[t]
        rows.append(st)
    h = h + torch.stack(rows)
    h = h + routed(plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), p + "mlp.", 40)
    # layers 1 and 2
    for layer, rope_fn in ((1, lambda t: pair_rope_plain(t, 1e4)), (2, None)):
        p = f"model.layers.{layer}."
        x = plain.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        a, _ = plain_attention_layer(x, w, p + "self_attn.", 3, 1, 16, eps, 1e4, 0, None, rope_fn=rope_fn)
        h = h + a
        x = plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        if layer == 1:
            m = plain.linear(plain.swiglu(plain.linear(x, w[p + "mlp.gate_proj.weight"]), plain.linear(x, w[p + "mlp.up_proj.weight"])),
                             w[p + "mlp.down_proj.weight"])
        else:
            m = routed(x, p + "mlp.", 24)
        h = h + m
    return plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("graph", [False, True])
def test_toy_parts_register_build_and_step(graph):
    """A mixer with a state, a routed feed-forward and another position encoding, all defined
    in this file: whole prompts, token by token, unequal batches, slots used again."""
    from toyinfer_b200.engine import Engine
    from toyinfer_b200.parts.model import DecoderModel
    make_toy_parts()
    model = DecoderModel(toy_spec(), torch.float32, DEV)
    w = bind_random(model, 7, torch.float32)
    reqs = model.memory_requests()
    assert type(reqs[0]).__name__ == "StateRequest" and type(reqs[1]).__name__ == "KVRequest"
    eng = Engine(model, max_tokens=64 * 6, max_batch=4, max_seq_len=256, use_cuda_graph=graph)
    g = torch.Generator().manual_seed(8)
    for round_ in range(3):
        lens, dec = [9, 30, 2], [5, 2, 7]
        seqs = [torch.randint(0, 90, (n + d,), generator=g).tolist() for n, d in zip(lens, dec)]
        want = [toy_plain_forward(w, s) for s in seqs]
        slots = [eng.new_sequence() for _ in seqs]
        logits = eng.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)], None).clone()
        for i, n in enumerate(lens):
            torch.testing.assert_close(logits[i].cpu().double(), want[i][n - 1], rtol=1e-4, atol=1e-5)
        live, t = [0, 1, 2], 0
        while live:
            logits = eng.step([(slots[i], [seqs[i][lens[i] + t]]) for i in live], None).clone()
            for row, i in enumerate(live):
                torch.testing.assert_close(logits[row].cpu().double(), want[i][lens[i] + t], rtol=1e-4, atol=1e-5)
            t += 1
            for i in [i for i in live if t >= dec[i]]:
                eng.end_sequence(slots[i])          # its state must not leak into the slot's next user
            live = [i for i in live if t < dec[i]]
    if graph:
        assert eng.graph_replays > 0
    # the toy mixer walks the host's lists when sequences start, and does not say captures_start:
    # this model's prompt steps stay plain launches
    assert eng.prompt_graph_tokens == 0 and not eng._prompt_graphs


def test_a_toy_part_that_says_so_is_captured_in_prompt_steps():
    """The routed toy feed-forward uses device tensors only; a subclass that says ``captures_start``
    beside the library's attention makes a model whose prompt shapes are captured when they come back."""
    from toyinfer_b200.engine import Engine
    from toyinfer_b200.parts import PartSpec, build_part, register_part
    from toyinfer_b200.parts.model import DecoderModel, LayerSpec, ModelSpec
    make_toy_parts()
    routed = type(build_part("feed_forward", PartSpec("toy_routed", {"inner": 8}), ctx_for(torch.float32, 48), "x."))
    register_part("feed_forward", "toy_routed_device_only", type("RoutedDeviceOnly", (routed,), {"captures_start": True}), replace=True)
    H, V, eps = 48, 90, 1e-5
    norm = PartSpec("rmsnorm", {"size": H, "eps": eps})
    block = PartSpec("prenorm", {"norm": norm, "feed_forward": PartSpec("toy_routed_device_only", {"inner": 24}),
                                 "mixer": PartSpec("gqa_attention", {"n_heads": 3, "n_kv_heads": 1, "head_dim": 16, "qk_norm_eps": eps,
                                                                     "position": "halves"})})
    spec = ModelSpec(vocab_size=V, hidden_size=H, max_positions=256, layers=[LayerSpec("model.layers.0.", block)], final_norm=norm,
                     positions={"halves": PartSpec("rotary_half", {"dim": 16, "theta": 1e4, "max_positions": 256})}, tie_head=True)
    model = DecoderModel(spec, torch.float32, DEV)
    w = bind_random(model, 17, torch.float32)
    eng = Engine(model, max_tokens=64 * 6, max_batch=4, max_seq_len=256)
    assert eng.prompt_graph_tokens > 0

    def plain_logits(ids):
        p = "model.layers.0."
        h = plain.embedding(w["model.embed_tokens.weight"], ids)
        a, _ = plain_attention_layer(plain.rms_norm(h, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.", 3, 1, 16, eps, 1e4, 0, None)
        h = h + a
        x = plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        pick = (x @ w[p + "mlp.router.weight"].double().T).float()
        ys = [torch.relu(x @ w[f"{p}mlp.e{e}.up.weight"].double().T) @ w[f"{p}mlp.e{e}.down.weight"].double().T for e in range(2)]
        h = h + torch.where((pick[:, 1] > pick[:, 0])[:, None], ys[1], ys[0])
        return plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])

    g = torch.Generator().manual_seed(28)
    for lens in ([20, 5], [9, 30], [31, 31], [2, 17]):          # one shape: two sequences, 64 token rows, at most 32 each
        seqs = [torch.randint(0, V, (n + 1,), generator=g).tolist() for n in lens]
        slots = [eng.new_sequence() for _ in seqs]
        first = eng.step([(sl, s[:-1]) for sl, s in zip(slots, seqs)], None).clone()
        second = eng.step([(sl, [s[-1]]) for sl, s in zip(slots, seqs)], None).clone()
        for i, s in enumerate(seqs):
            want = plain_logits(s)
            torch.testing.assert_close(first[i].cpu().double(), want[-2], rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(second[i].cpu().double(), want[-1], rtol=1e-4, atol=1e-5)
        for sl in slots:
            eng.end_sequence(sl)
    assert list(eng._prompt_graphs) == [(2, 64, 32)]


def test_toy_parts_in_pieces_and_beside_decoding_sequences():
    """The same toy model (a mixer with a state, a routed feed-forward, two position encodings) under the
    step function's general form: a prompt fed in pieces, and a prompt that starts while another sequence
    decodes.  Nothing in the toy parts knows about these cuts: the state mixer scans whatever tokens a
    step brings from the state its slot holds."""
    from toyinfer_b200.engine import Engine
    from toyinfer_b200.parts.model import DecoderModel
    make_toy_parts()
    model = DecoderModel(toy_spec(), torch.float32, DEV)
    w = bind_random(model, 7, torch.float32)
    eng = Engine(model, max_tokens=64 * 6, max_batch=4, max_seq_len=256)
    g = torch.Generator().manual_seed(18)
    a, b = (torch.randint(0, 90, (n,), generator=g).tolist() for n in (75, 40))
    wa, wb = toy_plain_forward(w, a), toy_plain_forward(w, b)
    sa = eng.new_sequence()
    got = [eng.step([(sa, a[lo:hi])], [list(range(hi - lo))]).clone() for lo, hi in ((0, 9), (9, 10), (10, 50))]
    torch.testing.assert_close(torch.cat(got).cpu().double(), wa[:50], rtol=1e-4, atol=1e-5)
    sb = eng.new_sequence()
    out = eng.step([(sa, [a[50]]), (sb, b[:30])], [[0], [0, 29]]).clone()          # b starts beside a
    torch.testing.assert_close(out.cpu().double(), torch.stack([wa[50], wb[0], wb[29]]), rtol=1e-4, atol=1e-5)
    out = eng.step([(sa, a[51:60]), (sb, [b[30]])], [[8], [0]]).clone()            # a goes on by nine, b by one
    torch.testing.assert_close(out.cpu().double(), torch.stack([wa[59], wb[30]]), rtol=1e-4, atol=1e-5)
    out = eng.step([(sa, [a[60]]), (sb, [b[31]])], None).clone()
    torch.testing.assert_close(out.cpu().double(), torch.stack([wa[60], wb[31]]), rtol=1e-4, atol=1e-5)


# ---------------------------------------------------------------------------
# the order of layers is data
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("window", [0, 40])
@pytest.mark.parametrize("dtype", DT)
def test_schedule_names_a_layer_twice_and_borrows_a_cache(dtype, window):
    """Layers A, B and C (C has no keys and values of its own).  Schedule: A, B, B again
    (same weights, a cache of its own), C reading the cache of the first B.  Whole prompts, single
    tokens, and then pieces of several tokens: with a window the first B's new keys must not reach its
    ring before C, which reads that ring, has run (the store waits in ``shared["deferred"]``)."""
    from toyinfer_b200.engine import Engine
    from toyinfer_b200.parts import PartSpec
    from toyinfer_b200.parts.model import DecoderModel, LayerSpec, ModelSpec, ScheduleEntry
    H, nh, nkv, hd, eps, theta, V = 64, 4, 2, 16, 1e-6, 1e4, 100
    norm = PartSpec("rmsnorm", {"size": H, "eps": eps})
    ffn = PartSpec("swiglu", {"intermediate_size": 72})
    att = lambda own: PartSpec("gqa_attention", {"n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "qk_norm_eps": eps,
                                                 "position": "rope", "own_kv": own, "window": window})
    layers = [LayerSpec(f"model.layers.{i}.", PartSpec("prenorm", {"norm": norm, "mixer": att(i < 2), "feed_forward": ffn}))
              for i in range(3)]
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(2, memory_of=1)]
    spec = ModelSpec(vocab_size=V, hidden_size=H, max_positions=128, layers=layers, final_norm=norm, schedule=schedule,
                     positions={"rope": PartSpec("rotary_half", {"dim": hd, "theta": theta, "max_positions": 128})},
                     tie_head=False)
    model = DecoderModel(spec, dtype, DEV)
    w = bind_random(model, 9, dtype)
    assert "model.layers.2.self_attn.k_proj.weight" not in w
    eng = Engine(model, max_tokens=64 * 4, max_batch=2, max_seq_len=128)
    assert len(eng.cache.kv_groups) == 1 and eng.cache.kv_groups[0].entries == [0, 1, 2]
    r = rmode(dtype)

    def plain_forward(ids):
        h = plain.rnd(plain.embedding(w["model.embed_tokens.weight"], ids), r)
        kept = {}
        for e, ent in enumerate(schedule):
            p = f"model.layers.{ent.layer}."
            x = plain.rms_norm(h, w[p + "input_layernorm.weight"], eps, r)
            if ent.memory_of is None:
                a, kept[e] = plain_attention_layer(x, w, p + "self_attn.", nh, nkv, hd, eps, theta, window, r)
            else:
                T = x.shape[0]
                q = plain.linear(x, w[p + "self_attn.q_proj.weight"], r).view(T, nh, hd)
                q = plain.rope(plain.rms_norm(q, w[p + "self_attn.q_norm.weight"], eps, r), plain.rope_angles(hd, theta, range(T)), r)
                k, v = kept[ent.memory_of]
                a = plain.linear(plain.attention(q, k, v, 1 / math.sqrt(hd), window, r).reshape(T, nh * hd), w[p + "self_attn.o_proj.weight"], r)
            h = plain.rnd(h + a, r)
            x = plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps, r)
            m = plain.linear(plain.swiglu(plain.linear(x, w[p + "mlp.gate_proj.weight"], r), plain.linear(x, w[p + "mlp.up_proj.weight"], r), r),
                             w[p + "mlp.down_proj.weight"], r)
            h = plain.rnd(h + m, r)
        return plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps, r), w["lm_head.weight"])

    from helpers import assert_logits_close
    name = "float32" if dtype == torch.float32 else "bfloat16"
    g = torch.Generator().manual_seed(10)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (100, 120)]
    want = [plain_forward(s) for s in seqs]
    slots = [eng.new_sequence() for _ in seqs]
    heads = [30, 70]
    logits = eng.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, heads)], [list(range(n)) for n in heads])
    assert_logits_close(logits, torch.cat([want[0][:30], want[1][:70]]), name, "schedule, whole")
    for t in range(5):
        logits = eng.step([(slots[i], [seqs[i][heads[i] + t]]) for i in range(2)], None).clone()
        assert_logits_close(logits, torch.stack([want[i][heads[i] + t] for i in range(2)]), name, f"schedule, step {t}")
    # pieces: the first sequence goes on by 50 tokens at once (more than the ring has slack), the second by one
    at = [heads[0] + 5, heads[1] + 5]
    logits = eng.step([(slots[0], seqs[0][at[0]:at[0] + 50]), (slots[1], [seqs[1][at[1]]])], [[0, 24, 49], [0]]).clone()
    assert_logits_close(logits, torch.stack([want[0][at[0]], want[0][at[0] + 24], want[0][at[0] + 49], want[1][at[1]]]), name,
                        "schedule, pieces")
    logits = eng.step([(slots[0], [seqs[0][at[0] + 50]]), (slots[1], seqs[1][at[1] + 1:at[1] + 4])], [[0], [2]]).clone()
    assert_logits_close(logits, torch.stack([want[0][at[0] + 50], want[1][at[1] + 3]]), name, "schedule, after the pieces")


def test_unknown_part_and_bad_schedule_are_refused():
    from toyinfer_b200.parts import PartSpec
    from toyinfer_b200.parts.model import DecoderModel, LayerSpec, ModelSpec, ScheduleEntry
    norm = PartSpec("rmsnorm", {"size": 32, "eps": 1e-5})
    blk = PartSpec("prenorm", {"norm": norm, "mixer": PartSpec("no_such_mixer", {}), "feed_forward": PartSpec("swiglu", {"intermediate_size": 8})})
    with pytest.raises(ValueError) as e:
        DecoderModel(ModelSpec(10, 32, 64, [LayerSpec("l.", blk)], norm), torch.float32, DEV)
    assert "no_such_mixer" in str(e.value) and "gqa_attention" in str(e.value)
    ok = PartSpec("prenorm", {"norm": norm, "mixer": PartSpec("gqa_attention", {"n_heads": 2, "n_kv_heads": 1, "head_dim": 16}),
                              "feed_forward": PartSpec("swiglu", {"intermediate_size": 8})})
    with pytest.raises(ValueError):
        DecoderModel(ModelSpec(10, 32, 64, [LayerSpec("l.", ok)], norm, schedule=[ScheduleEntry(0, memory_of=0)]), torch.float32, DEV)
    with pytest.raises(ValueError):
        DecoderModel(ModelSpec(10, 32, 64, [LayerSpec("l.", ok)], norm, schedule=[ScheduleEntry(3)]), torch.float32, DEV)


def test_a_whole_toy_architecture_registered_from_here(tmp_path):
    """An architecture of its own, added without touching the library: a configuration class with
    its own keys, a description that arranges the toy parts above, registered under a name; then
    the library's own paths carry it: a model folder with random weights, the loader, the entry
    point's greedy generation, against the plain toy forward."""
    from toyinfer_b200 import LLM, SamplingParams
    from toyinfer_b200.config import register_architecture, unregister_architecture
    from toyinfer_b200.config.base import Key, ModelConfig
    from toyinfer_b200.weights import write_model_folder
    make_toy_parts()

    class ToyConfig(ModelConfig):
        KEYS = {"architectures": Key("str_list"), "width": Key("int"), "words": Key("int"),
                "stop_word": Key("int", required=False, default=None, nullable=True)}

        def validate(self):
            return [] if self.width % 16 == 0 else [f"width: {self.width} is not a multiple of 16"]

    def describe(cfg):
        spec = toy_spec(H=cfg.width, V=cfg.words)
        if cfg.stop_word is not None:
            spec.stop_token_ids = (cfg.stop_word,)
        return spec

    register_architecture("ToyForCausalLM", ToyConfig, describe)
    try:
        folder = write_model_folder({"architectures": ["ToyForCausalLM"], "width": 48, "words": 90}, 5, str(tmp_path),
                                    store_dtype=torch.float32)
        llm = LLM(folder, dtype="float32", max_seq_len=128, max_batch=2, max_tokens=512)
        prompts = [[3, 14, 15, 9, 26], [5, 3], [58, 9, 7, 9, 3, 2, 38, 46]]
        got = [r.tokens for r in llm.generate(prompts, SamplingParams(temperature=0.0), max_new_tokens=6)]
        w = {k: v.double() for k, v in plain.read_weights(folder).items()}
        for p, g in zip(prompts, got):
            ids = list(p)
            for _ in range(6):
                ids.append(int(torch.argmax(toy_plain_forward(w, ids)[-1])))
            assert g == ids[len(p):]
        with pytest.raises(Exception, match="width"):
            write_model_folder({"architectures": ["ToyForCausalLM"], "width": 50, "words": 90}, 5, str(tmp_path / "bad"))
    finally:
        unregister_architecture("ToyForCausalLM")
