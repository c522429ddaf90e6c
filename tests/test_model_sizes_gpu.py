"""Real Qwen3 layer sizes with random weights: two layers of the 4B shape (hidden 2560, 32
heads over 8 kv heads of 128, intermediate 9728, vocabulary 151936).  At this size the plain
implementation is too slow for a test, so the bfloat16 engine (tcgen05 matrix products and
attention, TMA, CUDA graph) is compared with the library's own float32 engine (CUDA-core
kernels only), which the other tests tie to the plain implementation at small sizes.  Both get
the same bfloat16-valued weights."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 2560,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728,
    "vocab_size": 151936, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "max_position_embeddings": 40960,
    "tie_word_embeddings": True,
}


# one layer of the 32B shape: 64 heads over 8 kv heads (8 query heads per kv head), untied head
CFG_32B = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 5120,
    "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 25600,
    "vocab_size": 32000, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "max_position_embeddings": 40960,
    "tie_word_embeddings": False,
}


def _engines(cfg):
    from toyinfer_b200 import models  # noqa: F401
    from toyinfer_b200.config import Qwen3Config, resolve_architecture
    from toyinfer_b200.engine import Engine
    from toyinfer_b200.parts.model import DecoderModel
    from toyinfer_b200.weights import random_parameters
    arch = resolve_architecture("Qwen3ForCausalLM")
    spec = arch.describe(Qwen3Config.from_dict(dict(cfg)))
    out = {}
    ref = None
    for dt in (torch.bfloat16, torch.float32):
        model = DecoderModel(spec, dt, "cuda")
        if ref is None:
            ref = random_parameters(model.param_specs(), 123, torch.bfloat16, "cuda")
        model.bind({k: v.to(dt) if v.dtype != torch.int32 else v for k, v in ref.items()})
        out[dt] = Engine(model, max_tokens=64 * 64, max_batch=4, max_seq_len=2048)
    return out


def _close(bf, fp, what):
    bf, fp = bf.float().cpu(), fp.float().cpu()
    assert torch.isfinite(bf).all(), what
    scale = fp.abs().amax(dim=-1, keepdim=True)
    bad = (bf - fp).abs() > 0.03 * scale + 0.03 * fp.abs()
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} logits off, worst {(bf - fp).abs().max():.4g} vs scale {scale.max():.4g}"
    # the two engines agree on what matters for a greedy step unless the top two are within rounding
    top = fp.argmax(-1)
    picked = bf.argmax(-1)
    for i in range(fp.shape[0]):
        assert fp[i, picked[i]] >= fp[i, top[i]] - 0.03 * scale[i, 0], what


@pytest.mark.parametrize("cfg", [CFG, CFG_32B], ids=["4B-shape", "32B-shape"])
def test_prompts_then_decoding_agree_between_the_engines(cfg):
    import toyinfer_b200.kernels as K
    engines = _engines(cfg)
    g = torch.Generator().manual_seed(5)
    lens, dec = [700, 129, 1], 6
    seqs = [torch.randint(0, cfg["vocab_size"], (n + dec,), generator=g).tolist() for n in lens]
    results = {}
    for dt, eng in engines.items():
        slots = [eng.new_sequence() for _ in seqs]
        rows = [eng.step([(s, q[:n]) for s, q, n in zip(slots, seqs, lens)], [[n - 1, n // 2] for n in lens]).clone()]
        for t in range(dec):
            rows.append(eng.step([(s, [q[n + t]]) for s, q, n in zip(slots, seqs, lens)], None).clone())
        for s in slots:
            eng.end_sequence(s)
        K.check_status()
        results[dt] = torch.cat(rows)
    _close(results[torch.bfloat16], results[torch.float32], "real layer sizes")
    assert engines[torch.bfloat16].graph_replays > 0
