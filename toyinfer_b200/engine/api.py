"""The Python entry point: a model folder (or a configuration with random weights)
in, generated token ids out.

    llm = LLM("path/to/model", dtype="bfloat16", max_seq_len=8192)
    results = llm.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.0), max_new_tokens=16)

Prompts are token ids: the reference's tokenizer and chat template
(src/tokenizer.cpp) are not part of this library.  Option names follow the
reference's command line (src/options.cpp:7-45) where it has them.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..sampling import GREEDY, Sampler, SamplingParams
from .engine import Engine, parse_dtype
from .generate import GenerationLoop, GenerationResult, GenerationStats


class _Stepper:
    """What the generation loop drives: the engine's steps plus a sampler."""

    def __init__(self, engine: Engine, sampler: Sampler):
        self.engine, self.sampler = engine, sampler
        self._side = None
        self._host = None

    def new_sequence(self) -> int:
        return self.engine.new_sequence()

    def end_sequence(self, slot: int) -> None:
        self.engine.end_sequence(slot)

    def step(self, entries, want):
        return self.engine.step(entries, want)

    def sample(self, logits, keys, steps) -> List[int]:
        with self.engine.tracer.range("sample"):
            return self.sampler.sample(logits, keys, steps).tolist()   # device -> host, waits for the step

    # -- the next step started from tokens that are still on the device ---------------------
    def draw(self, logits, keys, steps):
        """Draws on the device; the handle is read later, beside whatever was started since."""
        with self.engine.tracer.range("sample"):
            ids = self.sampler.sample(logits, keys, steps)
        if ids.device.type != "cuda":
            return ids, None
        drawn = torch.cuda.Event()
        drawn.record()
        return ids, drawn

    def step_from(self, slots, handle):
        return self.engine.step([(s, None) for s in slots], [[0] for _ in slots], token_source=handle[0])

    def read(self, handle) -> List[int]:
        ids, drawn = handle
        if drawn is None:
            return ids.tolist()
        # on a stream of its own, after the draw only: the step started meanwhile is not waited for
        if self._side is None:
            self._side = torch.cuda.Stream(device=ids.device)
            self._host = torch.empty(self.engine.max_batch, dtype=torch.int32, pin_memory=True)
        n = ids.shape[0]
        with torch.cuda.stream(self._side):
            self._side.wait_event(drawn)
            self._host[:n].copy_(ids, non_blocking=True)
        self._side.synchronize()
        return self._host[:n].tolist()

    def rows(self, logits, indices):
        return logits[torch.tensor(indices, dtype=torch.long, device=logits.device)]


def default_max_tokens(engine_kw: dict, model, max_batch: int, max_seq_len: int) -> int:
    """Cache capacity when the caller gives none: what max_batch full sequences need,
    limited to 60 % of the device memory that is free once the weights are loaded."""
    from ..cache import PAGE, bytes_per_token
    want = max_batch * ((max_seq_len + PAGE - 1) // PAGE * PAGE)
    per_token = bytes_per_token(model.memory_requests(), model.dtype)
    if model.device.type == "cuda" and per_token:
        free, _ = torch.cuda.mem_get_info(model.device)
        want = min(want, max(PAGE, int(free * 0.6) // per_token))
    return max(PAGE, want // PAGE * PAGE)


class LLM:
    def __init__(self, model_dir: Optional[str] = None, *, config: Optional[dict] = None, seed: int = 0,
                 dtype="bfloat16", max_seq_len: Optional[int] = None, max_batch: int = 64,
                 max_tokens: Optional[int] = None, enable_cuda_graph: bool = True,
                 use_dedicated_prefill: bool = True, prefill_chunk: Optional[int] = None,
                 detail_time: bool = False, nvtx: bool = True, device="cuda"):
        """``detail_time``: CUDA events around every step and, where steps run as plain launches
        (prompts always; single-token steps with ``enable_cuda_graph=False``), around the stages of
        every layer; ``timing_report()`` returns their sums.  ``nvtx``: NVTX ranges with the same
        names, for a profiler's timeline.  ``prefill_chunk``: the most prompt tokens one step takes
        (prompts are then fed in pieces, so a step's activations stay bounded; None: whole prompts)."""
        if (model_dir is None) == (config is None):
            raise ValueError("give either model_dir or config (random weights)")
        from .. import models  # noqa: F401
        from ..config.registry import architecture_of, load_config
        from ..parts.model import DecoderModel
        from ..weights import load_parameters, random_parameters
        dt = parse_dtype(dtype)
        if model_dir is not None:
            arch, cfg = load_config(model_dir)
        else:
            arch = architecture_of(config)
            cfg = arch.config_cls.from_dict(config)
        model = DecoderModel(arch.describe(cfg), dt, device)
        if model_dir is not None:
            model.bind(load_parameters(model.param_specs(), model_dir, dt, model.device,
                                       ignorable=model.ignorable_names()))
        else:
            model.bind(random_parameters(model.param_specs(), seed, dt, model.device))
        limit = model.spec.max_positions
        msl = int(min(max_seq_len or limit, limit))
        if max_tokens is None:
            max_tokens = default_max_tokens({}, model, max_batch, msl)
        from ..tracing import Tracer
        self.engine = Engine(model, max_tokens=max_tokens, max_batch=max_batch, max_seq_len=msl,
                             use_cuda_graph=enable_cuda_graph,
                             tracer=Tracer(nvtx=nvtx and model.device.type == "cuda", timing=detail_time))
        self.config = cfg
        self._stepper = _Stepper(self.engine, None)
        self.use_dedicated_prefill = use_dedicated_prefill
        self.prefill_chunk = prefill_chunk
        self.last_stats: Optional[GenerationStats] = None

    def timing_report(self):
        """name -> (count, total device milliseconds) of the ranges timed since the last reset
        (empty without ``detail_time``): ``prefill_step``, ``prefill.layer.attn_block``,
        ``prefill.layer.mlp_block``, ``prefill.mixer.qkv`` ..., ``decode_step``, ``sample``."""
        return self.engine.tracer.report()

    @property
    def stop_token_ids(self):
        return tuple(self.engine.spec.stop_token_ids)

    def generate(self, prompts: Sequence[Sequence[int]], sampling: Optional[SamplingParams] = None,
                 max_new_tokens: int = 16, stop_token_ids: Optional[Sequence[int]] = None,
                 ignore_eos: bool = False) -> List[GenerationResult]:
        sampling = sampling or SamplingParams()
        stops = set(self.stop_token_ids)
        stops.update(stop_token_ids or ())
        e = self.engine
        self._stepper.sampler = Sampler(sampling, e.device)
        loop = GenerationLoop(self._stepper, stops, e.max_batch, e.max_seq_len,
                              e.cache.max_tokens, ignore_eos=ignore_eos,
                              dedicated_prefill=self.use_dedicated_prefill, prefill_chunk=self.prefill_chunk)
        out = loop.run(prompts, max_new_tokens)
        self.last_stats = loop.stats
        if e.device.type == "cuda":
            from .. import kernels as K
            K.check_status()     # raises if a kernel gave up on a bounded wait: its tokens are not to be trusted
        return out
