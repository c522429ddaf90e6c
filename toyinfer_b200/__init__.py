"""toyinfer_b200: a small model library with generation of its own for one B200.

Everything between a request's token ids and its next token for the Qwen3 dense
decoder: typed configuration and registry (config/), safetensors by name and random
weights (weights/), model parts (parts/) described per architecture (models/), a paged
cache with slots (cache/), one step function, a generation loop and entry points
(engine/), sampling (sampling/), and hand-written CUDA kernels for sm_100a (csrc/,
kernels/).
"""
from . import models  # noqa: F401  (registers the architectures)
from .engine import LLM, Engine, GenerationResult
from .sampling import GREEDY, SamplingParams

__all__ = ["LLM", "Engine", "GenerationResult", "GREEDY", "SamplingParams"]
__version__ = "0.1.0"
