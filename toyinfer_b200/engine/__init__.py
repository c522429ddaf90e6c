"""Step function, generation loop, entry points."""
from .api import LLM
from .batch import BatchBuffers, StepBatch, fill_batch
from .engine import Engine, StepError, parse_dtype
from .generate import GenerationLoop, GenerationResult, GenerationStats, plan_batches

__all__ = ["LLM", "BatchBuffers", "StepBatch", "fill_batch", "Engine", "StepError", "parse_dtype",
           "GenerationLoop", "GenerationResult", "GenerationStats", "plan_batches"]
