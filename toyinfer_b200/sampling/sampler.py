"""Picks next tokens from logits on the device.

Greedy is the argmax with the lowest index on ties (src/sampler.cpp:71-81).  Otherwise
temperature, top-k and top-p as the reference orders them (src/sampler.cpp:24-68), with
two differences: the temperature divides the logits once (the reference divides a
second time inside the exponent, :38), and the uniform number is a function of
(seed, sequence key, number of tokens the sequence has drawn), not of the clock (:57-60),
so a sequence gets the same tokens whatever batch it runs in.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .. import kernels as K
from .params import SamplingParams


class Sampler:
    def __init__(self, params: SamplingParams, device):
        params.check()
        self.params = params
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, keys: Sequence[int], steps: Sequence[int]) -> torch.Tensor:
        """logits float32 [rows, vocab]; keys and steps name each row's sequence and how
        many tokens it has drawn.  Returns int32 [rows] on the device."""
        p = self.params
        if p.greedy:
            return K.argmax(logits)
        keys_t = torch.tensor(list(keys), dtype=torch.int64, device=self.device)
        steps_t = torch.tensor(list(steps), dtype=torch.int32, device=self.device)
        vocab = logits.shape[1]
        top_k = p.top_k if 0 < p.top_k < vocab else 0
        return K.sample(logits, p.temperature, top_k, p.top_p, p.seed, keys_t, steps_t)
