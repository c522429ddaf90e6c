"""Picks next tokens from logits on the device.

Greedy is the argmax with the lowest index on ties (src/sampler.cpp:71-81).  Otherwise
temperature, top-k and top-p as the reference orders them (src/sampler.cpp:24-68), with
two differences: the temperature divides the logits once (the reference divides a
second time inside the exponent, :38), and the uniform number is a function of
(seed, sequence key, number of tokens the sequence has drawn), not of the clock (:57-60),
so a sequence gets the same tokens whatever batch it runs in.  Every combination of top_k
and top_p runs on the device: top_k up to 1,024, temperature alone, and top_p whose nucleus
lies within the row's 64 largest entries as two short kernels over many blocks; more
candidates (or a larger nucleus) tier by tier in one block per row (csrc/sampling.cu).
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
        self._cap = 0
        self._pending = False

    def _upload(self, keys: Sequence[int], steps: Sequence[int]):
        """The rows' keys and step counts on the device, through pinned memory and without
        waiting for the device: the host may run ahead of the step whose logits these go with."""
        n = len(keys)
        if self.device.type != "cuda":
            return (torch.tensor(list(keys), dtype=torch.int64, device=self.device),
                    torch.tensor(list(steps), dtype=torch.int32, device=self.device))
        if n > self._cap:
            if self._pending:
                self._copied.synchronize()
                self._pending = False
            self._cap = max(64, 2 * n)
            self._host = torch.zeros(3 * self._cap, dtype=torch.int32, pin_memory=True)   # keys (as int64), then steps
            self._dev = torch.zeros(3 * self._cap, dtype=torch.int32, device=self.device)
            self._copied = torch.cuda.Event()
        if self._pending:              # the host buffer may be rewritten once its last copy has left it
            self._copied.synchronize()
        cap = self._cap
        host_keys = self._host[:2 * cap].view(torch.int64).numpy()
        host_steps = self._host[2 * cap:].numpy()
        host_keys[:n] = list(keys)
        host_steps[:n] = list(steps)
        self._dev.copy_(self._host, non_blocking=True)
        self._copied.record()
        self._pending = True
        return self._dev[:2 * cap].view(torch.int64)[:n], self._dev[2 * cap:][:n]

    def sample(self, logits: torch.Tensor, keys: Sequence[int], steps: Sequence[int]) -> torch.Tensor:
        """logits float32 [rows, vocab]; keys and steps name each row's sequence and how
        many tokens it has drawn.  Returns int32 [rows] on the device."""
        p = self.params
        if p.greedy:
            return K.argmax(logits)
        keys_t, steps_t = self._upload(keys, steps)
        vocab = logits.shape[1]
        top_k = p.top_k if 0 < p.top_k < vocab else 0
        return K.sample(logits, p.temperature, top_k, p.top_p, p.seed, keys_t, steps_t)
