"""Token selection: greedy, or temperature with optional top-k and top-p, with the
reference's options, defaults and rules (src/sampler.c, src/main.c:98-102,160-170,212-214):
temperature 0 is greedy; ties go to the lowest id; top-k 40 (0 = all), top-p 0.95 and seed 1
by default; a non-zero 32-bit seed; banned ids are never chosen. All of it runs on the GPU;
every sequence has its own xorshift32 state, so what a sequence draws does not depend on
what else is in the batch."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Optional, Sequence

import torch


@dataclass(frozen=True)
class SamplingOptions:
    temperature: float = 0.0
    top_k: int = 40
    top_p: float = 0.95
    seed: int = 1

    def validate(self) -> "SamplingOptions":
        t = self.temperature
        if t < 0 or t > 100 or (0 < t < 1e-6):
            raise ValueError("temperature must be 0 or in [1e-6, 100]")  # src/main.c:168
        if not 0 < self.top_p <= 1:
            raise ValueError("top-p must be in (0, 1]")  # src/main.c:163
        if self.top_k < 0:
            raise ValueError("top-k must not be negative")
        if not 0 < self.seed <= 0xFFFFFFFF:
            raise ValueError("seed must be nonzero")  # src/sampler.c:9
        return self


def sequence_seed(seed: int, index: int) -> int:
    """The xorshift32 state request ``index`` starts from: request 0 uses ``seed`` itself."""
    s = (seed + index) & 0xFFFFFFFF
    return s if s else 1


class Sampler:
    def __init__(self, ops, vocab_size: int, options: SamplingOptions, device: torch.device,
                 banned_token_ids: Iterable[int] = ()):
        self.ops = ops
        self.options = options.validate()
        self.vocab_size = vocab_size
        self.device = device
        banned = sorted(set(int(b) for b in banned_token_ids))
        self.banned: Optional[torch.Tensor] = None
        if banned:
            if banned[0] < 0 or banned[-1] >= vocab_size:
                raise ValueError("a banned token id is outside the vocabulary")
            mask = torch.zeros(vocab_size, dtype=torch.uint8)
            mask[torch.tensor(banned, dtype=torch.long)] = 1
            self.banned = mask.to(device)

    def new_states(self, request_indices: Sequence[int]) -> torch.Tensor:
        seeds = [sequence_seed(self.options.seed, i) for i in request_indices]
        # the kernel reads the words as unsigned; int32 is only the container
        return torch.tensor(seeds, dtype=torch.int64).to(torch.int32).to(self.device)

    def choose(self, logits: torch.Tensor, states: torch.Tensor) -> torch.Tensor:
        """``logits`` float32 [B, vocab]; returns int32 [B] on the device and advances the states
        (a greedy choice draws nothing). -1 marks a row whose every id is banned."""
        if self.options.temperature == 0:
            return self.ops.argmax(logits, self.banned)
        return self.ops.sample(logits, states, self.options.temperature, self.options.top_k, self.options.top_p,
                               self.banned)

    @staticmethod
    def select(values: torch.Tensor, keep: Sequence[int]) -> torch.Tensor:
        """The rows of the sequences that go on (tokens or states) when others have ended."""
        return values[torch.tensor(list(keep), dtype=torch.long, device=values.device)].contiguous()
