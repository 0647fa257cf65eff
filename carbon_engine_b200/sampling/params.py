"""Sampling options of a request, with the reference's names, defaults and meanings
(src/sampling.rs:10-45)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class SamplingParams:
    temperature: float = 0.0          # <= 0: greedy
    top_k: int = -1                   # <= 0: off; 1: greedy
    top_p: float = 1.0
    min_p: float = 0.0
    max_tokens: int = 1024
    ignore_eos: bool = False
    stop_token_ids: List[int] = field(default_factory=list)
    seed: Optional[int] = None        # None: drawn from the system's entropy
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    logprobs: int = 0                 # report this many most likely alternatives per output token

    def is_greedy(self) -> bool:
        """src/sampling.rs:48-50"""
        return self.temperature <= 0.0 or self.top_k == 1

    def has_penalties(self) -> bool:
        """src/sampling.rs:52-56"""
        return self.presence_penalty != 0.0 or self.frequency_penalty != 0.0 or self.repetition_penalty != 1.0
