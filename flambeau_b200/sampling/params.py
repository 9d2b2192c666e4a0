"""Sampling parameters of one request, with the reference's names and meanings
(crates/runtime/src/sampling.rs:39-108; crates/server/src/state.rs:133-243)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 0.0              # <= 0: greedy (argmax, lowest index wins a tie)
    top_p: Optional[float] = None         # used when in (0, 1)
    top_k: Optional[int] = None           # used when > 0
    min_p: Optional[float] = None         # used when > 0
    repetition_penalty: float = 1.0       # 1.0 = off; divides positive, multiplies negative logits of seen tokens
    presence_penalty: float = 0.0         # subtracted once from every seen token
    frequency_penalty: float = 0.0        # subtracted count times
    logit_bias: Optional[dict] = None     # token id -> additive bias
    seed: int = 0
    max_tokens: int = 64                  # new tokens to generate
    stop_token_ids: tuple = ()            # generation ends after one of these is produced
    ignore_eos: bool = False

    def __post_init__(self):
        if self.top_p is not None and not 0.0 < self.top_p < 1.0:
            self.top_p = None
        if self.top_k is not None and self.top_k <= 0:
            self.top_k = None
        if self.min_p is not None and self.min_p <= 0.0:
            self.min_p = None
        if self.max_tokens < 0:
            raise ValueError("max_tokens must not be negative")
        self.stop_token_ids = tuple(self.stop_token_ids or ())

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0

    @classmethod
    def greedy(cls, **kw) -> "SamplingParams":
        return cls(temperature=0.0, **kw)


_MASK = (1 << 64) - 1


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform_for(seed: int, draw: int) -> float:
    """The uniform number in [0, 1) of a request's `draw`-th sampled token.  It depends on the request's seed
    and the count of its own draws only, so a request samples the same tokens whatever shares its batches.
    24 random bits, as the reference's generator yields (crates/runtime/src/sampling.rs:145-148)."""
    return (splitmix64(splitmix64(seed & _MASK) ^ (draw & _MASK)) >> 40) * (1.0 / (1 << 24))
