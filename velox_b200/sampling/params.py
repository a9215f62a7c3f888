"""What a request asks of the sampler.

Names, defaults and limits are the reference's ``SamplingParams`` (engine/utils.py of that
project), which is part of the Python entry point; the way they are checked (one table of
ranges) and the derived questions the sampler asks (greedy? any penalty? any filter?) are
this engine's.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

# option -> (lowest allowed, lowest is allowed itself, highest allowed or None), for the
# options that are numbers with a range
_RANGES = {
    "temperature": (0.0, True, None),          # 0 is greedy; else logits / max(temperature, 1e-5)
    "top_p": (0.0, False, 1.0),                # smallest most-probable set reaching this mass; 1 keeps all
    "top_k": (0, True, None),                  # the k most probable tokens; 0 keeps all
    "repetition_penalty": (0.0, False, None),  # > 1 makes seen tokens less likely
    "max_tokens": (1, True, None),
}


@dataclass
class SamplingParams:
    n: int = 1  # one continuation per request; nothing else is supported
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0   # subtracted once from every token seen so far
    frequency_penalty: float = 0.0  # subtracted once per occurrence
    ignore_eos: bool = False        # end-of-sequence and stop tokens do not end the request
    max_tokens: int = 512
    # With a seed the draws depend on (seed, index of the output token) only, whatever else is
    # in the batch; without one the engine derives a seed from its own and the request's name.
    seed: Optional[int] = None
    stop_token_ids: List[int] = field(default_factory=list)

    def __post_init__(self) -> None:
        if self.n != 1:
            raise ValueError(f"n={self.n}: only n=1 is supported")
        for name, (low, low_ok, high) in _RANGES.items():
            value = getattr(self, name)
            above = value >= low if low_ok else value > low
            if not above or (high is not None and value > high):
                span = f"{'[' if low_ok else '('}{low}, {'inf)' if high is None else str(high) + ']'}"
                raise ValueError(f"{name} must be in {span}, got {value}")

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def has_penalties(self) -> bool:
        neutral = (self.repetition_penalty == 1.0, self.presence_penalty == 0.0, self.frequency_penalty == 0.0)
        return not all(neutral)

    @property
    def filters_candidates(self) -> bool:
        """Whether top-k or top-p leaves anything out."""
        return self.top_k > 0 or self.top_p < 1.0
