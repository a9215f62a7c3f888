"""Per-request sampling options, with the reference's names, defaults and checks
(engine/utils.py:9-35)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class SamplingParams:
    n: int = 1
    # 0 means greedy (argmax); otherwise logits are divided by max(temperature, 1e-5).
    temperature: float = 1.0
    # Smallest set of most probable tokens whose probability reaches top_p; 1 keeps all.
    top_p: float = 1.0
    # Keep only the k most probable tokens; 0 disables the filter.
    top_k: int = 0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    ignore_eos: bool = False
    max_tokens: int = 512
    # With a seed, a request's draws depend on (seed, index of the output token) only.
    seed: Optional[int] = None
    stop_token_ids: List[int] = field(default_factory=list)

    def __post_init__(self) -> None:
        if self.n != 1:
            raise ValueError("only n=1 is supported")
        if self.temperature < 0.0:
            raise ValueError("temperature must be non-negative")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be non-negative (0 disables the filter)")
        if self.repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be positive")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def has_penalties(self) -> bool:
        return (
            self.repetition_penalty != 1.0
            or self.presence_penalty != 0.0
            or self.frequency_penalty != 0.0
        )

    @property
    def filters_candidates(self) -> bool:
        return self.top_k > 0 or self.top_p < 1.0
