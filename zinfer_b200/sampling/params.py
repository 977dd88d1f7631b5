"""Sampling options of one request: the reference's ``SamplingConfig`` with its
names, defaults and meanings (src/sampling/sampler.zig:8-16), plus what ends a
request."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0          # <= 0, or top_k == 1: greedy (sampler.zig:31-33)
    top_k: int = 0                    # 0 keeps every token
    top_p: float = 1.0
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: int = 0
    max_new_tokens: int = 64          # the reference's default for `generate` (src/app/cli/args.zig:100)
    eos_token_ids: Optional[Sequence[int]] = None   # None: the model family's own
    # Sequences of token ids that end the response when the generated ids end with one of them; the
    # sequence itself is not part of the response (the reference's --stop strings, args.zig:462-466,
    # streaming.zig:11-40, on ids).
    stop_sequences: Optional[Sequence[Sequence[int]]] = None
    ignore_eos: bool = False

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    @property
    def has_penalties(self) -> bool:
        return (self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
                or (self.repetition_penalty > 0.0 and self.repetition_penalty != 1.0))

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be >= 0")
        if not 0 <= self.seed < 2 ** 63:
            raise ValueError("seed must fit in 63 bits")
