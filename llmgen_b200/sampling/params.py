"""Per-request sampling parameters (src/runner/batching.zig:6-10)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 1.0    # <= 0: greedy (argmax, ties to the smaller id)
    max_tokens: int = 64        # completion tokens to generate at most
    ignore_eos: bool = False    # keep generating past the end-of-sequence token
