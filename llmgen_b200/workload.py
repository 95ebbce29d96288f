"""Workloads for the `bench` command: seeded random requests in the reference's JSON format.

    {"name": ..., "rounds": [[{"prompt_ids": [...], "max_tokens": n, "temperature": t,
                               "ignore_eos": true}, ...], ...]}

The rounds of a workload run one after another and the requests of a round are submitted
together (src/bench/workload.zig:6-16).  The reference ships a script that writes five fixed
scenarios (bench/gen_workload.py:1-17); here a workload is a `Shape`: how many requests and
rounds, a range of prompt lengths and a range of output lengths.  The reference's scenarios are
entries of `SCENARIOS`, and every number of a scenario can be overridden.

What is kept from the reference's generator:
  * every round has prompts of its own (an engine that remembers prefixes would otherwise do
    less work in later rounds), but the lengths are drawn once and are the same in every round,
    because the bench counts the tokens of round 0 (bench/gen_workload.py:55-60);
  * requests ignore the end-of-sequence token, so that every engine produces the same number
    of tokens, and sample at temperature 0.6 (bench/gen_workload.py:13).
Token ids are uniform in [0, vocab); the reference draws from [0, 10000], hence the default.
"""
from __future__ import annotations

import json
import random
from dataclasses import dataclass, replace
from typing import Dict, List, Optional, Tuple


class WorkloadError(ValueError):
    pass


@dataclass(frozen=True)
class Shape:
    requests: int                    # requests per round
    rounds: int
    input: Tuple[int, int]           # prompt length, lowest and highest (inclusive)
    output: Tuple[int, int]          # max_tokens, lowest and highest (inclusive)

    def check(self) -> None:
        if self.requests <= 0 or self.rounds <= 0:
            raise WorkloadError("a workload has at least one request and one round")
        for what, (lo, hi) in (("input", self.input), ("output", self.output)):
            if lo <= 0 or hi < lo:
                raise WorkloadError(f"{what} lengths {lo}:{hi} must be positive and ordered")


# The reference's scenarios by what they measure (bench/gen_workload.py:5-12).
SCENARIOS: Dict[str, Shape] = {
    "single": Shape(1, 5, (512, 512), (256, 256)),            # one stream: TTFT, ITL, tokens/s of one request
    "concurrent8": Shape(8, 3, (256, 512), (128, 512)),       # decode batches in the graph buckets 4 and 8
    "concurrent32": Shape(32, 1, (128, 512), (128, 512)),     # medium concurrency
    "bench256": Shape(256, 1, (100, 1024), (100, 1024)),      # throughput under load, preemption
    "longctx": Shape(1, 3, (3584, 3584), (512, 512)),         # decode attention over a long context
}


def parse_range(text: str, what: str) -> Tuple[int, int]:
    """"512" or "100:1024" -> (lowest, highest)."""
    try:
        parts = [int(p) for p in text.split(":")]
    except ValueError:
        parts = []
    if len(parts) == 1:
        return parts[0], parts[0]
    if len(parts) == 2:
        return parts[0], parts[1]
    raise WorkloadError(f"{what}: expected N or LOW:HIGH, got {text!r}")


def resolve_shape(scenario: Optional[str], requests: Optional[int] = None, rounds: Optional[int] = None,
                  input: Optional[Tuple[int, int]] = None, output: Optional[Tuple[int, int]] = None) -> Tuple[str, Shape]:
    """The scenario's shape with the given numbers put in its place; (name, shape)."""
    if scenario is None:
        if None in (requests, input, output):
            raise WorkloadError("without --scenario a workload needs --requests, --input and --output")
        shape, name = Shape(requests, rounds or 1, input, output), "custom"
    else:
        if scenario not in SCENARIOS:
            raise WorkloadError(f"unknown scenario {scenario!r}; known: {', '.join(sorted(SCENARIOS))}")
        shape, name = SCENARIOS[scenario], scenario
        changes = {k: v for k, v in (("requests", requests), ("rounds", rounds), ("input", input), ("output", output))
                   if v is not None}
        if changes:
            shape, name = replace(shape, **changes), scenario + "-modified"
    shape.check()
    return name, shape


def make_workload(name: str, shape: Shape, vocab: int = 10001, seed: int = 0, temperature: float = 0.6,
                  ignore_eos: bool = True, max_model_len: Optional[int] = None) -> dict:
    """Draw the workload.  With `max_model_len`, a request whose prompt and output together exceed it
    has its output shortened (the engine refuses such a request, src/engine.zig:86-93); a prompt
    that leaves no room at all is an error."""
    shape.check()
    if vocab <= 0:
        raise WorkloadError("vocab must be positive")
    rng = random.Random(seed)
    lengths: List[Tuple[int, int]] = []
    for _ in range(shape.requests):
        n_in = rng.randint(*shape.input)
        n_out = rng.randint(*shape.output)
        if max_model_len is not None:
            if n_in >= max_model_len:
                raise WorkloadError(f"a prompt of {n_in} tokens leaves no room under max_model_len {max_model_len}")
            n_out = min(n_out, max_model_len - n_in)
        lengths.append((n_in, n_out))
    rounds = [[{"prompt_ids": [rng.randrange(vocab) for _ in range(n_in)], "max_tokens": n_out,
                "temperature": float(temperature), "ignore_eos": bool(ignore_eos)} for n_in, n_out in lengths]
              for _ in range(shape.rounds)]
    return {"name": name, "rounds": rounds}


def summary(workload: dict) -> str:
    first = workload["rounds"][0]
    n_in = sum(len(r["prompt_ids"]) for r in first)
    n_out = sum(r["max_tokens"] for r in first)
    return (f"{workload['name']}: {len(first)} requests x {len(workload['rounds'])} rounds, "
            f"{n_in} input / {n_out} output tokens a round")


def write_workload(path: str, workload: dict) -> None:
    with open(path, "w", encoding="utf-8") as f:
        json.dump(workload, f)
