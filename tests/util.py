"""Shared by the tests: the tiny configurations, model folders in temporary places, and
helpers that drive the engine the way a trace does."""
from __future__ import annotations

import os
import random
import sys
from typing import Dict, List, Sequence

import torch

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Three tiny Qwen3 configurations that differ in every size and option.
TINY_A = {  # grouped heads 4/2, power-of-two sizes, tied head, no window
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 512,
    "tie_word_embeddings": True, "hidden_act": "silu",
}
TINY_B = {  # 8 query heads on 1 kv head, head_dim decoupled from hidden, untied head, odd sizes
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 384, "hidden_size": 96, "intermediate_size": 320, "num_hidden_layers": 3,
    "num_attention_heads": 8, "num_key_value_heads": 1, "head_dim": 32,
    "rms_norm_eps": 1e-5, "rope_theta": 1000000.0, "max_position_embeddings": 640,
    "tie_word_embeddings": False, "hidden_act": "silu",
}
TINY_C = {  # sizes that are no power of two, group of 3, a window on some layers
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 301, "hidden_size": 80, "intermediate_size": 176, "num_hidden_layers": 4,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 48,
    "rms_norm_eps": 3e-6, "rope_theta": 50000.0, "max_position_embeddings": 768,
    "tie_word_embeddings": False, "hidden_act": "silu",
    "sliding_window": 40, "use_sliding_window": True,
    "layer_types": ["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
}
TINY = {"A": (TINY_A, 0, 0.02, 0.1, "bfloat16", 16),     # config, seed, sigma, sigma_norm, stored as, page
        "B": (TINY_B, 1, 0.03, 0.05, "float32", 32),
        "C": (TINY_C, 5, 0.05, 0.2, "bfloat16", 16)}


def make_folder(tmpdir: str, name: str) -> str:
    from llmgen_b200.engine.api import write_random_model
    cfg, seed, sigma, sigma_norm, store, _ = TINY[name]
    path = os.path.join(tmpdir, f"tiny_{name}")
    if not os.path.isdir(path):
        write_random_model(path, cfg, seed, sigma, sigma_norm, store)
    return path


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


class Driver:
    """Drives an `Executor` the way `bin/trace_run` does: keeps each request's position,
    reserves pages, runs steps, gives pages back."""

    def __init__(self, model_dir: str, dtype: str, pool_tokens: int, page_size: int = 16, max_num_seqs: int = 8):
        from llmgen_b200.engine.api import load_model
        from llmgen_b200.engine.executor import EngineLimits, Executor
        self.model = load_model(model_dir, dtype)
        limits = EngineLimits(max_num_seqs=max_num_seqs, max_model_len=min(self.model.max_positions(), pool_tokens),
                              max_step_tokens=pool_tokens, page_size=page_size, num_pages=pool_tokens // page_size)
        self.executor = Executor(self.model, limits, eager=True)
        self.positions: Dict[object, int] = {}

    def step(self, entries: Sequence[tuple], end: Sequence = ()) -> torch.Tensor:
        """entries: (request id, tokens, want) tuples; returns float32 logits [wanted, V] on the CPU."""
        from llmgen_b200.engine.executor import StepEntry
        batch = []
        for rid, tokens, want in entries:
            start = self.positions.get(rid, 0)
            if rid not in self.positions:
                assert self.executor.admit(rid)
            assert self.executor.reserve(rid, start, start + len(tokens)), "out of pages"
            self.positions[rid] = start + len(tokens)
            batch.append(StepEntry(rid, list(tokens), start, list(want)))
        out = self.executor.step(batch, sample=False, return_logits=True)
        for rid in end:
            self.executor.release(rid)
            del self.positions[rid]
        return out.logits.float().cpu()
