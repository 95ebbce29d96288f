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
TINY_D = {  # head_dim 64 and a group of 3: the tensor-core and flash-decoding kernels of the bfloat16 path; a window
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 333, "hidden_size": 128, "intermediate_size": 208, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64,
    "rms_norm_eps": 2e-6, "rope_theta": 100000.0, "max_position_embeddings": 1024,
    "tie_word_embeddings": True, "hidden_act": "silu",
    "sliding_window": 150, "use_sliding_window": True,
    "layer_types": ["full_attention", "sliding_attention", "full_attention"],
}
TINY_E = {  # head_dim 128, group of 2, pages of 32: the benchmark's head geometry in small
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 290, "hidden_size": 96, "intermediate_size": 160, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 1024,
    "tie_word_embeddings": False, "hidden_act": "silu",
}
TINY = {"A": (TINY_A, 0, 0.02, 0.1, "bfloat16", 16),     # config, seed, sigma, sigma_norm, stored as, page
        "B": (TINY_B, 1, 0.03, 0.05, "float32", 32),
        "C": (TINY_C, 5, 0.05, 0.2, "bfloat16", 16),
        "D": (TINY_D, 6, 0.04, 0.1, "bfloat16", 16),
        "E": (TINY_E, 7, 0.05, 0.1, "float32", 32)}


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


FP32_TOL = 1e-4          # max abs difference of float32 logits (logits here are O(1))


def bf16_tol(ref: torch.Tensor) -> float:
    """bfloat16 keeps 8 bits of mantissa: logits may differ by a few percent of their scale."""
    return 4e-2 * max(1.0, float(ref.abs().max()))


def logits_close(got: torch.Tensor, ref: torch.Tensor, dtype: str) -> float:
    diff = float((got.float() - ref.float()).abs().max())
    limit = FP32_TOL if dtype == "float32" else bf16_tol(ref)
    assert diff <= limit, f"max |diff| {diff:.3e} above {limit:.3e} ({dtype})"
    return diff


def manual_context(q_lens, starts, tables, page_size, dtype, mixers=(), max_step_tokens=4096, state_slots=None):
    """A StepContext built by hand (one cache group), for tests that run a single part.
    `tables[s]` is the block table of sequence s."""
    import numpy as np
    from llmgen_b200.engine.context import GroupView, StepContext, StepMetaBuilder, Workspace
    S, T = len(q_lens), sum(q_lens)
    max_blocks = max(len(t) for t in tables)
    b = StepMetaBuilder(q_lens, starts, all(n == 1 for n in q_lens), page_size)
    pos, seq_of, slots = [], [], []
    cu = [0]
    for s, (n, st) in enumerate(zip(q_lens, starts)):
        for p in range(st, st + n):
            pos.append(p)
            seq_of.append(s)
            slots.append(tables[s][p // page_size] * page_size + p % page_size)
        cu.append(cu[-1] + n)
    bt = np.zeros((S, max_blocks), dtype=np.int32)
    for s, t in enumerate(tables):
        bt[s, :len(t)] = t
    for m in mixers:
        m.prepare_step(b)
    dev = lambda a, dt=torch.int32: torch.as_tensor(np.asarray(a), dtype=dt).cuda()
    ctx = StepContext(
        n_tokens=T, n_seqs=S, dtype=dtype, device=torch.device("cuda:0"), workspace=Workspace(torch.device("cuda:0"), max_step_tokens),
        requests=list(range(S)), starts=list(starts), q_lens=list(q_lens), pure_decode=b.pure_decode,
        max_ctx=max(s + n for s, n in zip(starts, q_lens)), max_ctx_bound=max_blocks * page_size, max_seqs_bound=S,
        ids=dev([0] * T), positions=dev(pos), cu_q=dev(cu), ctx_len=dev([s + n for s, n in zip(starts, q_lens)]),
        state_slots=dev(state_slots if state_slots is not None else list(range(S))), seq_of_token=dev(seq_of),
        groups=[GroupView(dev(slots), dev(bt.reshape(-1)), max_blocks)],
        extra={name: dev(arr) for name, arr in b.arrays.items()})
    return ctx
