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
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 128,
    "tie_word_embeddings": True, "hidden_act": "silu",
}
TINY_B = {  # 8 query heads on 1 kv head, head_dim decoupled from hidden, untied head, odd sizes
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 384, "hidden_size": 96, "intermediate_size": 320, "num_hidden_layers": 3,
    "num_attention_heads": 8, "num_key_value_heads": 1, "head_dim": 32,
    "rms_norm_eps": 1e-5, "rope_theta": 1000000.0, "max_position_embeddings": 256,
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


def make_folder(tmpdir: str, name: str, **overrides) -> str:
    """The model folder of tiny configuration `name`; `overrides` change keys of its config.json (for the
    tests that need more positions than the configuration has: the weights stay the same)."""
    from llmgen_b200.engine.api import write_random_model
    cfg, seed, sigma, sigma_norm, store, _ = TINY[name]
    tag = "".join(f"_{k}{v}" for k, v in sorted(overrides.items()))
    path = os.path.join(tmpdir, f"tiny_{name}{tag}")
    if not os.path.isdir(path):
        write_random_model(path, dict(cfg, **overrides), seed, sigma, sigma_norm, store)
    return path


NEEDLE_ID, PROBE_ID, FILLER_ID = 7, 11, 13


def needle_folder(tmpdir: str, name: str, n_slow: int = 8) -> str:
    """A copy of tiny model `name` in which the first layer's heads of kv head 0 look for one token.

    Random weights spread attention thinly, so that one key read from the wrong place moves the logits
    by less than bfloat16 rounding does.  Here the q rows of those heads and the k rows of kv head 0
    are rebuilt so that (i) q and k live in the `n_slow` slowest rotary pairs only, which the rotary
    encoding turns by less than 0.1 rad over a thousand positions, and (ii) the query of token
    PROBE_ID equals the key of token NEEDLE_ID.  After the per-head norm the score of that pair is
    about sqrt(head_dim) while other keys score like random directions in 2 n_slow dimensions: a probe
    token puts most of its weight on the needle, wherever it lies, and the last row's logits move by
    20 to 30 times the bfloat16 bound when the needle's key or value is not the one that was written."""
    from safetensors.torch import load_file, save_file
    from tests.plain import qwen3_plain as plain
    base = make_folder(tmpdir, name)
    out = os.path.join(tmpdir, f"needle_{name}")
    if os.path.isdir(out):
        return out
    cfg = TINY[name][0]
    os.makedirs(out)
    with open(os.path.join(base, "config.json")) as f, open(os.path.join(out, "config.json"), "w") as g:
        g.write(f.read())
    t = load_file(os.path.join(base, "model.safetensors"))
    H, hd = cfg["hidden_size"], cfg["head_dim"]
    group = cfg["num_attention_heads"] // cfg["num_key_value_heads"]
    half = hd // 2
    dims = torch.tensor([i for i in range(half - n_slow, half)] + [i + half for i in range(half - n_slow, half)])
    emb = t["model.embed_tokens.weight"].float()
    gain = t["model.layers.0.input_layernorm.weight"].float()
    x_needle = plain.rmsnorm(emb[NEEDLE_ID], gain, cfg["rms_norm_eps"])
    x_probe = plain.rmsnorm(emb[PROBE_ID], gain, cfg["rms_norm_eps"])
    gen = torch.Generator().manual_seed(0)
    B = torch.randn(len(dims), H, generator=gen) * 0.05
    A = torch.randn(len(dims), H, generator=gen) * 0.05
    A = A + torch.outer(B @ x_needle - A @ x_probe, x_probe) / (x_probe @ x_probe)      # A x_probe = B x_needle
    wq, wk = t["model.layers.0.self_attn.q_proj.weight"], t["model.layers.0.self_attn.k_proj.weight"]
    q, k = wq.float(), wk.float()
    for h in range(group):
        q[h * hd:(h + 1) * hd] = 0
        q[h * hd + dims] = A
    k[0:hd] = 0
    k[dims] = B
    t["model.layers.0.self_attn.q_proj.weight"] = q.to(wq.dtype)
    t["model.layers.0.self_attn.k_proj.weight"] = k.to(wk.dtype)
    save_file(t, os.path.join(out, "model.safetensors"))
    return out


def needle_ids(n: int, vocab: int, needle_at: int, seed: int) -> List[int]:
    """`n` random ids with the needle token at `needle_at` only and the probe token last only."""
    ids = [t if t not in (NEEDLE_ID, PROBE_ID) else FILLER_ID for t in random_ids(n, vocab, seed)]
    ids[needle_at] = NEEDLE_ID
    ids[-1] = PROBE_ID
    return ids


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


class Driver:
    """Drives an `Executor` the way `bin/trace_run` does: keeps each request's position,
    reserves pages, runs steps, gives pages back."""

    def __init__(self, model_dir: str, dtype: str, pool_tokens: int, page_size: int = 16, max_num_seqs: int = 8, model=None,
                 eager: bool = True):
        from llmgen_b200.engine.api import load_model
        from llmgen_b200.engine.executor import EngineLimits, Executor
        self.model = model if model is not None else load_model(model_dir, dtype)
        limits = EngineLimits(max_num_seqs=max_num_seqs, max_model_len=min(self.model.max_positions(), pool_tokens),
                              max_step_tokens=pool_tokens, page_size=page_size, num_pages=pool_tokens // page_size)
        self.executor = Executor(self.model, limits, eager=eager)
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
BF16_FACTOR = 3.0        # the engine's bfloat16 logits stay within this many times what bfloat16 storage costs the plain model

_plain_models: Dict[tuple, object] = {}


def plain_model(path: str, rounded: bool = False):
    from tests.plain.qwen3_plain import PlainQwen3
    key = (path, rounded)
    if key not in _plain_models:
        _plain_models[key] = PlainQwen3(path, round_to=torch.bfloat16 if rounded else None)
    return _plain_models[key]


def forget_plain_models() -> None:
    _plain_models.clear()


def reference(path: str, ids: Sequence[int]):
    """(exact logits [T, V] of the plain implementation, the bfloat16 bound for this model on these ids).

    The bound is BF16_FACTOR times the largest difference between the plain model run exactly and run the way
    the reference runs in bfloat16 (weights and every node's output rounded to bfloat16): it is tied to this
    model and these tokens, so a configuration with small logits gets a small bound."""
    exact = plain_model(path).logits(ids)
    rounded = plain_model(path, rounded=True).logits(ids)
    return exact, BF16_FACTOR * float((exact - rounded).abs().max())


def logits_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, bound: float = None) -> float:
    """float32: within FP32_TOL of the plain logits.  bfloat16: within `bound` (from `reference`)."""
    diff = float((got.float() - ref.float()).abs().max())
    if dtype == "float32":
        limit = FP32_TOL
    else:
        assert bound is not None and bound > 0, "a bfloat16 comparison needs the model's own bound (tests.util.reference)"
        limit = bound
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
