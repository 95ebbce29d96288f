"""A plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache, one
function per part, float32 (or float64) on the CPU.  It shares no code with `llmgen_b200`;
it reads a model folder with the `safetensors` library.

It rests on the reference's formulas, not on running the reference: the reference's model code
is Zig (src/models/qwen3.zig, src/backend/cpu/*.zig) and no Zig compiler exists here, so it
cannot be imported or compiled.  Each function cites the lines it restates.  Two of its
functions are pinned to the reference's own PyTorch-made fixtures
(testdata/linear_case.*, testdata/norm_case.*; copies of the numbers in
tests/golden/reference_fixtures.json, made by tests/golden/make_reference_fixtures.py).
The reference's CUDA kernels, which are plain C entry points, do compile here (for sm_100a,
unmodified): the per-head norm, the rotary pairing and angles, the place of a key in a page,
the attention of a chunk's tail over shuffled pages with grouped heads (prompt and split decode
kernels) and the sampler are pinned to their outputs on a B200
(tests/golden/reference_kernel_fixtures.json, made by
tests/golden/make_reference_kernel_fixtures.py; tests/test_plain.py).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open


# ------------------------------------------------------------------------- parts
def embedding(ids: Sequence[int], table: torch.Tensor) -> torch.Tensor:
    """x[t, :] = E[ids[t], :]; an id outside [0, V) is an error
    (src/backend/cpu/embedding.zig:20-27)."""
    V = table.shape[0]
    for i in ids:
        if not 0 <= int(i) < V:
            raise IndexError(f"token id {i} out of range [0, {V})")
    return table[torch.as_tensor(list(ids), dtype=torch.long)]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, weight_offset: float = 0.0) -> torch.Tensor:
    """ss = sum x^2; r = 1/sqrt(ss/D + eps); y = x * r * (w + w_offset)
    (src/backend/cpu/norm.zig:60-93; its rounding of x*r to bfloat16 applies only to bfloat16
    activations and is not part of the formula)."""
    D = x.shape[-1]
    ss = (x * x).sum(dim=-1, keepdim=True)
    r = 1.0 / torch.sqrt(ss / D + eps)
    return x * r * (weight + weight_offset)


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = x W^T with W stored [out, in], no bias (src/backend/cpu/linear.zig:7-28)."""
    return x @ weight.t()


def rope_tables(max_positions: int, rotary_dim: int, theta: float):
    """inv_f[i] = 1 / theta^(2i / rotary_dim); angle = pos * inv_f[i]; computed in float64
    (src/backend/cpu/rope.zig:47-75)."""
    half = rotary_dim // 2
    inv = torch.tensor([1.0 / (float(theta) ** (2.0 * i / rotary_dim)) for i in range(half)], dtype=torch.float64)
    ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, positions: Sequence[int], cos: torch.Tensor, sin: torch.Tensor,
               rotary_dim: int) -> torch.Tensor:
    """Half-split pairing on x [T, heads, hd]: y[i] = x[i] cos - x[i+half] sin,
    y[i+half] = x[i+half] cos + x[i] sin for i < rotary_dim/2; the rest is copied
    (src/backend/cpu/rope.zig:13-45)."""
    half = rotary_dim // 2
    pos = torch.as_tensor(list(positions), dtype=torch.long)
    c = cos[pos].to(x.dtype)[:, None, :]
    s = sin[pos].to(x.dtype)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:rotary_dim]
    out = x.clone()
    out[..., :half] = x0 * c - x1 * s
    out[..., half:rotary_dim] = x1 * c + x0 * s
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None) -> torch.Tensor:
    """q [T, nq, hd], k and v [T, nkv, hd] of ONE whole sequence: query t sees keys 0..t
    (with a window W: keys t-W+1..t); score = (q.k) * scale; softmax; head h reads kv head
    h // (nq / nkv) (src/backend/cpu/attention.zig:64-118)."""
    T, nq, hd = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    out = torch.zeros_like(q)
    idx = torch.arange(T)
    visible = idx[None, :] <= idx[:, None]
    if window:
        visible &= idx[None, :] > idx[:, None] - window
    for h in range(nq):
        kvh = h // group
        scores = (q[:, h, :] @ k[:, kvh, :].t()) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        out[:, h, :] = torch.softmax(scores, dim=-1) @ v[:, kvh, :]
    return out


def swiglu_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """g = x Wg^T; u = x Wu^T; act = g / (1 + exp(-g)); m = (act * u) Wd^T
    (src/models/qwen3.zig:153-162, src/backend/cpu/activation.zig:13-17,
    src/backend/cpu/arithmetic.zig:28-38)."""
    g = linear(x, w_gate)
    u = linear(x, w_up)
    act = g / (1.0 + torch.exp(-g))
    return linear(act * u, w_down)


def gumbel_sample(logits: torch.Tensor, temperature: float, step_seed: int, row: int) -> int:
    """temperature <= 0: argmax, ties to the smaller id.  Otherwise
    argmax(logit / T - log(-log u)), u = ((r >> 40) + 0.5) / 2^24, r = splitmix64(row_seed + id),
    row_seed = splitmix64(step_seed ^ (row << 40)) (src/backend/cpu/sample.zig:8-45)."""
    if temperature <= 0:
        return int(torch.argmax(logits).item())
    scores = gumbel_scores(logits, temperature, step_seed, row)
    return int(torch.argmax(scores).item())


def splitmix64(x: int) -> int:
    """src/backend/cpu/sample.zig:8-13."""
    m = (1 << 64) - 1
    x = (x + 0x9E3779B97F4A7C15) & m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    return x ^ (x >> 31)


def gumbel_scores(logits: torch.Tensor, temperature: float, step_seed: int, row: int) -> torch.Tensor:
    m = (1 << 64) - 1
    seed = splitmix64((step_seed ^ (row << 40)) & m)
    us = []
    for i in range(logits.shape[0]):
        r = splitmix64((seed + i) & m)
        us.append((float(r >> 40) + 0.5) * (1.0 / 16777216.0))
    u = torch.tensor(us, dtype=torch.float32)
    return logits.to(torch.float32) / temperature - torch.log(-torch.log(u))


# ------------------------------------------------------------------------- the model
class PlainQwen3:
    """Reads config.json and model.safetensors of a folder and computes logits of whole
    sequences (src/models/qwen3.zig:224-236, 300-330)."""

    def __init__(self, model_dir: str, dtype: torch.dtype = torch.float32, round_to: Optional[torch.dtype] = None):
        """`round_to=torch.bfloat16`: weights and the output of every node are rounded to bfloat16 and widened
        again, which is how the reference computes with bfloat16 activations (each node of its graph stores
        its result in the activation dtype, src/models/qwen3.zig:153-162, src/backend/cpu/norm.zig:60-93).
        The distance between such a run and the exact one is the scale of what bfloat16 arithmetic costs on
        this model; tests bound the engine's bfloat16 error by a multiple of it."""
        with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
            c = json.load(f)
        self.c = c
        self.dtype = dtype
        self.round_to = round_to
        self.L = c["num_hidden_layers"]
        self.H = c["hidden_size"]
        self.nq = c["num_attention_heads"]
        self.nkv = c["num_key_value_heads"]
        self.hd = c.get("head_dim") or self.H // self.nq
        self.eps = c["rms_norm_eps"]
        self.theta = c["rope_theta"]
        self.tied = bool(c.get("tie_word_embeddings", False))
        self.scale = 1.0 / math.sqrt(self.hd)           # src/executor.zig:877
        types = c.get("layer_types")
        window = c.get("sliding_window")
        if types is None:
            if c.get("use_sliding_window") and window:
                first = c.get("max_window_layers", self.L)
                types = ["sliding_attention" if i >= first else "full_attention" for i in range(self.L)]
            else:
                types = ["full_attention"] * self.L
        self.windows = [window if t == "sliding_attention" else None for t in types]
        self.w: Dict[str, torch.Tensor] = {}
        with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                if round_to is not None and t.dim() >= 2:           # matrices and tables; gains stay as stored
                    t = t.to(round_to)
                self.w[name] = t.to(dtype)
        self.cos, self.sin = rope_tables(c["max_position_embeddings"], self.hd, self.theta)

    def rnd(self, x: torch.Tensor) -> torch.Tensor:
        """A node's output as it is stored: rounded to the activation dtype when one is set."""
        return x if self.round_to is None else x.to(self.round_to).to(x.dtype)

    def layer(self, i: int, x: torch.Tensor, positions: Sequence[int]) -> torch.Tensor:
        w, p, r = self.w, f"model.layers.{i}.", self.rnd
        T = x.shape[0]
        h = r(rmsnorm(x, w[p + "input_layernorm.weight"], self.eps))
        q = r(linear(h, w[p + "self_attn.q_proj.weight"])).view(T, self.nq, self.hd)
        k = r(linear(h, w[p + "self_attn.k_proj.weight"])).view(T, self.nkv, self.hd)
        v = r(linear(h, w[p + "self_attn.v_proj.weight"])).view(T, self.nkv, self.hd)
        q = r(rmsnorm(q, w[p + "self_attn.q_norm.weight"], self.eps))     # per head, before RoPE
        k = r(rmsnorm(k, w[p + "self_attn.k_norm.weight"], self.eps))     # (src/models/qwen3.zig:200-201)
        q = r(apply_rope(q, positions, self.cos, self.sin, self.hd))
        k = r(apply_rope(k, positions, self.cos, self.sin, self.hd))
        a = r(causal_attention(q, k, v, self.scale, self.windows[i])).reshape(T, self.nq * self.hd)
        x1 = r(x + r(linear(a, w[p + "self_attn.o_proj.weight"])))
        h2 = r(rmsnorm(x1, w[p + "post_attention_layernorm.weight"], self.eps))
        if self.round_to is None:
            m = swiglu_mlp(h2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        else:           # the same four nodes, each stored rounded
            g = r(linear(h2, w[p + "mlp.gate_proj.weight"]))
            u = r(linear(h2, w[p + "mlp.up_proj.weight"]))
            m = r(linear(r(r(g / (1.0 + torch.exp(-g))) * u), w[p + "mlp.down_proj.weight"]))
        return r(x1 + m)

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        """float logits [T, V] of one whole sequence starting at position 0."""
        x = embedding(ids, self.w["model.embed_tokens.weight"])
        positions = list(range(len(ids)))
        for i in range(self.L):
            x = self.layer(i, x, positions)
        x = self.rnd(rmsnorm(x, self.w["model.norm.weight"], self.eps))
        head = self.w["model.embed_tokens.weight"] if self.tied else self.w["lm_head.weight"]
        return self.rnd(linear(x, head))

    def greedy(self, prompt: Sequence[int], n_new: int) -> List[int]:
        ids = list(prompt)
        for _ in range(n_new):
            ids.append(int(torch.argmax(self.logits(ids)[-1]).item()))
        return ids[len(prompt):]
