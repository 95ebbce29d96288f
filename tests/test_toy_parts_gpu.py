"""Parts that no model of the framework has, defined here and registered with one call each: a
feed-forward with routing (top-2 of a few small experts) and another position encoding (rotation
angles that grow with the square root of the position, over a part of the head).  An architecture
made of them, with the framework's own attention and norms, is built and stepped in portions and
compared with plain torch on the CPU.  Nothing under `llmgen_b200/` knows these kinds."""
from dataclasses import dataclass
from typing import Tuple

import pytest
import torch

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class RoutedSpec:
    """y = sum over the `top_k` experts e with the largest router logit of p_e * W2_e relu(W1_e x),
    p = softmax over the chosen logits (float32)."""
    hidden_size: int
    expert_size: int
    num_experts: int
    top_k: int
    router: str
    w1: Tuple[str, ...]
    w2: Tuple[str, ...]
    kind: str = "toy_routed"


@dataclass(frozen=True)
class RootRopeSpec:
    """Half-split rotation of the first `rotary_dim` values of a head by angle sqrt(pos) * stretch / base^(2i/rotary_dim)."""
    rotary_dim: int
    base: float
    stretch: float
    max_positions: int
    kind: str = "toy_root_rope"


def root_rope_tables(spec):
    half = spec.rotary_dim // 2
    inv = 1.0 / torch.pow(torch.tensor(spec.base, dtype=torch.float64), torch.arange(half, dtype=torch.float64) * 2.0 / spec.rotary_dim)
    ang = torch.arange(spec.max_positions, dtype=torch.float64).sqrt()[:, None] * spec.stretch * inv[None, :]
    return ang.cos(), ang.sin()


def make_parts():
    from llmgen_b200.parts.base import FeedForward, Part
    from llmgen_b200.parts.spec import WeightDecl

    class RoutedFeedForward(FeedForward):
        capturable = False          # `forward` asks which rows chose an expert (a read-back): no graph can hold it

        @staticmethod
        def weight_decls(spec):
            decls = [WeightDecl(spec.router, (spec.num_experts, spec.hidden_size))]
            for e in range(spec.num_experts):
                decls += [WeightDecl(spec.w1[e], (spec.expert_size, spec.hidden_size)),
                          WeightDecl(spec.w2[e], (spec.hidden_size, spec.expert_size))]
            return decls

        def __init__(self, spec, weights, dtype, device):
            self.spec, self.dtype = spec, dtype
            self.router = weights.device_tensor(spec.router, torch.float32, device)
            self.w1 = [weights.device_tensor(n, dtype, device) for n in spec.w1]
            self.w2 = [weights.device_tensor(n, dtype, device) for n in spec.w2]

        def forward(self, ctx, x):
            logits = x.float() @ self.router.t()
            top, idx = logits.topk(self.spec.top_k, dim=-1)
            p = torch.softmax(top, dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e in range(self.spec.num_experts):
                rows, which = (idx == e).nonzero(as_tuple=True)
                if rows.numel():
                    h = torch.relu(x[rows] @ self.w1[e].t()) @ self.w2[e].t()
                    out.index_add_(0, rows, h.float() * p[rows, which][:, None])
            return out.to(self.dtype)

    class RootRope(Part):
        def __init__(self, spec, weights, dtype, device):
            cos, sin = root_rope_tables(spec)
            self.cos, self.sin = cos.float().to(device).contiguous(), sin.float().to(device).contiguous()
            self.rotary_dim, self.max_positions = spec.rotary_dim, spec.max_positions

        def tables(self):
            return self.cos, self.sin

    return RoutedFeedForward, RootRope


def plain_logits(tensors, d, ids):
    """The same model on a whole sequence: the plain implementation's functions, the toy formulas inline."""
    from tests.plain import qwen3_plain as plain
    w = {k: v.float() for k, v in tensors.items()}
    H, nq, nkv, hd = d["hidden_size"], d["heads"], d["kv_heads"], d["head_dim"]
    T = len(ids)
    cos, sin = root_rope_tables(RootRopeSpec(d["rotary_dim"], d["base"], d["stretch"], d["max_positions"]))
    x = w["emb"][torch.tensor(ids)]
    for i in range(d["layers"]):
        h = plain.rmsnorm(x, w[f"l{i}.n1"], d["eps"])
        q = plain.linear(h, w[f"l{i}.q"]).view(T, nq, hd)
        k = plain.linear(h, w[f"l{i}.k"]).view(T, nkv, hd)
        v = plain.linear(h, w[f"l{i}.v"]).view(T, nkv, hd)
        q = plain.apply_rope(q, range(T), cos, sin, d["rotary_dim"])
        k = plain.apply_rope(k, range(T), cos, sin, d["rotary_dim"])
        o = plain.causal_attention(q, k, v, d["scale"]).reshape(T, nq * hd)
        x = x + plain.linear(o, w[f"l{i}.o"])
        h = plain.rmsnorm(x, w[f"l{i}.n2"], d["eps"])
        if i % 2 == 0:
            logits = h @ w[f"l{i}.router"].t()
            top, idx = logits.topk(d["top_k"], dim=-1)
            p = torch.softmax(top, dim=-1)
            y = torch.zeros_like(h)
            for t in range(T):
                for j in range(d["top_k"]):
                    e = int(idx[t, j])
                    y[t] += p[t, j] * (torch.relu(h[t] @ w[f"l{i}.e{e}.w1"].t()) @ w[f"l{i}.e{e}.w2"].t())
        else:
            y = plain.swiglu_mlp(h, w[f"l{i}.g"], w[f"l{i}.u"], w[f"l{i}.d"])
        x = x + y
    return plain.linear(plain.rmsnorm(x, w["norm"], d["eps"]), w["head"])


def test_routed_feed_forward_and_another_position_encoding_register_build_and_step():
    from llmgen_b200.engine.api import require_cuda
    from llmgen_b200.engine.executor import EngineLimits, Executor, StepEntry
    from llmgen_b200.engine.model import DecoderModel
    from llmgen_b200.parts.registry import model_weight_decls, register_feed_forward, register_position
    from llmgen_b200.parts.spec import (AttentionSpec, GatedMLPSpec, ModelSpec, PreNormBlockSpec, RMSNormSpec,
                                        default_run_order)
    from llmgen_b200.registry import config_from_dict, register_architecture, unregister_architecture
    from llmgen_b200.weights import random_tensors, weights_from_dict

    routed_cls, rope_cls = make_parts()
    register_feed_forward("toy_routed", routed_cls)
    register_position("toy_root_rope", rope_cls)

    class ToyConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, data, where="config.json"):
            return cls(data)

    def build_spec(cfg):
        d = cfg.d
        H, E = d["hidden_size"], d["experts"]
        position = RootRopeSpec(d["rotary_dim"], d["base"], d["stretch"], d["max_positions"])
        layers = []
        for i in range(d["layers"]):
            mixer = AttentionSpec(H, d["heads"], d["kv_heads"], d["head_dim"], d["scale"], f"l{i}.q", f"l{i}.k", f"l{i}.v",
                                  f"l{i}.o", position=position)
            if i % 2 == 0:      # layers differ in their feed-forward: routed, dense, routed
                ffn = RoutedSpec(H, d["expert_size"], E, d["top_k"], f"l{i}.router",
                                 tuple(f"l{i}.e{e}.w1" for e in range(E)), tuple(f"l{i}.e{e}.w2" for e in range(E)))
            else:
                ffn = GatedMLPSpec(H, d["ffn"], f"l{i}.g", f"l{i}.u", f"l{i}.d")
            layers.append(PreNormBlockSpec(mixer_norm=RMSNormSpec(H, d["eps"], f"l{i}.n1"), mixer=mixer,
                                           ffn_norm=RMSNormSpec(H, d["eps"], f"l{i}.n2"), ffn=ffn))
        return ModelSpec(architecture="ToyRoutedForCausalLM", vocab_size=d["vocab"], hidden_size=H, embedding="emb",
                         layers=tuple(layers), run_order=default_run_order(d["layers"]),
                         final_norm=RMSNormSpec(H, d["eps"], "norm"), lm_head="head", max_positions=d["max_positions"])

    register_architecture("ToyRoutedForCausalLM", ToyConfig, build_spec)
    try:
        d = {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 48, "heads": 3, "kv_heads": 1, "head_dim": 32,
             "rotary_dim": 16, "base": 500.0, "stretch": 1.7, "scale": 0.21, "max_positions": 128, "eps": 2e-6,
             "experts": 5, "expert_size": 24, "top_k": 2, "ffn": 72, "layers": 3, "vocab": 111}
        arch, cfg = config_from_dict(d)
        spec = arch.build_spec(cfg)
        decls = model_weight_decls(spec)
        assert sum(1 for x in decls if ".e" in x.name) == 2 * 2 * 5          # two routed layers, five experts, two matrices
        tensors = random_tensors(decls, 23, 0.15, 0.1, torch.float32)
        model = DecoderModel(spec, weights_from_dict(tensors, decls), torch.float32, require_cuda())
        # graphs are asked for; the routed feed-forward says it cannot be recorded, so every step is launched
        ex = Executor(model, EngineLimits(max_num_seqs=2, max_model_len=64, max_step_tokens=64, page_size=16, num_pages=6))
        assert ex.eager and ex.uncapturable == ["RoutedFeedForward"] and not ex.shaped_steps
        gen = torch.Generator().manual_seed(4)
        ids_a = torch.randint(0, d["vocab"], (37,), generator=gen).tolist()
        ids_b = torch.randint(0, d["vocab"], (21,), generator=gen).tolist()
        ref_a, ref_b = plain_logits(tensors, d, ids_a), plain_logits(tensors, d, ids_b)
        assert ex.admit("a") and ex.reserve("a", 0, len(ids_a))
        assert ex.admit("b") and ex.reserve("b", 0, len(ids_b))
        got_a = [ex.step([StepEntry("a", ids_a[:18], 0, list(range(18)))]).logits.cpu()]     # crosses a page's edge
        both = ex.step([StepEntry("b", ids_b[:9], 0, list(range(9))), StepEntry("a", ids_a[18:20], 18, [0, 1])]).logits.cpu()
        got_b = [both[:9]]
        got_a.append(both[9:])
        pos_a, pos_b = 20, 9
        while pos_a < len(ids_a) or pos_b < len(ids_b):          # then token by token, both at once while both last
            entries, owners = [], []
            if pos_a < len(ids_a):
                entries.append(StepEntry("a", ids_a[pos_a:pos_a + 1], pos_a, [0]))
                owners.append(got_a)
                pos_a += 1
            if pos_b < len(ids_b):
                entries.append(StepEntry("b", ids_b[pos_b:pos_b + 1], pos_b, [0]))
                owners.append(got_b)
                pos_b += 1
            out = ex.step(entries).logits.cpu()
            for r, owner in enumerate(owners):
                owner.append(out[r:r + 1])
        assert float((torch.cat(got_a) - ref_a).abs().max()) < 2e-4
        assert float((torch.cat(got_b) - ref_b).abs().max()) < 2e-4
        # the stretch matters: with the framework's own rotary tables the logits would differ
        from tests.plain import qwen3_plain as plain
        cos_std, _ = plain.rope_tables(d["max_positions"], d["rotary_dim"], d["base"])
        cos_toy, _ = root_rope_tables(spec.layers[0].mixer.position)
        assert float((cos_std - cos_toy).abs().max()) > 0.5
    finally:
        unregister_architecture("ToyRoutedForCausalLM")
