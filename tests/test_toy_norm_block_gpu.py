"""A norm and a block arrangement that no model of the framework has, defined here and registered with one call
each: a layer norm (mean removed, gain and bias) and a "parallel" block in which the mixer and the feed-forward both
read one normed input and both add to the residual, x' = x + mixer(norm(x)) + ffn(norm(x)).  An architecture made of
them, with the framework's own attention and feed-forward, is built and stepped in portions beside another request
and token by token, and compared with plain torch on the CPU.  Nothing under `llmgen_b200/` knows these kinds."""
from dataclasses import dataclass

import pytest
import torch

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class ToyLayerNormSpec:
    """y = (x - mean(x)) / sqrt(var(x) + eps) * gain + bias over the last `dim` values (float32)."""
    dim: int
    eps: float
    gain: str
    bias: str
    kind: str = "toy_layernorm"


@dataclass(frozen=True)
class ParallelBlockSpec:
    norm: object
    mixer: object
    ffn: object
    kind: str = "toy_parallel"


def make_parts():
    from llmgen_b200.kernels import ops
    from llmgen_b200.parts.base import Part
    from llmgen_b200.parts.registry import (build_feed_forward, build_mixer, build_norm, feed_forward_class, mixer_class,
                                            norm_class)
    from llmgen_b200.parts.spec import INIT_ONE_PLUS_NORMAL, VECTOR, WeightDecl

    def finished(delta):
        """What a part returned as an array: a product cut along K is summed (a part with no kernel for slices)."""
        return delta.sum() if isinstance(delta, ops.Partials) else delta

    class ToyLayerNorm(Part):
        @staticmethod
        def weight_decls(spec):
            return [WeightDecl(spec.gain, (spec.dim,), VECTOR, INIT_ONE_PLUS_NORMAL), WeightDecl(spec.bias, (spec.dim,), VECTOR)]

        @staticmethod
        def kernel_modules(spec):
            return ()

        def __init__(self, spec, weights, dtype, device):
            self.spec = spec
            self.gain = weights.device_tensor(spec.gain, torch.float32, device)
            self.bias = weights.device_tensor(spec.bias, torch.float32, device)

        def add_norm(self, resid, delta, out, rows=None):
            if delta is not None:
                resid += finished(delta).float()
            x = resid if rows is None else resid.index_select(0, rows.long())
            out.copy_(torch.nn.functional.layer_norm(x, (self.spec.dim,), self.gain, self.bias, self.spec.eps))
            return out

    class ParallelBlock(Part):
        @staticmethod
        def weight_decls(spec):
            return (norm_class(spec.norm).weight_decls(spec.norm) + mixer_class(spec.mixer).weight_decls(spec.mixer)
                    + feed_forward_class(spec.ffn).weight_decls(spec.ffn))

        @staticmethod
        def kernel_modules(spec):
            return (tuple(norm_class(spec.norm).kernel_modules(spec.norm)) + tuple(mixer_class(spec.mixer).kernel_modules(spec.mixer))
                    + tuple(feed_forward_class(spec.ffn).kernel_modules(spec.ffn)))

        def __init__(self, spec, weights, dtype, device):
            self.spec, self.dtype = spec, dtype
            self.norm = build_norm(spec.norm, weights, dtype, device)
            self.mixer = build_mixer(spec.mixer, weights, dtype, device)
            self.ffn = build_feed_forward(spec.ffn, weights, dtype, device)

        def forward(self, ctx, resid, delta, cache):
            T, H = resid.shape
            x = self.norm.add_norm(resid, delta, ctx.workspace.buffer("toy_parallel_normed", T, H, self.dtype))
            mixed = finished(self.mixer.forward(ctx, x, cache)).float()
            fed = finished(self.ffn.forward(ctx, x)).float()
            return (mixed + fed).to(self.dtype)

    return ToyLayerNorm, ParallelBlock


def plain_logits(tensors, d, ids):
    """The same model on a whole sequence: the plain implementation's functions, the toy formulas inline."""
    from tests.plain import qwen3_plain as plain
    w = {k: v.float() for k, v in tensors.items()}
    H, nq, nkv, hd = d["hidden_size"], d["heads"], d["kv_heads"], d["head_dim"]
    T = len(ids)
    cos, sin = plain.rope_tables(d["max_positions"], hd, d["theta"])

    def layer_norm(x, name):
        mean = x.mean(-1, keepdim=True)
        var = ((x - mean) ** 2).mean(-1, keepdim=True)
        return (x - mean) / torch.sqrt(var + d["eps"]) * w[name + ".g"] + w[name + ".b"]

    x = w["emb"][torch.tensor(ids)]
    for i in range(d["layers"]):
        h = layer_norm(x, f"l{i}.n")
        q = plain.apply_rope(plain.linear(h, w[f"l{i}.q"]).view(T, nq, hd), range(T), cos, sin, hd)
        k = plain.apply_rope(plain.linear(h, w[f"l{i}.k"]).view(T, nkv, hd), range(T), cos, sin, hd)
        v = plain.linear(h, w[f"l{i}.v"]).view(T, nkv, hd)
        o = plain.causal_attention(q, k, v, d["scale"]).reshape(T, nq * hd)
        x = x + plain.linear(o, w[f"l{i}.o"]) + plain.swiglu_mlp(h, w[f"l{i}.g"], w[f"l{i}.u"], w[f"l{i}.d"])
    return plain.linear(layer_norm(x, "norm"), w["emb"])


def test_a_layer_norm_and_a_parallel_block_register_build_and_step():
    from llmgen_b200.engine.api import require_cuda
    from llmgen_b200.engine.executor import EngineLimits, Executor, StepEntry
    from llmgen_b200.engine.model import DecoderModel
    from llmgen_b200.parts.registry import model_weight_decls, register_block, register_norm
    from llmgen_b200.parts.spec import AttentionSpec, GatedMLPSpec, ModelSpec, RopeSpec, default_run_order
    from llmgen_b200.registry import config_from_dict, register_architecture, unregister_architecture
    from llmgen_b200.weights import random_tensors, weights_from_dict

    norm_cls, block_cls = make_parts()
    register_norm("toy_layernorm", norm_cls)
    register_block("toy_parallel", block_cls)

    class ToyConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, data, where="config.json"):
            return cls(data)

    def build_spec(cfg):
        d = cfg.d
        H = d["hidden_size"]
        rope = RopeSpec(rotary_dim=d["head_dim"], theta=d["theta"], max_positions=d["max_positions"])
        layers = tuple(ParallelBlockSpec(
            norm=ToyLayerNormSpec(H, d["eps"], f"l{i}.n.g", f"l{i}.n.b"),
            mixer=AttentionSpec(H, d["heads"], d["kv_heads"], d["head_dim"], d["scale"], f"l{i}.q", f"l{i}.k", f"l{i}.v",
                                f"l{i}.o", position=rope),
            ffn=GatedMLPSpec(H, d["ffn"], f"l{i}.g", f"l{i}.u", f"l{i}.d")) for i in range(d["layers"]))
        return ModelSpec(architecture="ToyParallelForCausalLM", vocab_size=d["vocab"], hidden_size=H, embedding="emb",
                         layers=layers, run_order=default_run_order(d["layers"]),
                         final_norm=ToyLayerNormSpec(H, d["eps"], "norm.g", "norm.b"), lm_head="emb",
                         max_positions=d["max_positions"])

    register_architecture("ToyParallelForCausalLM", ToyConfig, build_spec)
    try:
        d = {"architectures": ["ToyParallelForCausalLM"], "hidden_size": 80, "heads": 4, "kv_heads": 2, "head_dim": 32,
             "theta": 3000.0, "scale": 0.19, "max_positions": 128, "eps": 3e-5, "ffn": 112, "layers": 2, "vocab": 97}
        arch, cfg = config_from_dict(d)
        spec = arch.build_spec(cfg)
        decls = model_weight_decls(spec)
        assert {"l0.n.g", "l0.n.b", "norm.b"} <= {x.name for x in decls}
        tensors = random_tensors(decls, 31, 0.12, 0.1, torch.float32)
        for name in tensors:                       # biases are declared plain vectors (zeros at random init): give them values
            if name.endswith(".b"):
                tensors[name] = 0.1 * torch.randn(tensors[name].shape, generator=torch.Generator().manual_seed(len(name)))
        model = DecoderModel(spec, weights_from_dict(tensors, decls), torch.float32, require_cuda())
        ex = Executor(model, EngineLimits(max_num_seqs=2, max_model_len=64, max_step_tokens=64, page_size=16, num_pages=7),
                      eager=True)
        gen = torch.Generator().manual_seed(6)
        ids_a = torch.randint(0, d["vocab"], (41,), generator=gen).tolist()
        ids_b = torch.randint(0, d["vocab"], (19,), generator=gen).tolist()
        ref_a, ref_b = plain_logits(tensors, d, ids_a), plain_logits(tensors, d, ids_b)
        assert ex.admit("a") and ex.reserve("a", 0, len(ids_a))
        assert ex.admit("b") and ex.reserve("b", 0, len(ids_b))
        got_a = [ex.step([StepEntry("a", ids_a[:17], 0, list(range(17)))]).logits.cpu()]     # crosses a page's edge
        both = ex.step([StepEntry("b", ids_b[:7], 0, list(range(7))), StepEntry("a", ids_a[17:19], 17, [0, 1])]).logits.cpu()
        got_b = [both[:7]]
        got_a.append(both[7:])
        pos_a, pos_b = 19, 7
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
        # the bias and the mean matter: an RMS norm with the same gains would give other logits
        from tests.plain import qwen3_plain as plain
        x = torch.randn(3, d["hidden_size"]) + 0.5
        w = tensors["l0.n.g"].float()
        ln = torch.nn.functional.layer_norm(x, (d["hidden_size"],), w, tensors["l0.n.b"].float(), d["eps"])
        assert float((plain.rmsnorm(x, w, d["eps"]) - ln).abs().max()) > 0.05
    finally:
        unregister_architecture("ToyParallelForCausalLM")
