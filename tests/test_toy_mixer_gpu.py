"""A mixer with state of its own, defined here, is registered, built and stepped without a
change to the framework's files: a new spec, a runtime class, a registry entry, and an
architecture whose layers alternate it with attention."""
from dataclasses import dataclass

import pytest
import torch

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class DecaySpec:
    """y[t] = (decay * state + x[t]) W^T, state carried per request; a running mean in disguise."""
    hidden_size: int
    decay: float
    proj: str
    kind: str = "toy_decay"


def make_toy():
    from llmgen_b200.parts.base import Mixer, StateRequest
    from llmgen_b200.parts.spec import WeightDecl

    class DecayMixer(Mixer):
        @staticmethod
        def weight_decls(spec):
            return [WeightDecl(spec.proj, (spec.hidden_size, spec.hidden_size))]

        @staticmethod
        def kernel_modules(spec):
            return ()

        def __init__(self, spec, weights, dtype, device):
            self.spec, self.dtype = spec, dtype
            self.w = weights.device_tensor(spec.proj, dtype, device)

        def state_request(self):
            return StateRequest((self.spec.hidden_size,), torch.float32)

        def forward(self, ctx, x, cache):
            out = torch.empty_like(x)
            t = 0
            for s, n in enumerate(ctx.q_lens):                 # host view of the batch
                slot = int(ctx.state_slots[s].item())
                state = cache.state[slot]
                for i in range(n):
                    state.mul_(self.spec.decay).add_(x[t + i].float())
                    out[t + i] = (state.to(self.dtype) @ self.w.t())
                t += n
            return out

    return DecayMixer


def plain_toy_logits(tensors, cfg, ids):
    """The same model, whole sequence, no state carried: plain torch on the CPU."""
    from tests.plain import qwen3_plain as plain
    w = {k: v.float() for k, v in tensors.items()}
    x = w["emb"][torch.tensor(ids)]
    H = cfg["hidden_size"]
    for i in range(cfg["layers"]):
        h = plain.rmsnorm(x, w[f"l{i}.n1"], 1e-6)
        state = torch.zeros(H)
        mixed = torch.zeros_like(h)
        for t in range(len(ids)):
            state = state * cfg["decay"] + h[t]
            mixed[t] = state @ w[f"l{i}.mix"].t()
        x1 = x + mixed
        h2 = plain.rmsnorm(x1, w[f"l{i}.n2"], 1e-6)
        x = x1 + plain.swiglu_mlp(h2, w[f"l{i}.g"], w[f"l{i}.u"], w[f"l{i}.d"])
    return plain.linear(plain.rmsnorm(x, w["norm"], 1e-6), w["emb"])


def test_toy_mixer_with_state_registers_builds_and_steps():
    from llmgen_b200.engine.api import require_cuda
    from llmgen_b200.engine.executor import EngineLimits, Executor, StepEntry
    from llmgen_b200.engine.model import DecoderModel
    from llmgen_b200.parts.registry import model_weight_decls, register_mixer
    from llmgen_b200.parts.spec import GatedMLPSpec, ModelSpec, PreNormBlockSpec, RMSNormSpec, default_run_order
    from llmgen_b200.registry import config_from_dict, register_architecture, unregister_architecture
    from llmgen_b200.weights import random_tensors, weights_from_dict

    register_mixer("toy_decay", make_toy())

    class ToyConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, data, where="config.json"):
            return cls(data)

    def build_spec(cfg):
        d = cfg.d
        H = d["hidden_size"]
        layers = tuple(PreNormBlockSpec(
            mixer_norm=RMSNormSpec(H, 1e-6, f"l{i}.n1"), mixer=DecaySpec(H, d["decay"], f"l{i}.mix"),
            ffn_norm=RMSNormSpec(H, 1e-6, f"l{i}.n2"), ffn=GatedMLPSpec(H, d["ffn"], f"l{i}.g", f"l{i}.u", f"l{i}.d"))
            for i in range(d["layers"]))
        return ModelSpec(architecture="ToyForCausalLM", vocab_size=d["vocab"], hidden_size=H, embedding="emb",
                         layers=layers, run_order=default_run_order(d["layers"]),
                         final_norm=RMSNormSpec(H, 1e-6, "norm"), lm_head="emb", max_positions=512)

    register_architecture("ToyForCausalLM", ToyConfig, build_spec)
    try:
        cfg_dict = {"architectures": ["ToyForCausalLM"], "hidden_size": 40, "ffn": 56, "layers": 2, "vocab": 90, "decay": 0.8}
        arch, cfg = config_from_dict(cfg_dict)
        spec = arch.build_spec(cfg)
        decls = model_weight_decls(spec)
        tensors = random_tensors(decls, 11, 0.1, 0.1, torch.float32)
        model = DecoderModel(spec, weights_from_dict(tensors, decls), torch.float32, require_cuda())
        ex = Executor(model, EngineLimits(max_num_seqs=3, max_model_len=64, max_step_tokens=64, page_size=16, num_pages=8),
                      eager=True)
        assert set(ex.storage.state) == {0, 1} and ex.storage.state[0].shape == (3, 40) and not ex.storage.kv
        ids_a = [3, 14, 15, 9, 26, 5, 35, 8, 9, 7, 9, 3, 2]
        ids_b = [80, 1, 2, 60, 61]
        ref_a, ref_b = plain_toy_logits(tensors, cfg_dict, ids_a), plain_toy_logits(tensors, cfg_dict, ids_b)
        assert ex.admit("a") and ex.reserve("a", 0, len(ids_a))
        got_a = [ex.step([StepEntry("a", ids_a[:4], 0, [0, 1, 2, 3])]).logits.cpu()]
        assert ex.admit("b") and ex.reserve("b", 0, len(ids_b))
        both = ex.step([StepEntry("a", ids_a[4:6], 4, [0, 1]), StepEntry("b", ids_b[:3], 0, [0, 1, 2])]).logits.cpu()
        got_a.append(both[:2])
        got_b = [both[2:]]
        both = ex.step([StepEntry("b", ids_b[3:], 3, [0, 1]), StepEntry("a", ids_a[6:], 6, list(range(7)))]).logits.cpu()
        got_b.append(both[:2])
        got_a.append(both[2:])
        assert float((torch.cat(got_a) - ref_a).abs().max()) < 1e-4
        assert float((torch.cat(got_b) - ref_b).abs().max()) < 1e-4
        # a slot handed to a new request starts from zero state
        ex.release("a")
        assert ex.admit("c") and ex.reserve("c", 0, len(ids_b))
        got_c = ex.step([StepEntry("c", ids_b, 0, list(range(5)))]).logits.cpu()
        assert float((got_c - ref_b).abs().max()) < 1e-4
        # the toy reads the step's lengths on the host and does not say `replay_any_step`: an engine that replays
        # graphs launches this model's steps of portions kernel by kernel all the same
        ex2 = Executor(model, EngineLimits(max_num_seqs=3, max_model_len=64, max_step_tokens=64, page_size=16, num_pages=8))
        assert not ex2.shaped_steps
        assert ex2.admit("d") and ex2.reserve("d", 0, len(ids_b))
        got_d = ex2.step([StepEntry("d", ids_b, 0, list(range(5)))]).logits.cpu()
        assert float((got_d - ref_b).abs().max()) < 1e-4 and ex2.n_shaped_steps == 0
    finally:
        unregister_architecture("ToyForCausalLM")
