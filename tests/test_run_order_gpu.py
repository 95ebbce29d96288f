"""The order in which layers run is data, and so are two numbers around the layers (a scale on the embedding's rows, a
bound on the logits).  An architecture defined here, from the framework's own parts, has a run list that names one
layer twice (each pass with a cache of its own) and lets a later layer attend over the keys and values that an earlier
item stored (it projects q only).  It is registered, built and stepped through the engine without a change to the
framework's files, and compared with a plain composition of the parts' plain functions: whole prompts, portions of
changing size beside another request, and single tokens, in float32 and bfloat16, launched and replayed."""
import dataclasses
import math

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.util import FP32_TOL

pytestmark = pytest.mark.gpu

CFG = {"architectures": ["LoopedForCausalLM"], "hidden_size": 96, "intermediate_size": 144, "num_hidden_layers": 3,
       "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 211, "rms_norm_eps": 1e-5,
       "rope_theta": 50000.0, "max_position_embeddings": 256, "tie_word_embeddings": True, "hidden_act": "silu"}
# (layer, cache, writes): layer 1 runs twice with caches 1 and 2; layer 2 then reads cache 1, what the first pass of
# layer 1 stored, and keeps no keys of its own
RUN = [(0, 0, True), (1, 1, True), (1, 2, True), (2, 1, False)]


def plain_logits(w, ids, round_to=None):
    """The run list above, part by part, on one whole sequence (each function cites the reference in tests/plain)."""
    c = CFG
    nq, nkv, hd, eps = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"], c["rms_norm_eps"]
    r = (lambda t: t) if round_to is None else (lambda t: t.to(round_to).to(torch.float32))
    cos, sin = plain.rope_tables(c["max_position_embeddings"], hd, c["rope_theta"])
    positions = list(range(len(ids)))
    T = len(ids)
    x = plain.embedding(ids, w["model.embed_tokens.weight"])
    stored = {}
    for layer, cache, writes in RUN:
        p = f"model.layers.{layer}."
        h = r(plain.rmsnorm(x, w[p + "input_layernorm.weight"], eps))
        q = r(plain.linear(h, w[p + "self_attn.q_proj.weight"])).view(T, nq, hd)
        q = r(plain.apply_rope(r(plain.rmsnorm(q, w[p + "self_attn.q_norm.weight"], eps)), positions, cos, sin, hd))
        if writes:
            k = r(plain.linear(h, w[p + "self_attn.k_proj.weight"])).view(T, nkv, hd)
            v = r(plain.linear(h, w[p + "self_attn.v_proj.weight"])).view(T, nkv, hd)
            k = r(plain.apply_rope(r(plain.rmsnorm(k, w[p + "self_attn.k_norm.weight"], eps)), positions, cos, sin, hd))
            stored[cache] = (k, v)
        k, v = stored[cache]
        a = r(plain.causal_attention(q, k, v, 1.0 / math.sqrt(hd), None)).reshape(T, nq * hd)
        x1 = r(x + r(plain.linear(a, w[p + "self_attn.o_proj.weight"])))
        h2 = r(plain.rmsnorm(x1, w[p + "post_attention_layernorm.weight"], eps))
        g = r(plain.linear(h2, w[p + "mlp.gate_proj.weight"]))
        u = r(plain.linear(h2, w[p + "mlp.up_proj.weight"]))
        m = r(plain.linear(r(r(g / (1.0 + torch.exp(-g))) * u), w[p + "mlp.down_proj.weight"]))
        x = r(x1 + m)
    x = r(plain.rmsnorm(x, w["model.norm.weight"], eps))
    return r(plain.linear(x, w["model.embed_tokens.weight"]))


@pytest.fixture(scope="module")
def looped():
    from llmgen_b200.config.qwen3 import Qwen3Config
    from llmgen_b200.models.qwen3 import build_qwen3_spec
    from llmgen_b200.parts.registry import model_weight_decls
    from llmgen_b200.parts.spec import RunItem
    from llmgen_b200.registry import config_from_dict, register_architecture, unregister_architecture
    from llmgen_b200.weights import random_tensors

    def build_spec(cfg):
        spec = build_qwen3_spec(cfg)
        return dataclasses.replace(spec, architecture="LoopedForCausalLM",
                                   run_order=tuple(RunItem(layer=l, cache=c, writes_cache=wr) for l, c, wr in RUN))

    register_architecture("LoopedForCausalLM", Qwen3Config, build_spec)
    try:
        arch, cfg = config_from_dict(CFG)
        spec = arch.build_spec(cfg)
        decls = model_weight_decls(spec)
        tensors = random_tensors(decls, 23, 0.08, 0.1, torch.float32)
        yield spec, decls, tensors
    finally:
        unregister_architecture("LoopedForCausalLM")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
@pytest.mark.parametrize("eager", [True, False], ids=["launched", "replayed"])
def test_a_layer_run_twice_and_a_layer_reading_an_earlier_items_cache(looped, dtype, eager):
    from llmgen_b200.engine.api import require_cuda
    from llmgen_b200.engine.executor import EngineLimits, Executor, StepEntry
    from llmgen_b200.engine.model import DecoderModel
    from llmgen_b200.weights import weights_from_dict

    spec, decls, tensors = looped
    bf = dtype == torch.bfloat16
    w = {k: (v.to(torch.bfloat16).float() if bf and v.dim() >= 2 else v.float()) for k, v in tensors.items()}
    model = DecoderModel(spec, weights_from_dict(tensors, decls), dtype, require_cuda())
    ex = Executor(model, EngineLimits(max_num_seqs=4, max_model_len=128, max_step_tokens=128, page_size=16, num_pages=24),
                  eager=eager)
    # three caches are kept (0, 1, 2), none for the item that only reads
    assert sorted(ex.storage.kv) == [0, 1, 2]
    g = torch.Generator().manual_seed(5)
    ids_a = torch.randint(0, CFG["vocab_size"], (70,), generator=g).tolist()
    ids_b = torch.randint(0, CFG["vocab_size"], (37,), generator=g).tolist()
    ref_a, ref_b = plain_logits(w, ids_a, torch.bfloat16 if bf else None), plain_logits(w, ids_b, torch.bfloat16 if bf else None)
    if bf:      # what bfloat16 arithmetic costs on this model: the rounded plain run against the exact one
        noise = float((ref_a - plain_logits({k: v.float() for k, v in tensors.items()}, ids_a)).abs().max())
        bound = 3 * max(noise, 1e-3)
    else:
        bound = FP32_TOL * max(1.0, float(ref_a.abs().max()))
    # a: 33 tokens at once, then portions of changing size beside b's portions, then single tokens
    assert ex.admit("a") and ex.reserve("a", 0, len(ids_a))
    got_a = [ex.step([StepEntry("a", ids_a[:33], 0, list(range(33)))]).logits.cpu()]
    assert ex.admit("b") and ex.reserve("b", 0, len(ids_b))
    cuts_a, cuts_b = [33, 35, 48, 50, 60], [0, 20, 22, 37, 37]
    for i in range(4):
        entries, na = [], cuts_a[i + 1] - cuts_a[i]
        entries.append(StepEntry("a", ids_a[cuts_a[i]:cuts_a[i + 1]], cuts_a[i], list(range(na))))
        nb = cuts_b[i + 1] - cuts_b[i]
        if nb:
            entries.append(StepEntry("b", ids_b[cuts_b[i]:cuts_b[i + 1]], cuts_b[i], list(range(nb))))
        out = ex.step(entries).logits.cpu()
        got_a.append(out[:na])
        if nb:
            ref = ref_b[cuts_b[i]:cuts_b[i + 1]]
            assert float((out[na:] - ref).abs().max()) < bound
    ex.release("b")
    for t in range(60, len(ids_a)):
        got_a.append(ex.step([StepEntry("a", [ids_a[t]], t, [0])]).logits.cpu())
    got = torch.cat(got_a)
    assert got.shape == ref_a.shape
    assert float((got - ref_a).abs().max()) < bound
    if not bf:
        assert torch.equal(got.argmax(-1), ref_a.argmax(-1))
    ex.release("a")
    assert ex.cache.all_free()
    if not eager:
        assert ex.n_shaped_steps > 0 or not ex.shaped_steps


def test_an_embedding_scale_and_a_bound_on_the_logits_are_data_too(looped):
    """`ModelSpec.embedding_scale` and `ModelSpec.logit_cap`: rows enter the residual multiplied by the scale, logits
    leave as cap * tanh(logits / cap); the default values change nothing (every other test runs with them)."""
    from llmgen_b200.engine.api import require_cuda
    from llmgen_b200.engine.executor import EngineLimits, Executor, StepEntry
    from llmgen_b200.engine.model import DecoderModel
    from llmgen_b200.parts.spec import default_run_order
    from llmgen_b200.weights import weights_from_dict

    spec, decls, tensors = looped
    scale, cap = 2.5, 0.75
    spec = dataclasses.replace(spec, run_order=default_run_order(len(spec.layers)), embedding_scale=scale, logit_cap=cap)
    model = DecoderModel(spec, weights_from_dict(tensors, decls), torch.float32, require_cuda())
    ex = Executor(model, EngineLimits(max_num_seqs=2, max_model_len=64, max_step_tokens=64, page_size=16, num_pages=6), eager=True)
    ids = torch.randint(0, CFG["vocab_size"], (29,), generator=torch.Generator().manual_seed(8)).tolist()
    # plain: the default order, the table scaled, the logits bounded
    w = {k: v.float() for k, v in tensors.items()}
    w_scaled = dict(w)
    w_scaled["model.embed_tokens.weight"] = w["model.embed_tokens.weight"] * scale
    global RUN
    saved, RUN = RUN, [(i, i, True) for i in range(CFG["num_hidden_layers"])]
    try:
        hidden_ref = plain_logits(w_scaled, ids)            # its last product used the scaled table: undo that below
    finally:
        RUN = saved
    ref = cap * torch.tanh(hidden_ref / scale / cap)
    assert ex.admit("a") and ex.reserve("a", 0, len(ids))
    got = [ex.step([StepEntry("a", ids[:20], 0, list(range(20)))]).logits.cpu()]
    for t in range(20, len(ids)):
        got.append(ex.step([StepEntry("a", [ids[t]], t, [0])]).logits.cpu())
    got = torch.cat(got)
    assert float(got.abs().max()) <= cap and float(hidden_ref.abs().max()) / scale > cap        # the bound bites
    assert float((got - ref).abs().max()) < FP32_TOL
