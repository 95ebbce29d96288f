"""Each part alone on the GPU against its plain function, built from specs with sizes of its own."""
import math

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.util import manual_context

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (3e-5 if dtype == torch.float32 else 2.5e-2) * scale


def finished(out):
    """A part may hand back the float32 slices of a product cut along K; add them up."""
    from llmgen_b200.kernels.ops import Partials
    return out.sum() if isinstance(out, Partials) else out


def store(tensors, decls):
    from llmgen_b200.weights import weights_from_dict
    return weights_from_dict(tensors, decls)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from llmgen_b200.parts.registry import build_norm, norm_class
    from llmgen_b200.parts.spec import RMSNormSpec
    torch.manual_seed(0)
    spec = RMSNormSpec(dim=88, eps=2e-5, weight="n.weight", weight_offset=0.5)
    w = (1 + 0.1 * torch.randn(88)).to(torch.bfloat16)          # stored bfloat16, kept float32 on the device
    part = build_norm(spec, store({"n.weight": w}, norm_class(spec).weight_decls(spec)), dtype, "cuda")
    assert part.weight.dtype == torch.float32
    resid = torch.randn(5, 88)
    delta = torch.randn(5, 88).to(dtype)
    r = resid.cuda()
    out = torch.empty(5, 88, dtype=dtype, device="cuda")
    part.add_norm(r, delta.cuda(), out)
    ref = plain.rmsnorm(resid + delta.float(), w.float(), 2e-5, 0.5)
    assert float((out.float().cpu() - ref).abs().max()) < tol(dtype, 8)


def test_rope_part_tables():
    from llmgen_b200.parts.registry import build_position
    from llmgen_b200.parts.spec import RopeSpec
    part = build_position(RopeSpec(rotary_dim=48, theta=50000.0, max_positions=300), None, torch.float32, "cuda")
    cos, sin = plain.rope_tables(300, 48, 50000.0)
    assert part.cos.shape == (300, 24) and part.cos.dtype == torch.float32
    assert torch.equal(part.cos.cpu(), cos.float()) and torch.equal(part.sin.cpu(), sin.float())
    again = build_position(RopeSpec(rotary_dim=48, theta=50000.0, max_positions=300), None, torch.bfloat16, "cuda")
    assert again.cos.data_ptr() == part.cos.data_ptr()           # layers with the same spec share tables


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [1, 3, 37])
def test_gated_mlp_part(dtype, T):
    from llmgen_b200.parts.registry import build_feed_forward, feed_forward_class
    from llmgen_b200.parts.spec import GatedMLPSpec
    torch.manual_seed(1)
    H, F = 72, 200
    spec = GatedMLPSpec(H, F, "g", "u", "d")
    w = {"g": torch.randn(F, H) * 0.2, "u": torch.randn(F, H) * 0.2, "d": torch.randn(H, F) * 0.2}
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    part = build_feed_forward(spec, store(w, feed_forward_class(spec).weight_decls(spec)), dtype, "cuda")
    x = torch.randn(T, H).to(dtype)
    ctx = manual_context([T], [0], [[0, 1, 2]], 16, dtype)
    out = finished(part.forward(ctx, x.cuda()))
    ref = plain.swiglu_mlp(x.float(), w["g"].float(), w["u"].float(), w["d"].float())
    assert float((out.float().cpu() - ref).abs().max()) < tol(dtype, 20)


def attention_setup(dtype, nq, nkv, hd, H, window, with_norm=True, rot=None):
    from llmgen_b200.parts.registry import build_mixer, mixer_class
    from llmgen_b200.parts.spec import AttentionSpec, RMSNormSpec, RopeSpec
    torch.manual_seed(2)
    rot = hd if rot is None else rot
    spec = AttentionSpec(hidden_size=H, num_heads=nq, num_kv_heads=nkv, head_dim=hd, scale=1 / math.sqrt(hd),
                         q_proj="q", k_proj="k", v_proj="v", o_proj="o",
                         q_norm=RMSNormSpec(hd, 1e-5, "qn") if with_norm else None,
                         k_norm=RMSNormSpec(hd, 1e-5, "kn") if with_norm else None,
                         position=RopeSpec(rot, 10000.0, 512) if rot else None, window=window)
    w = {"q": torch.randn(nq * hd, H) * 0.3, "k": torch.randn(nkv * hd, H) * 0.3, "v": torch.randn(nkv * hd, H) * 0.3,
         "o": torch.randn(H, nq * hd) * 0.3}
    if with_norm:
        w.update({"qn": 1 + 0.2 * torch.randn(hd), "kn": 1 + 0.2 * torch.randn(hd)})
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    part = build_mixer(spec, store(w, mixer_class(spec).weight_decls(spec)), dtype, "cuda")
    return spec, {k: v.float() for k, v in w.items()}, part


def plain_attention_block(spec, w, x, window, rot):
    T = x.shape[0]
    nq, nkv, hd = spec.num_heads, spec.num_kv_heads, spec.head_dim
    q = plain.linear(x, w["q"]).view(T, nq, hd)
    k = plain.linear(x, w["k"]).view(T, nkv, hd)
    v = plain.linear(x, w["v"]).view(T, nkv, hd)
    if "qn" in w:
        q, k = plain.rmsnorm(q, w["qn"], 1e-5), plain.rmsnorm(k, w["kn"], 1e-5)
    if rot:
        cos, sin = plain.rope_tables(512, rot, 10000.0)
        q = plain.apply_rope(q, range(T), cos, sin, rot)
        k = plain.apply_rope(k, range(T), cos, sin, rot)
    a = plain.causal_attention(q, k, v, spec.scale, window)
    return plain.linear(a.reshape(T, nq * hd), w["o"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,H,window,with_norm,rot", [
    (4, 2, 32, 64, None, True, None), (6, 1, 48, 72, 20, True, None), (2, 2, 64, 40, None, False, 32),
    (8, 8, 16, 128, 5, False, 0)])
def test_attention_part_whole_then_in_portions(dtype, nq, nkv, hd, H, window, with_norm, rot):
    from llmgen_b200.parts.base import LayerCache
    spec, w, part = attention_setup(dtype, nq, nkv, hd, H, window, with_norm, rot)
    req = part.cache_request()
    assert (req.num_kv_heads, req.head_dim, req.window) == (nkv, hd, window or 0)
    assert req.group_kind == ("window" if window else "full")
    T, page = 50, 8
    x = torch.randn(T, H).to(dtype)
    ref = plain_attention_block(spec, w, x.float(), window, hd if rot is None else rot)
    table = [5, 2, 9, 0, 7, 3, 8]
    for cuts in ([T], [13, 1, 1, 20, 2, 13]):
        kc = torch.zeros(10, nkv, page, hd, dtype=dtype, device="cuda")
        vc = torch.zeros_like(kc)
        cache = LayerCache(k=kc, v=vc, group=0, page_size=page, writes=True)
        outs, start = [], 0
        for n in cuts:
            ctx = manual_context([n], [start], [table], page, dtype, mixers=[part])
            outs.append(finished(part.forward(ctx, x[start:start + n].cuda(), cache)).float().cpu().clone())
            start += n
        got = torch.cat(outs)
        assert float((got - ref).abs().max()) < tol(dtype, 30), cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_reading_another_items_cache(dtype):
    """A run item with writes=False projects q only and attends over what the writer stored."""
    from llmgen_b200.parts.base import LayerCache
    spec, w, part = attention_setup(dtype, 4, 2, 32, 64, None)
    T, page = 20, 8
    x = torch.randn(T, 64).to(dtype)
    kc = torch.zeros(4, 2, page, 32, dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    ctx = manual_context([T], [0], [[2, 0, 3]], page, dtype, mixers=[part])
    first = finished(part.forward(ctx, x.cuda(), LayerCache(k=kc, v=vc, group=0, page_size=page, writes=True))).clone()
    k_before = kc.clone()
    second = finished(part.forward(ctx, x.cuda(), LayerCache(k=kc, v=vc, group=0, page_size=page, writes=False)))
    assert torch.equal(kc, k_before)
    assert float((first.float() - second.float()).abs().max()) < tol(dtype, 2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block(dtype):
    from llmgen_b200.engine.api import require_cuda
    from llmgen_b200.parts.base import LayerCache
    from llmgen_b200.parts.registry import block_class, build_block
    from llmgen_b200.registry import config_from_dict
    from llmgen_b200.weights import random_tensors
    from tests.util import TINY_C
    require_cuda()
    arch, cfg = config_from_dict(TINY_C)
    spec = arch.build_spec(cfg)
    layer = spec.layers[1]                                  # a windowed layer
    decls = block_class(layer).weight_decls(layer)
    tensors = random_tensors(decls, 3, 0.08, 0.2, torch.bfloat16)
    block = build_block(layer, store(tensors, decls), dtype, "cuda")
    T, H, page = 70, cfg.hidden_size, 16
    torch.manual_seed(3)
    x = torch.randn(T, H)
    prev = (torch.randn(T, H) * 0.5).to(dtype)              # the previous block's output, not yet added
    resid = x.cuda()
    kc = torch.zeros(6, cfg.num_key_value_heads, page, cfg.head_dim, dtype=dtype, device="cuda")
    ctx = manual_context([T], [0], [[4, 1, 0, 5, 2]], page, dtype, mixers=[block.mixer])
    delta = finished(block.forward(ctx, resid, prev.cuda(), LayerCache(k=kc, v=torch.zeros_like(kc), group=0, page_size=page)))
    got = resid.cpu() + delta.float().cpu()
    # plain: the same layer on x + prev
    w = {k: v.float() for k, v in tensors.items()}
    m = object.__new__(plain.PlainQwen3)
    m.round_to = None
    m.w, m.nq, m.nkv, m.hd, m.eps = w, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps
    m.scale, m.windows = 1 / math.sqrt(cfg.head_dim), [None, cfg.sliding_window]
    m.cos, m.sin = plain.rope_tables(cfg.max_position_embeddings, cfg.head_dim, cfg.rope_theta)
    ref = m.layer(1, x + prev.float(), list(range(T)))
    assert float((got - ref).abs().max()) < tol(dtype, 40)
