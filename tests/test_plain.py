"""The plain implementation against the reference's own fixtures, and against itself."""
import json
import os
import tempfile

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.util import TINY, make_folder, random_ids

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_fixtures.json")


def _fixtures():
    with open(GOLDEN, "r", encoding="utf-8") as f:
        return json.load(f)


def test_linear_matches_reference_fixture():
    c = _fixtures()["linear_case"]
    x, w, y = (torch.tensor(c[k], dtype=torch.float32) for k in ("x", "weight", "y"))
    got = plain.linear(x, w)
    assert got.shape == (c["seq_len"], c["out_dim"])
    assert torch.allclose(got, y, rtol=1e-3, atol=1e-3)   # the reference's own tolerance


def test_rmsnorm_matches_reference_fixture():
    c = _fixtures()["norm_case"]
    x, w, y = (torch.tensor(c[k], dtype=torch.float32) for k in ("x", "weight", "y"))
    got = plain.rmsnorm(x, w, c["eps"])
    assert torch.allclose(got, y, rtol=1e-3, atol=1e-3)
    assert float((got - y).abs().max()) < 1e-5


def test_rope_is_a_rotation_and_position_zero_is_identity():
    cos, sin = plain.rope_tables(64, 16, 10000.0)
    x = torch.randn(5, 3, 16, dtype=torch.float64)
    y = plain.apply_rope(x, [0, 1, 7, 30, 63], cos, sin, 16)
    assert torch.allclose(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    # relative property: <rope(q, m), rope(k, n)> depends on m - n only
    q, k = torch.randn(1, 1, 16, dtype=torch.float64), torch.randn(1, 1, 16, dtype=torch.float64)
    d1 = (plain.apply_rope(q, [9], cos, sin, 16) * plain.apply_rope(k, [4], cos, sin, 16)).sum()
    d2 = (plain.apply_rope(q, [25], cos, sin, 16) * plain.apply_rope(k, [20], cos, sin, 16)).sum()
    assert abs(float(d1 - d2)) < 1e-9


def test_partial_rotary_leaves_the_tail_untouched():
    cos, sin = plain.rope_tables(16, 8, 100.0)
    x = torch.randn(2, 1, 12)
    y = plain.apply_rope(x, [3, 5], cos, sin, 8)
    assert torch.equal(y[..., 8:], x[..., 8:])


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    T, nq, nkv, hd = 12, 4, 2, 8
    q, k, v = torch.randn(T, nq, hd), torch.randn(T, nkv, hd), torch.randn(T, nkv, hd)
    out = plain.causal_attention(q, k, v, 0.3)
    # first query sees only key 0
    assert torch.allclose(out[0, 0], v[0, 0], atol=1e-6)
    assert torch.allclose(out[0, 3], v[0, 1], atol=1e-6)
    # a later key does not change earlier outputs
    k2, v2 = k.clone(), v.clone()
    k2[8:] += 5.0
    v2[8:] -= 3.0
    out2 = plain.causal_attention(q, k2, v2, 0.3)
    assert torch.allclose(out2[:8], out[:8], atol=1e-6)
    # window 1: every query sees only its own key
    w1 = plain.causal_attention(q, k, v, 0.3, window=1)
    assert torch.allclose(w1[:, 0], v[:, 0], atol=1e-6)
    # window W: changing key t-W does not change query t
    w3 = plain.causal_attention(q, k, v, 0.3, window=3)
    k3 = k.clone()
    k3[5] += 100.0
    w3b = plain.causal_attention(q, k3, v, 0.3, window=3)
    assert torch.allclose(w3b[8:], w3[8:], atol=1e-6) and not torch.allclose(w3b[7], w3[7], atol=1e-3)


def test_sampler_greedy_ties_and_reproducible():
    logits = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert plain.gumbel_sample(logits, 0.0, 1, 0) == 1
    a = plain.gumbel_sample(logits, 0.7, 1234, 3)
    assert a == plain.gumbel_sample(logits, 0.7, 1234, 3)
    draws = [plain.gumbel_sample(torch.tensor([0.0, 0.0]), 1.0, s, 0) for s in range(200)]
    assert 60 < sum(draws) < 140
    assert plain.splitmix64(0) == 0xE220A8397B1DCDAF


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_equals_prefixes(name):
    """Logits at position t depend on tokens 0..t only (no cache to get wrong here)."""
    with tempfile.TemporaryDirectory() as tmp:
        m = plain.PlainQwen3(make_folder(tmp, name))
        ids = random_ids(60, TINY[name][0]["vocab_size"], 3)
        whole = m.logits(ids)
        for cut in (1, 17, 45):
            assert torch.allclose(m.logits(ids[:cut])[-1], whole[cut - 1], atol=2e-6)
        assert whole.dtype == torch.float32 and whole.shape == (60, TINY[name][0]["vocab_size"])


def test_float64_agrees_with_float32():
    with tempfile.TemporaryDirectory() as tmp:
        path = make_folder(tmp, "B")
        ids = random_ids(50, 384, 4)
        a = plain.PlainQwen3(path, torch.float32).logits(ids)
        b = plain.PlainQwen3(path, torch.float64).logits(ids)
        assert float((a.double() - b).abs().max()) < 2e-5


# ------------------------------------------------------------------ the reference's own kernels as the second anchor
KERNEL_GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_kernel_fixtures.json")


def _kernel_fixtures():
    with open(KERNEL_GOLDEN, "r", encoding="utf-8") as f:
        return json.load(f)


def _bf16(text, *shape):
    """A bfloat16 array stored as base64 of its bytes, widened to float32 (exactly)."""
    import base64
    import numpy as np
    raw = np.frombuffer(base64.b64decode(text), dtype=np.int16).copy()
    return torch.from_numpy(raw).view(torch.bfloat16).float().reshape(*shape)


def _ulp_bf16(ref: torch.Tensor) -> torch.Tensor:
    """One unit in the last place of bfloat16 at each value's magnitude (8 bits of mantissa)."""
    return torch.clamp(ref.abs(), min=2.0 ** -20) * 2.0 ** -7


def test_head_norm_matches_the_references_kernel():
    """rmsnorm over each head of 128 with one shared gain vector (norm/norm_final.cu:28-45).  The kernel rounds
    x * rstd to bfloat16 before the gain and the product again on store: two roundings against the formula."""
    c = _kernel_fixtures()
    f = c["head_norm"]
    x, y = _bf16(f["x"], *f["shape"]), _bf16(f["y"], *f["shape"])
    got = plain.rmsnorm(x, torch.tensor(f["gain"]), f["eps"])
    assert float(((got - y).abs() / _ulp_bf16(y)).max()) <= 2.0


def test_rope_pairing_and_angles_match_the_references_kernel():
    """Half-split pairs (i, i + 64) turned by positions[t] / theta^(2i/128) (rope/rope_v1.cu:11-45): an interleaved
    pairing, a wrong sign or angles by row instead of by position would be off by whole values, not by rounding."""
    c = _kernel_fixtures()
    f = c["rope"]
    x, y = _bf16(f["x"], *f["shape"]), _bf16(f["y"], *f["shape"])
    cos, sin = plain.rope_tables(64, c["hd"], f["theta"])
    got = plain.apply_rope(x, f["positions"], cos, sin, c["hd"])
    assert float(((got - y).abs() / _ulp_bf16(y)).max()) <= 1.0
    assert float((x[1:] - y[1:]).abs().max()) > 0.5            # the fixture does turn its values


def test_store_kv_layout_matches_the_references_kernel():
    """A slot is (block, place in block); a block holds [kv head][place][head_dim]; slot -1 writes nothing
    (attention/attention.cu:18-33)."""
    c = _kernel_fixtures()
    f, bs = c["store_kv"], c["block_size"]
    k = _bf16(f["k"], 3, c["nkv"], c["hd"])
    expected = sorted([s // bs, h, s % bs] for s in f["slots"] if s >= 0 for h in range(c["nkv"]))
    assert sorted(f["written"]) == expected
    assert torch.equal(_bf16(f["row_2_5_head_1"], c["hd"]), k[0, 1])          # token 0 went to slot 2 * 16 + 5


def test_attention_of_a_chunk_tail_matches_the_references_kernels():
    """The last q_len positions of a longer context over shuffled pages: query i of the chunk sees keys
    0 .. ctx - q_len + i, query head h reads kv head h // 2 (attention/attention.cu:300-466); and the last
    position alone through the split decode kernel and its merge (attention.cu:51-207)."""
    c = _kernel_fixtures()
    f, nq, nkv, hd = c["prefill"], c["nq"], c["nkv"], c["hd"]
    ctx, q_len = f["ctx"], f["q_len"]
    q = _bf16(f["q"], q_len, nq, hd)
    k, v = _bf16(f["k_seq"], ctx, nkv, hd), _bf16(f["v_seq"], ctx, nkv, hd)
    out = _bf16(f["out"], q_len, nq, hd)
    # the plain function takes whole sequences: pad the queries in front, keep the chunk's rows
    q_full = torch.zeros(ctx, nq, hd)
    q_full[ctx - q_len:] = q
    got = plain.causal_attention(q_full, k, v, 1.0 / hd ** 0.5)[ctx - q_len:]
    assert float((got - out).abs().max()) < 2e-2               # the reference's own tolerance for this kernel
    assert float((got - out).abs().mean()) < 2e-3
    one = _bf16(c["decode"]["out"], 1, nq, hd)
    assert float((got[-1:] - one).abs().max()) < 2e-2
    # a wrong group mapping (head h on kv head h % nkv) or a causal offset of the chunk alone is far outside
    wrong = plain.causal_attention(q_full, k.flip(1), v.flip(1), 1.0 / hd ** 0.5)[ctx - q_len:]
    assert float((wrong - out).abs().max()) > 0.2
    alone = plain.causal_attention(q, k[:q_len], v[:q_len], 1.0 / hd ** 0.5)
    assert float((alone - out).abs().max()) > 0.2


def test_sampler_matches_the_references_kernel():
    """argmax with ties to the smaller id, and the Gumbel-max draw from splitmix64(seed ^ (row << 40)) + id
    (sample/sample.cu:33-77)."""
    f = _kernel_fixtures()["sample"]
    logits = _bf16(f["logits"], 3, f["V"])
    assert f["ids"][0] == 40                                    # ids 40 and 250 tie: the smaller wins
    for row, temp in enumerate(f["temps"]):
        if temp <= 0:
            assert plain.gumbel_sample(logits[row], temp, f["seed"], row) == f["ids"][row]
        else:
            scores = plain.gumbel_scores(logits[row], temp, f["seed"], row)
            top = scores.topk(2)
            # the kernel computes logit * (1 / T) with the fast log: equal unless the two best are that close
            assert f["ids"][row] == int(top.indices[0]) or float(top.values[0] - top.values[1]) < 1e-3
