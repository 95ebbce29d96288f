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
