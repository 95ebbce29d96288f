"""The whole model at the Qwen3-0.6B shape (28 layers, hidden 1,024, 16 query heads on 8 kv heads of 128,
intermediate 3,072, vocabulary 151,936, tied embeddings, random weights of seed 2 stored as bfloat16) in true
float32 against the plain implementation, in the four ways of cutting the work: each request whole; most of
it in one step and the last 32 tokens one by one; portions of changing size; and mixed, four live requests
with so few pages that they are used again.  Then once in bfloat16 against the model's own bound.

The reference checks its whole model by the ids it generates from the real 0.6B file (src/llmgen.zig:171-176,
Makefile:37-39); there is no such file here, so the check is against the plain implementation on random weights.
"""
import random
import tempfile

import pytest
import torch

from tests.test_replay_gpu import mixed_trace
from tests.util import FP32_TOL, Driver, forget_plain_models, logits_close, plain_model, random_ids, reference

pytestmark = pytest.mark.gpu

SHAPE_06B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 151936, "hidden_size": 1024, "intermediate_size": 3072, "num_hidden_layers": 28,
    "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 4096,
    "tie_word_embeddings": True, "hidden_act": "silu",
}
LENGTHS = [150, 100, 230, 120, 64, 181]
PAGE = 16


class Case:
    def __init__(self, tmp):
        from llmgen_b200.engine.api import load_model, write_random_model
        self.path = write_random_model(tmp + "/shape_06b", SHAPE_06B, 2, None, None, "bfloat16")
        self.reqs = [random_ids(n, SHAPE_06B["vocab_size"], 700 + i) for i, n in enumerate(LENGTHS)]
        plain = plain_model(self.path)
        self.refs = [plain.logits(r) for r in self.reqs]
        forget_plain_models()                       # 2.4 GB of float32 weights on the host
        self.model = load_model(self.path, "float32")

    def driver(self, pool_tokens):
        return Driver(self.path, "float32", pool_tokens, PAGE, model=self.model)


@pytest.fixture(scope="module")
def case():
    with tempfile.TemporaryDirectory() as tmp:
        yield Case(tmp)


def close32(got, ref):
    """Within 1e-4 of the plain logits, and the same greedy id wherever the plain logits themselves decide it
    by more than twice that."""
    worst = logits_close(got, ref, "float32")
    differ = (got.argmax(-1) != ref.argmax(-1)).nonzero().flatten().tolist()
    for row in differ:
        top = ref[row].topk(2).values
        assert float(top[0] - top[1]) <= 2 * FP32_TOL, f"row {row}: greedy id differs although the plain logits are {float(top[0] - top[1]):.2e} apart"
    return worst


def test_whole(case):
    d = case.driver(256)
    for ids, ref in zip(case.reqs, case.refs):
        close32(d.step([("r", ids, range(len(ids)))], end=["r"]), ref)
    assert d.executor.cache.all_free()


def test_last_32_one_by_one(case):
    d = case.driver(256)
    for ids, ref in list(zip(case.reqs, case.refs))[:3]:
        n = len(ids)
        head = n - 32
        got = [d.step([("r", ids[:head], [head - 1])])]
        for t in range(head, n):
            got.append(d.step([("r", ids[t:t + 1], [0])], end=["r"] if t == n - 1 else []))
        close32(torch.cat(got), ref[head - 1:])


def test_portions_of_changing_size(case):
    d = case.driver(256)
    rng = random.Random(5)
    for ids, ref in list(zip(case.reqs, case.refs))[:3]:
        n, p, got = len(ids), 0, []
        sizes = [7, 2, 16, 3]
        while p < n:
            c = sizes.pop(0) if sizes else rng.choice([2, 2, 5, 11, 17, 31, 64])
            c = min(c, n - p)
            if n - p - c == 1:
                c += 1
            got.append(d.step([("r", ids[p:p + c], range(c))], end=["r"] if p + c == n else []))
            p += c
        close32(torch.cat(got), ref)


def test_mixed_with_pages_used_again(case):
    steps, pool = mixed_trace(case.reqs, seed=3)
    assert pool < sum((len(r) + 63) // 64 * 64 for r in case.reqs)
    d = case.driver(pool)
    seen = set()
    for entries, ended in steps:
        got = d.step([(r, case.reqs[r][lo:hi], range(hi - lo)) for r, lo, hi in entries], end=[])
        row = 0
        for r, lo, hi in entries:
            close32(got[row:row + hi - lo], case.refs[r][lo:hi])
            row += hi - lo
            seen |= set(p for p in d.executor.cache.groups[0].table(r) if p >= 0)
        for r in ended:
            d.executor.release(r)
            del d.positions[r]
        d.executor.cache.check_consistency()
    assert d.executor.cache.all_free()
    assert len(seen) < sum((len(r) + PAGE - 1) // PAGE for r in case.reqs)       # some page served two requests


def test_bfloat16_whole_and_decoded(case):
    """The serving precision at the same shape: a request whole, then another with its last 32 tokens decoded
    one by one, against the model's own bfloat16 bound."""
    from llmgen_b200.engine.api import load_model
    ids_a, ids_b = case.reqs[1], case.reqs[3]
    (ref_a, bound_a), (ref_b, bound_b) = reference(case.path, ids_a), reference(case.path, ids_b)
    forget_plain_models()
    bound = max(bound_a, bound_b)
    d = Driver(case.path, "bfloat16", 256, PAGE, model=load_model(case.path, "bfloat16"))
    logits_close(d.step([("a", ids_a, range(len(ids_a)))], end=["a"]), ref_a, "bfloat16", bound)
    n = len(ids_b)
    got = [d.step([("b", ids_b[:n - 32], [n - 33])])]
    for t in range(n - 32, n):
        got.append(d.step([("b", ids_b[t:t + 1], [0])]))
    logits_close(torch.cat(got), ref_b[n - 33:], "bfloat16", bound)
