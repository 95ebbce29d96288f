"""Latency metrics, the model's cost formulas and the per-kernel profiler (no GPU: the profiler
runs here around stand-ins of the kernel bindings, with a clock that counts)."""
import json
import random
import types

import pytest
import torch

from tests.util import TINY_C

from llmgen_b200.config.qwen3 import Qwen3Config
from llmgen_b200.engine import profiler as pf
from llmgen_b200.models.qwen3 import build_qwen3_spec

QWEN3_06B = {
    "architectures": ["Qwen3ForCausalLM"], "vocab_size": 151936, "hidden_size": 1024, "intermediate_size": 3072,
    "num_hidden_layers": 28, "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 40960, "tie_word_embeddings": True,
}


# ------------------------------------------------------------------------------ GenMetrics
def test_percentile_interpolates():
    assert pf.percentile([], 50) == 0.0
    assert pf.percentile([3.0], 99) == 3.0
    assert pf.percentile([1.0, 2.0, 3.0, 4.0], 50) == 2.5
    assert pf.percentile([1.0, 2.0, 3.0, 4.0], 100) == 4.0
    assert abs(pf.percentile([0.0, 10.0], 99) - 9.9) < 1e-12


def test_gen_metrics_report(tmp_path, monkeypatch):
    m = pf.GenMetrics()
    m.start(prompt_tokens=100, now=10.0)
    for t in (10.5, 10.51, 10.53, 10.56, 10.60):          # first token after 0.5 s, then gaps of 10, 20, 30, 40 ms
        m.on_token(t)
    m.finish(10.7)
    r = m.report()
    assert r["prompt_tokens"] == 100 and r["gen_tokens"] == 5 and r["backend"] == "llmgen_b200"
    assert abs(r["ttft_ms"] - 500.0) < 1e-6 and abs(r["e2e_ms"] - 700.0) < 1e-6
    assert abs(r["tpot_ms"] - 25.0) < 1e-6                  # 100 ms over four gaps
    assert abs(r["itl_p50_ms"] - 25.0) < 1e-6 and abs(r["itl_p99_ms"] - 39.7) < 1e-6
    assert abs(r["prefill_tps"] - 200.0) < 1e-6 and abs(r["decode_tps"] - 40.0) < 1e-6
    text = m.text()
    assert "TTFT" in text and "ITL p50/p90/p99/max" in text and "decode" in text
    # the JSON goes where LLMGEN_METRICS_JSON says, and nowhere without it
    monkeypatch.delenv("LLMGEN_METRICS_JSON", raising=False)
    assert m.write_json() is None
    path = str(tmp_path / "m.json")
    monkeypatch.setenv("LLMGEN_METRICS_JSON", path)
    assert m.write_json() == path
    with open(path, "r", encoding="utf-8") as f:
        assert json.load(f) == r


def test_gen_metrics_without_tokens_or_with_one():
    m = pf.GenMetrics()
    m.start(7, 1.0)
    m.finish(2.0)
    r = m.report()
    assert r["gen_tokens"] == 0 and r["ttft_ms"] == 0.0 and r["decode_tps"] == 0.0 and r["tpot_ms"] == 0.0
    m.on_token(1.25)
    r = m.report()
    assert r["gen_tokens"] == 1 and abs(r["ttft_ms"] - 250.0) < 1e-9 and r["itl_p99_ms"] == 0.0
    assert "TPOT" not in m.text()


# ------------------------------------------------------------------------------- ModelCost
def test_model_cost_of_the_benchmark_shape():
    """Weights in products, cache bytes per token and a prompt's FLOPs of the 0.6B shape by hand."""
    spec = build_qwen3_spec(Qwen3Config.from_dict(QWEN3_06B))
    cost = pf.ModelCost.from_spec(spec, w_elem=2, kv_elem=2)
    per_layer = 1024 * 2048 + 2 * 1024 * 1024 + 2048 * 1024 + 3 * 1024 * 3072
    assert cost.complete and cost.head_params == 1024 * 151936
    assert cost.n_mm == 28 * per_layer + 1024 * 151936 == 595_984_384
    assert cost.kv_bytes_per_token() == 114_688
    P = 2048
    by_hand = 2 * 28 * per_layer * P + 2 * 1024 * 151936 + 4 * 28 * 2048 * P * (P + 1) // 2
    assert cost.prefill_flops(P) == by_hand
    assert cost.prefill_flops(P, logits_rows=P) == 2 * cost.n_mm * P + 4 * 28 * 2048 * P * (P + 1) // 2
    # 256 steps from a 512-token prompt: contexts 513 .. 768
    ctx = sum(range(513, 769))
    assert cost.decode_flops(513, 256) == 2 * cost.n_mm * 256 + 4 * 28 * 2048 * ctx
    assert cost.decode_bytes(513, 256) == cost.n_mm * 2 * 256 + 114_688 * ctx


def test_model_cost_counts_a_window():
    spec = build_qwen3_spec(Qwen3Config.from_dict(TINY_C))        # window 40 on layers 1 and 2 of 4
    cost = pf.ModelCost.from_spec(spec, 4, 4)
    assert [t.window for t in cost.attention] == [0, 40, 40, 0]
    q_dim = 6 * 48
    for c0, n in ((1, 1), (1, 100), (30, 25), (41, 3), (500, 7)):
        full = sum(range(c0, c0 + n))
        windowed = sum(min(c, 40) for c in range(c0, c0 + n))
        assert cost.decode_flops(c0, n) == 2 * cost.n_mm * n + 4 * q_dim * (2 * full + 2 * windowed)
    rng = random.Random(0)
    for _ in range(200):
        c0, n, w = rng.randrange(1, 90), rng.randrange(0, 90), rng.choice([0, 1, 2, 7, 40, 64])
        assert pf.ModelCost._visible_sum(c0, n, w) == sum(min(c, w) if w else c for c in range(c0, c0 + n))


def test_model_cost_says_when_a_part_is_unknown():
    spec = build_qwen3_spec(Qwen3Config.from_dict(TINY_C))
    odd = types.SimpleNamespace(kind="something_else")
    layers = (types.SimpleNamespace(mixer=odd, ffn=spec.layers[0].ffn),) + tuple(spec.layers[1:])
    patched = types.SimpleNamespace(run_order=spec.run_order, layers=layers, hidden_size=spec.hidden_size,
                                    vocab_size=spec.vocab_size)
    cost = pf.ModelCost.from_spec(patched)
    assert not cost.complete and len(cost.attention) == 3


def test_efficiency_text_uses_the_peaks(monkeypatch):
    spec = build_qwen3_spec(Qwen3Config.from_dict(QWEN3_06B))
    cost = pf.ModelCost.from_spec(spec)
    m = pf.GenMetrics()
    m.start(2048, 0.0)
    m.on_token(0.005)
    for i in range(1, 11):
        m.on_token(0.005 + i * 0.001)
    m.finish(0.02)
    monkeypatch.delenv("LLMGEN_PEAK_TFLOPS", raising=False)
    monkeypatch.delenv("LLMGEN_PEAK_GBPS", raising=False)
    plain = pf.efficiency_text(m, cost)
    assert "MFU" not in plain and "MBU" not in plain and "596.0 M" in plain
    monkeypatch.setenv("LLMGEN_PEAK_TFLOPS", "1000")
    monkeypatch.setenv("LLMGEN_PEAK_GBPS", "6000")
    text = pf.efficiency_text(m, cost)
    mfu = cost.prefill_flops(2048) / 0.005 / 1e15 * 100
    mbu = cost.decode_bytes(2049, 10) / 0.010 / 6e12 * 100
    assert f"MFU (prefill) : {mfu:.1f} %" in text and f"MBU (decode)  : {mbu:.1f} %" in text


# ------------------------------------------------------------------------------ OpProfiler
class CountingClock:
    """Every mark is the next integer; a millisecond per unit."""

    def __init__(self):
        self.now, self.waits = 0, 0

    def mark(self):
        self.now += 1
        return self.now

    def wait(self):
        self.waits += 1

    def elapsed_ms(self, a, b):
        return float(b - a)


def fake_ops():
    """Stand-ins with the real bindings' parameter names that advance nothing and return nothing."""
    calls = []
    mod = types.SimpleNamespace(calls=calls)

    def gemm_tc(out, a, w, gated=False, pdl=True):
        calls.append("gemm_tc")

    def add_rmsnorm(resid, delta, weight, out, eps, weight_offset=0.0, rows=None, write_resid=True):
        calls.append("add_rmsnorm")

    def attention_tc(out, q, q_stride, kcache, vcache, block_tables, max_blocks, ctx_len, cu_q, tile_seq, tile_q0,
                     n_tiles, n_tokens, nq, nkv, hd, page_size, window, scale, v_lbo=0, v_sbo=0):
        calls.append("attention_tc")

    def embed_rows(out, table, ids, bad_flag=None, ids_from=None, sampled=None):
        calls.append("embed_rows")

    def gemm_tc_usable(a, w):                                # not a launch: must stay as it is
        return True

    mod.gemm_tc, mod.add_rmsnorm, mod.attention_tc, mod.embed_rows, mod.gemm_tc_usable = \
        gemm_tc, add_rmsnorm, attention_tc, embed_rows, gemm_tc_usable
    return mod


def test_profiler_wraps_times_counts_and_restores():
    ops = fake_ops()
    originals = (ops.gemm_tc, ops.add_rmsnorm, ops.gemm_tc_usable)
    prof = pf.OpProfiler(ops_module=ops, clock=CountingClock())
    x = torch.zeros(6, 32, dtype=torch.bfloat16)
    w = torch.zeros(48, 32, dtype=torch.bfloat16)
    y = torch.zeros(6, 48, dtype=torch.bfloat16)
    with prof:
        assert ops.gemm_tc is not originals[0] and ops.gemm_tc_usable is originals[2]
        with pytest.raises(RuntimeError, match="another OpProfiler"):
            pf.OpProfiler(ops_module=ops, clock=CountingClock()).enable()
        prof.begin_pass([0], [6])
        ops.gemm_tc(y, x, w)
        ops.gemm_tc(out=y, a=x, w=w, gated=False)
        prof.begin_pass([6, 9], [1, 1])
        ops.gemm_tc(y[:2], x[:2], w)
    assert (ops.gemm_tc, ops.add_rmsnorm, ops.gemm_tc_usable) == originals        # restored
    assert pf.OpProfiler._active is None and ops.calls == ["gemm_tc"] * 3
    s = prof.stats[(pf.PREFILL, "gemm_tc")]
    assert s.calls == 2 and s.flops == 2 * (2 * 6 * 48 * 32) and s.bytes == 2 * 2 * (6 * 32 + 48 * 32 + 6 * 48)
    assert s.ms == 2.0                                       # one unit between the two marks of each call
    assert prof.phase_ms[pf.PREFILL] == 3.0 and prof.passes == {pf.PREFILL: 1, pf.DECODE: 1}
    d = prof.stats[(pf.DECODE, "gemm_tc")]
    assert d.calls == 1 and d.flops == 2 * 2 * 48 * 32
    rows = prof.rows(pf.PREFILL)
    assert [r["op"] for r in rows] == ["gemm_tc"] and abs(rows[0]["pct"] - 200.0 / 3.0) < 1e-9
    assert rows[0]["avg_us"] == 1000.0
    text = prof.text()
    assert "[prefill] (1 passes, 3.00 ms)" in text and "[decode]" in text and "(between kernels)" in text
    # a second round with the same object works after disable
    with prof:
        ops.gemm_tc(y, x, w)
    assert prof.stats[(pf.DECODE, "gemm_tc")].calls == 2


def test_profiler_phases_and_attention_cost():
    ops = fake_ops()
    prof = pf.OpProfiler(ops_module=ops, clock=CountingClock()).enable()
    try:
        kc = torch.zeros(4, 2, 16, 64, dtype=torch.bfloat16)
        o = torch.zeros(9, 6 * 64, dtype=torch.bfloat16)
        args = (o, o, 384, kc, kc, None, 8, None, None, None, None, 3, 9, 6, 2, 64, 16)
        prof.begin_pass([0, 10], [5, 4])                     # two portions of prompts
        assert prof.info.phase == pf.PREFILL
        ops.attention_tc(*args, 0, 0.125)
        seen = sum(range(1, 6)) + sum(range(11, 15))
        s = prof.stats[(pf.PREFILL, "attention_tc")]
        assert s.flops == 4 * 6 * 64 * seen
        assert s.bytes == 2 * 2 * 64 * 2 * (5 + 14) + 2 * 9 * 6 * 64 * 2
        prof.begin_pass([0, 30], [8, 1])                     # a portion beside a decoded token, window 4
        assert prof.info.phase == pf.MIXED
        ops.attention_tc(*args, 4, 0.125)
        seen = (1 + 2 + 3 + 4 * 5) + 4
        m = prof.stats[(pf.MIXED, "attention_tc")]
        assert m.flops == 4 * 6 * 64 * seen
        assert m.bytes == 2 * 2 * 64 * 2 * (8 + 4) + 2 * 9 * 6 * 64 * 2
        prof.begin_pass([0], [1])                            # the first token of a prompt of one is a prompt
        assert prof.info.phase == pf.DECODE
    finally:
        prof.disable()


def test_costs_of_the_small_kernels():
    info = pf.PassInfo()
    table = torch.zeros(300, 80, dtype=torch.bfloat16)
    out = torch.zeros(7, 80, dtype=torch.float32)
    ids = torch.zeros(7, dtype=torch.int32)
    assert pf._cost_embed({"out": out, "table": table, "ids": ids}, info) == (0, 7 * 4 + 7 * 80 * 4 + 7 * 80 * 2)
    resid = torch.zeros(7, 80, dtype=torch.float32)
    delta = torch.zeros(7, 80, dtype=torch.bfloat16)
    gain = torch.zeros(80, dtype=torch.float32)
    y = torch.zeros(7, 80, dtype=torch.bfloat16)
    flops, nbytes = pf._cost_norm({"resid": resid, "delta": delta, "weight": gain, "out": y, "rows": None, "write_resid": True}, info)
    assert nbytes == 2 * 7 * 80 * 4 + 7 * 80 * 2 + 7 * 80 * 2 + 80 * 4 and flops == 5 * 7 * 80
    flops, nbytes = pf._cost_norm({"resid": resid, "delta": None, "weight": gain, "out": y[:2], "rows": ids[:2], "write_resid": True}, info)
    assert nbytes == 2 * 80 * 4 + 2 * 80 * 2 + 80 * 4
    # slices of a product cut along K count with all their bytes
    slices = types.SimpleNamespace(tensor=torch.zeros(4, 7, 80, dtype=torch.float32))
    assert pf._nbytes(slices) == 4 * 7 * 80 * 4 and pf._nbytes(None) == 0
    x = torch.zeros(7, 80, dtype=torch.bfloat16)
    w = torch.zeros(48, 80, dtype=torch.bfloat16)
    flops, nbytes = pf._cost_product({"out": slices.tensor, "a": x, "w": w}, info)
    assert flops == 2 * 7 * 48 * 80 and nbytes == 48 * 80 * 2 + 7 * 80 * 2 + 4 * 7 * 80 * 4


def test_launches_into_a_graph_are_not_timed():
    class Capturing(CountingClock):
        def mark(self):
            return None

    ops = fake_ops()
    with pf.OpProfiler(ops_module=ops, clock=Capturing()) as prof:
        ops.embed_rows(torch.zeros(2, 8), torch.zeros(10, 8), torch.zeros(2, dtype=torch.int32))
    assert ops.calls == ["embed_rows"] and prof.stats == {} and prof.text() == ""


def test_every_listed_binding_exists_with_the_operands_its_cost_reads():
    """The cost functions name parameters of the real bindings: a renamed parameter must show here."""
    import inspect
    from llmgen_b200.kernels import ops
    needs = {pf._cost_product: [("w",), ("a", "x"), ("out", "slices")], pf._cost_attention: [("nq",), ("nkv",), ("hd",), ("window",), ("kcache",)],
             pf._cost_attn_prep: [("qkv",), ("nq",), ("nk",), ("hd",), ("rot",), ("kcache",), ("cos",)],
             pf._cost_embed: [("out",), ("table",), ("ids",)], pf._cost_norm: [("out",), ("weight",), ("delta",), ("rows",), ("write_resid",)],
             pf._cost_all_operands: [("out", "out_ids")]}
    for name, cost in pf.OP_COSTS.items():
        params = inspect.signature(getattr(ops, name)).parameters
        for alternatives in needs[cost]:
            assert any(p in params for p in alternatives), f"{name} has none of {alternatives}"


def test_llm_profile_needs_eager_steps_and_cleans_up(monkeypatch):
    from llmgen_b200.engine.api import LLM
    monkeypatch.setattr(pf, "CudaEventClock", CountingClock)
    llm = LLM.__new__(LLM)                                   # no GPU here: only what profile() touches
    llm.executor = types.SimpleNamespace(eager=False, profiler=None)
    with pytest.raises(ValueError, match="eager=True"):
        with llm.profile():
            pass
    llm.executor.eager = True
    with pytest.raises(KeyError):
        with llm.profile() as prof:
            assert llm.executor.profiler is prof and pf.OpProfiler._active is prof
            raise KeyError("inside")
    assert llm.executor.profiler is None and pf.OpProfiler._active is None
