"""The per-kernel profiler around the real kernel bindings, and `chat` with the reference's
LLMGEN_PROFILE / LLMGEN_METRICS switches.  (The formulas and the bookkeeping are tested without a
GPU in tests/test_profiler.py.)"""
import json
import os
import subprocess
import sys
import tempfile

import pytest

from tests.plain.qwen3_plain import PlainQwen3
from tests.util import ROOT, TINY, Driver, logits_close, make_folder, random_ids

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tmp():
    with tempfile.TemporaryDirectory() as d:
        yield d


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_profiled_steps_give_the_same_logits_and_a_table(tmp, dtype):
    from llmgen_b200.engine import profiler as pf
    from llmgen_b200.kernels import ops
    path = make_folder(tmp, "D")
    ids = random_ids(61, TINY["D"][0]["vocab_size"], 3)
    plain = Driver(path, dtype, 256)
    ref_prompt = plain.step([("a", ids[:60], [0, 59])])
    ref_token = plain.step([("a", ids[60:], [0])])

    drv = Driver(path, dtype, 256)
    prof = pf.OpProfiler().enable()
    drv.executor.profiler = prof
    try:
        assert hasattr(ops.add_rmsnorm, "__wrapped__")
        got_prompt = drv.step([("a", ids[:60], [0, 59])])
        got_token = drv.step([("a", ids[60:], [0])])
    finally:
        prof.disable()
        drv.executor.profiler = None
    assert not hasattr(ops.add_rmsnorm, "__wrapped__") and pf.OpProfiler._active is None
    # the same kernels with marks between them: the same values
    logits_close(got_prompt, ref_prompt, dtype, 1e-5)
    logits_close(got_token, ref_token, dtype, 1e-5)

    assert prof.passes == {pf.PREFILL: 1, pf.DECODE: 1}
    for phase in (pf.PREFILL, pf.DECODE):
        rows = prof.rows(phase)
        names = [r["op"] for r in rows]
        assert any(n.startswith(("gemm", "gemv")) for n in names), names
        assert any("attention" in n for n in names), names
        assert "embed_rows" in names and "add_rmsnorm" in names
        assert all(r["calls"] > 0 and r["total_ms"] >= 0 for r in rows) and sum(r["total_ms"] for r in rows) > 0
        assert [r["total_ms"] for r in rows] == sorted((r["total_ms"] for r in rows), reverse=True)
        products = [r for r in rows if r["op"].startswith(("gemm", "gemv"))]
        assert all(r["gflops"] > 0 and r["gbps"] > 0 for r in products)
        # a pass lasts at least as long as its kernels (the events' resolution aside)
        assert prof.phase_ms[phase] >= 0.9 * prof.op_ms(phase)
    text = prof.text()
    assert "[prefill] (1 passes" in text and "[decode] (1 passes" in text and "(between kernels)" in text


def test_chat_with_the_profile_and_metrics_switches(tmp):
    path = make_folder(tmp, "A")
    prompt = random_ids(11, 256, 95)
    ref = PlainQwen3(path).greedy(prompt, 6)
    report = os.path.join(tmp, "metrics.json")
    env = dict(os.environ, LLMGEN_PROFILE="1", LLMGEN_METRICS="1", LLMGEN_METRICS_JSON=report, LLMGEN_PEAK_GBPS="6500")
    cmd = [sys.executable, "-m", "llmgen_b200", "chat", ",".join(map(str, prompt)), "6", "--model", path,
           "--dtype", "float32", "--max-model-len", "64", "--kv-blocks", "8", "--max-num-seqs", "4",
           "--max-batched-tokens", "64"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("token ids:")][0]
    assert [int(x) for x in line.split(":")[1].split()] == ref
    err = proc.stderr
    assert "=== kernel time [prefill] (1 passes" in err and "=== kernel time [decode] (5 passes" in err
    assert "=== generation metrics ===" in err and "=== hardware efficiency ===" in err and "MBU (decode)" in err
    with open(report, "r", encoding="utf-8") as f:
        r = json.load(f)
    assert r["prompt_tokens"] == 11 and r["gen_tokens"] == 6
    assert r["ttft_ms"] > 0 and r["tpot_ms"] > 0 and r["decode_tps"] > 0 and r["e2e_ms"] >= r["ttft_ms"]
