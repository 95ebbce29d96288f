"""The workload generator of the `bench` command (no GPU): format, seeding, limits, command line."""
import json
import os
import subprocess
import sys

import pytest

from tests.util import ROOT

from llmgen_b200 import workload as wl


def test_scenarios_have_the_references_numbers():
    """bench/gen_workload.py:5-12 of the reference: requests x rounds, input and output ranges."""
    s = wl.SCENARIOS
    assert (s["single"].requests, s["single"].rounds, s["single"].input, s["single"].output) == (1, 5, (512, 512), (256, 256))
    assert (s["concurrent32"].requests, s["concurrent32"].rounds) == (32, 1)
    assert s["concurrent32"].input == (128, 512) and s["concurrent32"].output == (128, 512)
    assert (s["bench256"].requests, s["bench256"].input, s["bench256"].output) == (256, (100, 1024), (100, 1024))
    assert (s["concurrent8"].requests, s["concurrent8"].rounds) == (8, 3)
    assert s["concurrent8"].input == (256, 512) and s["concurrent8"].output == (128, 512)
    assert (s["longctx"].rounds, s["longctx"].input, s["longctx"].output) == (3, (3584, 3584), (512, 512))


def test_format_bounds_and_rounds():
    name, shape = wl.resolve_shape("concurrent8")
    made = wl.make_workload(name, shape, vocab=301, seed=3)
    assert made["name"] == "concurrent8" and len(made["rounds"]) == 3
    first = made["rounds"][0]
    assert len(first) == 8
    for rnd in made["rounds"]:
        for r, r0 in zip(rnd, first):
            assert set(r) == {"prompt_ids", "max_tokens", "temperature", "ignore_eos"}
            assert 256 <= len(r["prompt_ids"]) <= 512 and 128 <= r["max_tokens"] <= 512
            assert all(isinstance(t, int) and 0 <= t < 301 for t in r["prompt_ids"])
            assert r["temperature"] == 0.6 and r["ignore_eos"] is True
            # the lengths of every round are those of round 0; the ids are not
            assert len(r["prompt_ids"]) == len(r0["prompt_ids"]) and r["max_tokens"] == r0["max_tokens"]
    assert made["rounds"][1][0]["prompt_ids"] != first[0]["prompt_ids"]
    assert len({len(r["prompt_ids"]) for r in first}) > 1          # a range gives different lengths


def test_seed_decides_everything():
    name, shape = wl.resolve_shape(None, requests=5, rounds=2, input=(3, 40), output=(1, 9))
    a = wl.make_workload(name, shape, vocab=50, seed=11)
    b = wl.make_workload(name, shape, vocab=50, seed=11)
    c = wl.make_workload(name, shape, vocab=50, seed=12)
    assert a == b and a != c and a["name"] == "custom"


def test_overrides_and_max_model_len():
    name, shape = wl.resolve_shape("bench256", requests=64)
    assert name == "bench256-modified" and shape.requests == 64 and shape.input == (100, 1024)
    made = wl.make_workload(name, shape, seed=0, max_model_len=1100)
    assert len(made["rounds"][0]) == 64
    assert all(len(r["prompt_ids"]) + r["max_tokens"] <= 1100 and r["max_tokens"] >= 1 for r in made["rounds"][0])
    assert any(len(r["prompt_ids"]) + r["max_tokens"] == 1100 for r in made["rounds"][0])    # some were shortened
    with pytest.raises(wl.WorkloadError, match="no room"):
        wl.make_workload(*wl.resolve_shape("longctx"), max_model_len=2048)


@pytest.mark.parametrize("kwargs, text", [
    (dict(scenario="nope"), "unknown scenario"),
    (dict(scenario=None, requests=3), "needs --requests, --input and --output"),
    (dict(scenario="single", requests=0), "at least one request"),
    (dict(scenario="single", input=(9, 3)), "positive and ordered"),
    (dict(scenario="single", output=(0, 3)), "positive and ordered"),
])
def test_bad_shapes_are_refused(kwargs, text):
    with pytest.raises(wl.WorkloadError, match=text):
        wl.resolve_shape(kwargs.pop("scenario"), **kwargs)


def test_parse_range():
    assert wl.parse_range("512", "--input") == (512, 512)
    assert wl.parse_range("100:1024", "--input") == (100, 1024)
    for bad in ("", "a", "1:2:3", "1:"):
        with pytest.raises(wl.WorkloadError, match="--input"):
            wl.parse_range(bad, "--input")


def test_command_line_writes_what_bench_reads(tmp_path):
    out = str(tmp_path / "w.json")
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "llmgen_b200", "workload", out, "--requests", "3", "--rounds", "2", "--input", "4:9",
           "--output", "5", "--vocab", "256", "--seed", "7", "--request-temp", "0", "--max-model-len", "12"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert "3 requests x 2 rounds" in r.stderr
    with open(out, "r", encoding="utf-8") as f:
        made = json.load(f)
    assert [len(rnd) for rnd in made["rounds"]] == [3, 3]
    for req in made["rounds"][0]:
        assert 4 <= len(req["prompt_ids"]) <= 9 and len(req["prompt_ids"]) + req["max_tokens"] <= 12
        assert req["temperature"] == 0.0 and max(req["prompt_ids"]) < 256
    # the same call again gives the same file; a bad option is one line, not a traceback
    first = open(out, "rb").read()
    assert subprocess.run(cmd, env=env, capture_output=True, timeout=300).returncode == 0
    assert open(out, "rb").read() == first
    bad = subprocess.run(cmd[:5] + ["--scenario", "nope"], env=env, capture_output=True, text=True, timeout=300)
    assert bad.returncode != 0 and "unknown scenario" in bad.stderr and "Traceback" not in bad.stderr
