"""Replay through the engine's own step function, cache manager and kernels, compared with the
plain implementation: each request alone and whole; most of it in one step and the last 32
tokens one by one; in portions of changing size down to two tokens; mixed, up to four live
requests with so few pages that they are used again; long decoding; the first tokens of a
sequence; prompts of several hundred tokens.  In float32 and in bfloat16, on five tiny
configurations (D and E have the head sizes the tensor-core and flash-decoding kernels take)."""
import json
import os
import random
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from tests.util import (NEEDLE_ID, FILLER_ID, ROOT, TINY, Driver, logits_close, make_folder, needle_folder, needle_ids,
                        plain_model, random_ids, reference)

pytestmark = pytest.mark.gpu

LENGTHS = [70, 45, 100, 33, 64, 90]
_cache = {}


@pytest.fixture(scope="module")
def tmp():
    with tempfile.TemporaryDirectory() as d:
        yield d


def case(tmp, name, sharp=False):
    """(model folder, requests' token ids, plain logits per request, the model's bfloat16 bound on these requests)."""
    key = (name, sharp)
    if key not in _cache:
        path = make_folder(tmp, name)
        if sharp:
            path = sharpen(path, tmp, name)
        vocab = TINY[name][0]["vocab_size"]
        reqs = [random_ids(n, vocab, 100 + i) for i, n in enumerate(LENGTHS)]
        refs = [reference(path, r) for r in reqs]
        _cache[key] = (path, reqs, [r[0] for r in refs], max(r[1] for r in refs))
    return _cache[key]


def sharpen(path, tmp, name):
    """A copy of the model whose q/k norm gains are 3x: scores grow 9x, attention becomes
    peaked, and a single missed or misplaced key shows in the logits.  Run in float32 only: in
    bfloat16 the rounding of q and k is magnified 9x in the scores as well, so a comparison with
    float32 arithmetic would measure that and not the cache."""
    from safetensors.torch import load_file, save_file
    out = os.path.join(tmp, f"sharp_{name}")
    if not os.path.isdir(out):
        os.makedirs(out)
        with open(os.path.join(path, "config.json")) as f, open(os.path.join(out, "config.json"), "w") as g:
            g.write(f.read())
        t = load_file(os.path.join(path, "model.safetensors"))
        for k in t:
            if k.endswith("q_norm.weight") or k.endswith("k_norm.weight"):
                t[k] = (t[k].float() * 3).to(t[k].dtype)
        save_file(t, os.path.join(out, "model.safetensors"))
    return out


CASES = [(n, d) for n in "ABCDE" for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole(tmp, name, dtype):
    path, reqs, refs, bound = case(tmp, name)
    d = Driver(path, dtype, 128, TINY[name][5])
    for ids, ref in zip(reqs, refs):
        got = d.step([("r", ids, range(len(ids)))], end=["r"])
        logits_close(got, ref, dtype, bound)
        if dtype == "float32":
            assert torch.equal(got.argmax(-1), ref.argmax(-1))       # identical greedy ids
    assert d.executor.cache.all_free()


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_one_by_one(tmp, name, dtype):
    path, reqs, refs, bound = case(tmp, name)
    d = Driver(path, dtype, 128, TINY[name][5])
    for ids, ref in zip(reqs, refs):
        n = len(ids)
        head = n - 32
        got = [d.step([("r", ids[:head], [head - 1])])]
        for t in range(head, n):
            got.append(d.step([("r", ids[t:t + 1], [0])], end=["r"] if t == n - 1 else []))
        logits_close(torch.cat(got), ref[head - 1:], dtype, bound)


@pytest.mark.parametrize("eager", [True, False], ids=["launched", "replayed"])
@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_changing_size(tmp, name, dtype, eager):
    path, reqs, refs, bound = case(tmp, name)
    d = Driver(path, dtype, 128, TINY[name][5], eager=eager)
    rng = random.Random(5)
    for ids, ref in zip(reqs, refs):
        n, p, got = len(ids), 0, []
        sizes = [7, 2, 16, 3]
        while p < n:
            c = sizes.pop(0) if sizes else rng.choice([2, 2, 5, 11, 17, 31])
            c = min(c, n - p)
            if n - p - c == 1:
                c += 1                                   # never leave a portion of one token here
            got.append(d.step([("r", ids[p:p + c], range(c))], end=["r"] if p + c == n else []))
            p += c
        logits_close(torch.cat(got), ref, dtype, bound)
    assert eager or d.executor.n_shaped_steps > 0            # portions went through the graphs of their shapes


def mixed_trace(reqs, seed, max_live=4):
    """Steps of a mixed run: up to `max_live` live requests; each step takes portions of some
    (2..24 tokens, or single tokens once a request is within its last 32) and leaves others out.
    Returns (steps, pool tokens) with steps = [(entries [(id, lo, hi)], ended ids)]."""
    rng = random.Random(seed)
    todo = list(range(len(reqs)))
    live, pos, steps = [], {}, []
    peak = 0
    while todo or live:
        while todo and len(live) < max_live and (not live or rng.random() < 0.6):
            r = todo.pop(0)
            live.append(r)
            pos[r] = 0
        entries, ended = [], []
        for r in list(live):
            if len(live) > 1 and rng.random() < 0.25:
                continue                                  # left out of this step, goes on later
            n = len(reqs[r])
            left = n - pos[r]
            c = 1 if left <= 32 else min(rng.choice([2, 3, 8, 13, 24]), left - 32)
            entries.append((r, pos[r], pos[r] + c))
            pos[r] += c
            if pos[r] == n:
                ended.append(r)
        if not entries:
            continue
        peak = max(peak, sum((pos[r] + 63) // 64 * 64 for r in live))
        for r in ended:
            live.remove(r)
        steps.append((entries, ended))
    return steps, peak


@pytest.mark.parametrize("eager", [True, False], ids=["launched", "replayed"])
@pytest.mark.parametrize("name,dtype", CASES + [("C-sharp", "float32"), ("B-sharp", "float32"), ("A-sharp", "float32")])
def test_mixed_with_pages_used_again(tmp, name, dtype, eager):
    sharp = name.endswith("-sharp")
    name = name[0]
    path, reqs, refs, bound = case(tmp, name, sharp)
    steps, pool = mixed_trace(reqs, seed=3)
    assert pool < sum((len(r) + 63) // 64 * 64 for r in reqs)          # so pages must be used again
    d = Driver(path, dtype, pool, TINY[name][5], eager=eager)
    seen_pages = set()
    reused = False
    worst = 0.0
    for entries, ended in steps:
        got = d.step([(r, reqs[r][lo:hi], range(hi - lo)) for r, lo, hi in entries], end=[])
        row = 0
        for r, lo, hi in entries:
            worst = max(worst, logits_close(got[row:row + hi - lo], refs[r][lo:hi], dtype, bound))
            row += hi - lo
        for r in [e[0] for e in entries]:
            pages = set(p for p in d.executor.cache.groups[0].table(r) if p >= 0)
            seen_pages |= pages
        for r in ended:
            d.executor.release(r)
            del d.positions[r]
        d.executor.cache.check_consistency()
    assert d.executor.cache.all_free()
    total_pages_taken = sum((len(r) + TINY[name][5] - 1) // TINY[name][5] for r in reqs)
    assert len(seen_pages) < total_pages_taken                           # some page served two requests
    assert eager or (d.executor.n_shaped_steps > 0 and d.executor.shaped_steps)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "float32"), ("C", "bfloat16"), ("B", "bfloat16")])
def test_long_decoding(tmp, name, dtype):
    path = make_folder(tmp, name, max_position_embeddings=320)        # more positions than A and B have
    vocab = TINY[name][0]["vocab_size"]
    ids = random_ids(260, vocab, 77)
    ref, bound = reference(path, ids)
    d = Driver(path, dtype, 320, TINY[name][5])
    got = [d.step([("r", ids[:3], [0, 1, 2])])]
    for t in range(3, 260):
        got.append(d.step([("r", ids[t:t + 1], [0])]))
    logits_close(torch.cat(got), ref, dtype, bound)


@pytest.mark.parametrize("eager", [True, False], ids=["launched", "replayed"])
@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens(tmp, name, dtype, eager):
    path, reqs, refs, bound = case(tmp, name)
    d = Driver(path, dtype, 128, TINY[name][5], eager=eager)
    ids, ref = reqs[0], refs[0]
    # a prompt of one token, then single tokens; beside it a request cut 1 + 1 + 2
    got_a = [d.step([("a", ids[:1], [0])])]
    got_a.append(d.step([("a", ids[1:2], [0]), ("b", reqs[1][:1], [0])]))
    got_b = [got_a[-1][1:]]
    got_a[-1] = got_a[-1][:1]
    both = d.step([("a", ids[2:3], [0]), ("b", reqs[1][1:2], [0])])
    got_a.append(both[:1])
    got_b.append(both[1:])
    got_b.append(d.step([("b", reqs[1][2:4], [0, 1])]))
    logits_close(torch.cat(got_a), ref[:3], dtype, bound)
    logits_close(torch.cat(got_b), refs[1][:4], dtype, bound)


@pytest.mark.parametrize("eager", [True, False], ids=["launched", "replayed"])
@pytest.mark.parametrize("name", ["D", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_in_portions_beside_decoding(tmp, name, dtype, eager):
    """517 and 330 tokens: several query and key tiles of the tensor-core kernel, portions that
    start inside a tile, a portion beside a decoded token, then both decoding (the flash-decoding
    kernel with several key parts), then a portion again."""
    path = make_folder(tmp, name)
    vocab = TINY[name][0]["vocab_size"]
    a, b = random_ids(517, vocab, 41), random_ids(330, vocab, 42)
    (ref_a, bound_a), (ref_b, bound_b) = reference(path, a), reference(path, b)
    bound = max(bound_a, bound_b)
    d = Driver(path, dtype, 1024, TINY[name][5], eager=eager)
    worst = 0.0

    def check(got, *parts):
        nonlocal worst
        row = 0
        for ref, lo, hi in parts:
            worst = max(worst, logits_close(got[row:row + hi - lo], ref[lo:hi], dtype, bound))
            row += hi - lo

    check(d.step([("a", a[0:260], range(260))]), (ref_a, 0, 260))
    check(d.step([("a", a[260:500], range(240)), ("b", b[0:150], range(150))]), (ref_a, 260, 500), (ref_b, 0, 150))
    check(d.step([("a", a[500:501], [0]), ("b", b[150:300], range(150))]), (ref_a, 500, 501), (ref_b, 150, 300))
    for i in range(16):
        check(d.step([("a", a[501 + i:502 + i], [0]), ("b", b[300 + i:301 + i], [0])]),
              (ref_a, 501 + i, 502 + i), (ref_b, 300 + i, 301 + i))
    check(d.step([("b", b[316:330], range(14))], end=["a", "b"]), (ref_b, 316, 330))
    assert d.executor.cache.all_free()


def needle_case(tmp, name, n, needle_at, seed=5, positions=0):
    """(folder, ids, exact logits, bfloat16 bound) of a sequence whose last token looks for the needle, after a
    check on the plain model alone that losing the needle moves the last row by at least 10 times the bound."""
    path = needle_folder(tmp, name)
    if positions:
        path = make_folder_with_positions(tmp, path, positions)
    vocab = TINY[name][0]["vocab_size"]
    ids = needle_ids(n, vocab, needle_at, seed)
    ref, bound = reference(path, ids)
    lost = list(ids)
    lost[needle_at] = FILLER_ID
    moved = float((plain_model(path).logits(lost)[-1] - ref[-1]).abs().max())
    assert moved >= 10 * bound, f"the needle at {needle_at} of {n} moves the last row by {moved:.3f}, the bound is {bound:.3f}"
    return path, ids, ref, bound


@pytest.mark.parametrize("eager", [True, False], ids=["launched", "replayed"])
@pytest.mark.parametrize("name", ["D", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,needle_at", [(100, 3), (300, 15), (300, 16), (300, 160), (600, 127), (600, 128), (600, 31), (600, 597)])
def test_one_key_that_matters_is_found_wherever_it_lies(tmp, name, dtype, n, needle_at, eager):
    """The needle model (tests.util.needle_folder): the probe token at the end reads mostly one key, which lies
    at a page's first or last place, at a key tile's edge, hundreds of keys back or next to the probe.  Its
    logits are compared when the probe comes with the whole prompt, as the last of a portion after portions of
    uneven size, and as a single decoded token after pages were given back and taken again."""
    path, ids, ref, bound = needle_case(tmp, name, n, needle_at)
    page = TINY[name][5]
    d = Driver(path, dtype, 1024, page, eager=eager)
    got = d.step([("w", ids, [n - 1])], end=["w"])
    logits_close(got, ref[n - 1:], dtype, bound)
    # pages of "w" are free again; another request takes some of them first, so that "p" gets them in another order
    d.step([("other", ids[:37], [])])
    p, sizes = 0, [7, 50, 2, 129, 33]
    while p < n:
        c = min(sizes[(p // 7) % len(sizes)], n - p)
        if n - p - c == 1:
            c += 1
        got = d.step([("p", ids[p:p + c], [c - 1])], end=["p"] if p + c == n else [])
        p += c
    logits_close(got, ref[n - 1:], dtype, bound)
    d.executor.release("other")
    del d.positions["other"]
    d.step([("d", ids[:n - 9], [])])
    for t in range(n - 9, n):
        got = d.step([("d", ids[t:t + 1], [0])], end=["d"] if t == n - 1 else [])
        logits_close(got, ref[t:t + 1], dtype, bound)
    assert d.executor.cache.all_free()


@pytest.mark.parametrize("name,dtype,n,needle_at", [("D", "bfloat16", 1100, 5), ("E", "bfloat16", 1100, 5), ("E", "float32", 1100, 5),
                                                    ("E", "bfloat16", 2100, 1531), ("E", "float32", 2100, 1531)])
def test_decoding_over_thousands_of_keys(tmp, name, dtype, n, needle_at):
    """Single tokens against 1,100 and 2,100 keys (the context classes of 2,048 and 4,096 keys: many key parts,
    some of them empty), beside a short sequence, the last token looking for a needle far back."""
    path, ids, ref, bound = needle_case(tmp, name, n, needle_at, seed=6, positions=4096)
    short = random_ids(40, TINY[name][0]["vocab_size"], 9)
    ref_s, bound_s = reference(path, short)
    bound = max(bound, bound_s)
    d = Driver(path, dtype, 4096, TINY[name][5])
    d.step([("long", ids[:n - 12], [])])
    d.step([("short", short[:28], [])])
    for i in range(12):
        got = d.step([("long", ids[n - 12 + i:n - 11 + i], [0]), ("short", short[28 + i:29 + i], [0])])
        logits_close(got[:1], ref[n - 12 + i:n - 11 + i], dtype, bound)
        logits_close(got[1:], ref_s[28 + i:29 + i], dtype, bound)


def make_folder_with_positions(tmp, path, positions):
    """A copy of the model folder `path` whose config.json allows `positions` positions (same weights)."""
    out = f"{path}_p{positions}"
    if not os.path.isdir(out):
        os.makedirs(out)
        with open(os.path.join(path, "config.json")) as f:
            cfg = json.load(f)
        cfg["max_position_embeddings"] = positions
        with open(os.path.join(out, "config.json"), "w") as g:
            json.dump(cfg, g)
        os.symlink(os.path.join(path, "model.safetensors"), os.path.join(out, "model.safetensors"))
    return out


def test_want_order_and_empty_want(tmp):
    path, reqs, refs, bound = case(tmp, "A")
    d = Driver(path, "float32", 128, 16)
    got = d.step([("a", reqs[0][:10], [9, 0, 4]), ("b", reqs[1][:6], []), ("c", reqs[2][:5], [2])])
    ref = torch.stack([refs[0][9], refs[0][0], refs[0][4], refs[2][2]])
    logits_close(got, ref, "float32")
    # a step in which nothing is wanted still fills the cache
    assert d.step([("b", reqs[1][6:20], [])]).shape == (0, 256)
    logits_close(d.step([("b", reqs[1][20:21], [0])]), refs[1][20:21], "float32")


def test_more_tokens_than_one_pass_holds(tmp):
    """A step above the tokens-per-pass limit is cut into passes; logits keep their order."""
    from llmgen_b200.engine.api import load_model
    from llmgen_b200.engine.executor import EngineLimits, Executor, StepEntry
    path, reqs, refs, bound = case(tmp, "A")
    ex = Executor(load_model(path, "float32"), EngineLimits(max_num_seqs=4, max_model_len=128, max_step_tokens=24,
                                                            page_size=16, num_pages=32), eager=True)
    for r in ("x", "y"):
        assert ex.admit(r)
    assert ex.reserve("x", 0, 70) and ex.reserve("y", 0, 45)
    out = ex.step([StepEntry("x", reqs[0], 0, [69, 3, 30]), StepEntry("y", reqs[1], 0, [44, 0])], return_logits=True)
    ref = torch.stack([refs[0][69], refs[0][3], refs[0][30], refs[1][44], refs[1][0]])
    logits_close(out.logits.cpu(), ref, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp, dtype):
    """The program itself, as a user calls it: JSON lines in, <step>.f32 files and `done` lines out."""
    path, reqs, refs, bound = case(tmp, "C")
    steps, pool = mixed_trace(reqs, seed=9)
    out_dir = os.path.join(tmp, f"trace_out_{dtype}")
    lines = []
    for i, (entries, ended) in enumerate(steps):
        lines.append(json.dumps({"step": i, "entries": [{"id": f"r{r}", "tokens": reqs[r][lo:hi],
                                                          "want": list(range(hi - lo)) if (i + r) % 3 else [hi - lo - 1]}
                                                         for r, lo, hi in entries],
                                 "end": [f"r{r}" for r in ended]}))
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", dtype,
                           "--out", out_dir, "--max-tokens", str(pool)], input="\n".join(lines) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    vocab = TINY["C"][0]["vocab_size"]
    for i, (entries, ended) in enumerate(steps):
        got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, vocab))
        want = []
        for r, lo, hi in entries:
            want.append(refs[r][lo:hi] if (i + r) % 3 else refs[r][hi - 1:hi])
        logits_close(got, torch.cat(want), dtype, bound)
