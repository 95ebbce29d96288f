"""Generation through the Python entry point and the command line: greedy ids against the plain
implementation, both scheduling policies, preemption when pages run out, CUDA-graph replay
against eager steps, temperature sampling."""
import json
import os
import subprocess
import sys
import tempfile

import pytest
import torch

from tests.plain.qwen3_plain import PlainQwen3
from tests.util import ROOT, TINY, make_folder, random_ids, reference

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tmp():
    with tempfile.TemporaryDirectory() as d:
        yield d


def greedy_reference(path, prompts, n_new):
    m = PlainQwen3(path)
    return [m.greedy(p, n_new) for p in prompts]


@pytest.mark.parametrize("name,policy,eager", [("A", "prefill_first", False), ("A", "chunked", True),
                                               ("B", "chunked", False), ("C", "prefill_first", True)])
def test_greedy_generation_matches_plain(tmp, name, policy, eager):
    from llmgen_b200 import LLM, SamplingParams
    path = make_folder(tmp, name)
    vocab = TINY[name][0]["vocab_size"]
    prompts = [random_ids(n, vocab, 40 + i) for i, n in enumerate((5, 17, 33))]
    ref = greedy_reference(path, prompts, 16)
    llm = LLM(path, dtype="float32", max_model_len=128, max_num_seqs=4, max_batched_tokens=128, pass_tokens=64,
              block_size=TINY[name][5], kv_blocks=24, policy=policy, chunk=8, eager=eager)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    assert [o["token_ids"] for o in outs] == ref
    assert llm.executor.cache.all_free()
    if not eager:
        assert llm.executor.n_graph_steps > 0


def test_bfloat16_generation_runs_and_agrees_mostly(tmp):
    from llmgen_b200 import LLM, SamplingParams
    path = make_folder(tmp, "A")
    prompts = [random_ids(n, 256, 50 + i) for i, n in enumerate((9, 40))]
    ref = greedy_reference(path, prompts, 8)
    llm = LLM(path, dtype="bfloat16", max_model_len=128, max_num_seqs=4, max_batched_tokens=128, kv_blocks=16)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for o, r in zip(outs, ref):
        assert len(o["token_ids"]) == 8
        same = 0
        while same < 8 and o["token_ids"][same] == r[same]:
            same += 1
        assert same >= 7, f"bfloat16 ids {o['token_ids']} leave the plain ids {r} after {same} tokens"


def test_preemption_recomputes_and_gives_the_same_ids(tmp):
    """Five prompts, four sequences at a time, eight pages of 32 tokens: pages run out while
    decoding, the last running sequence is preempted and later computed again from position 0."""
    from llmgen_b200 import LLM, SamplingParams
    path = make_folder(tmp, "B")
    prompts = [random_ids(n, 384, 60 + i) for i, n in enumerate((1, 9, 40, 64, 100))]
    ref = greedy_reference(path, prompts, 40)
    for policy in ("chunked", "prefill_first"):
        llm = LLM(path, dtype="float32", max_model_len=256, max_num_seqs=4, max_batched_tokens=256, pass_tokens=256,
                  block_size=32, kv_blocks=8, policy=policy, chunk=16)
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
        assert llm.engine.scheduler.num_preemptions > 0
        assert [o["token_ids"] for o in outs] == ref
        assert llm.executor.cache.all_free()


@pytest.mark.parametrize("name,prompt_len,model_len", [("C", 21, 128), ("D", 21, 128), ("D", 505, 1024), ("E", 500, 1024)])
def test_graph_replay_equals_eager_and_duplicates_agree(tmp, name, prompt_len, model_len):
    """The reference's `--dup` check (src/llmgen.zig:229-240): copies of one prompt in one batch
    give identical ids; and graph replay gives what eager steps give.  D and E run the
    flash-decoding kernel; the long prompts cross a context-length class while decoding."""
    from llmgen_b200 import LLM, SamplingParams
    path = make_folder(tmp, name)
    prompt = random_ids(prompt_len, TINY[name][0]["vocab_size"], 70)
    outs = {}
    for eager in (False, True):
        llm = LLM(path, dtype="bfloat16", max_model_len=model_len, max_num_seqs=8, max_batched_tokens=8 * model_len,
                  kv_blocks=8 * model_len // TINY[name][5], block_size=TINY[name][5], eager=eager)
        res = llm.generate([prompt] * 5, SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True))
        assert all(r["token_ids"] == res[0]["token_ids"] for r in res)
        outs[eager] = res[0]["token_ids"]
        assert (llm.executor.n_graph_steps > 0) == (not eager)
    assert outs[False] == outs[True]


def test_temperature_sampling_is_seeded(tmp):
    from llmgen_b200 import LLM, SamplingParams
    path = make_folder(tmp, "B")
    prompts = [random_ids(n, 384, 80 + i) for i, n in enumerate((9, 40))]
    runs = []
    for seed in (7, 7, 8):
        llm = LLM(path, dtype="float32", seed=seed, max_model_len=256, max_num_seqs=4, max_batched_tokens=256,
                  block_size=32, kv_blocks=16, policy="chunked", chunk=16)
        runs.append([o["token_ids"] for o in llm.generate(prompts, SamplingParams(temperature=0.7, max_tokens=20, ignore_eos=True))])
    assert runs[0] == runs[1] and runs[0] != runs[2]
    greedy = greedy_reference(path, prompts, 20)
    assert runs[0] != greedy


def test_eos_ends_a_request(tmp):
    from llmgen_b200 import LLM, SamplingParams
    path = make_folder(tmp, "A")
    prompt = random_ids(12, 256, 90)
    ref = greedy_reference(path, [prompt], 10)[0]
    llm = LLM(path, dtype="float32", max_model_len=64, max_num_seqs=2, max_batched_tokens=64, kv_blocks=8)
    llm.engine.scheduler.config.eos_token_ids = (ref[4],)
    out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=10))[0]["token_ids"]
    stop = ref.index(ref[4])
    assert out == ref[:stop + 1]


def test_requests_that_cannot_be_served_are_refused(tmp):
    from llmgen_b200 import LLM, SamplingParams
    from llmgen_b200.engine.engine import EngineError
    path = make_folder(tmp, "A")
    llm = LLM(path, dtype="float32", max_model_len=64, max_num_seqs=2, max_batched_tokens=64, kv_blocks=4)
    with pytest.raises(EngineError, match="too long"):
        llm.engine.add_request([1] * 60, SamplingParams(max_tokens=10))
    with pytest.raises(EngineError, match="empty"):
        llm.engine.add_request([], SamplingParams(max_tokens=10))
    with pytest.raises(EngineError, match="vocabulary"):
        llm.engine.add_request([1, 256], SamplingParams(max_tokens=1))
    with pytest.raises(Exception, match="max_model_len"):
        LLM(path, dtype="float32", max_model_len=4096)            # beyond the model's positions


def test_steps_with_ids_outside_the_vocabulary_are_refused(tmp):
    """The step function checks every id before a kernel reads the table with it: lists, arrays, ids too
    large for 32 bits, negative ones and ones that are no integers; a good step still runs afterwards."""
    import numpy as np
    from llmgen_b200.engine.executor import StepEntry, StepError
    from tests.util import Driver
    d = Driver(make_folder(tmp, "A"), "float32", 128, 16)
    assert d.executor.admit("x") and d.executor.reserve("x", 0, 3)
    for bad in ([1, 2, 256], [1, -1, 3], [1, 2 ** 40, 3], [1, 2.5, 3], np.array([3, 4, 999]), [300]):
        with pytest.raises(StepError, match="vocabulary"):
            d.executor.step([StepEntry("x", bad, 0, [0])])
    d.executor.release("x")
    ids = random_ids(9, 256, 3)
    got = d.step([("y", ids, range(9))])
    assert float((got - PlainQwen3(make_folder(tmp, "A")).logits(ids)).abs().max()) < 1e-4
    got2 = d.step([("z", np.asarray(ids, dtype=np.int64), range(9))])          # ids as an array
    assert torch.equal(got, got2)


def test_command_line_chat_and_bench(tmp):
    path = make_folder(tmp, "A")
    prompt = random_ids(11, 256, 95)
    ref = greedy_reference(path, [prompt], 6)[0]
    cmd = [sys.executable, "-m", "llmgen_b200", "chat", ",".join(map(str, prompt)), "6", "--model", path,
           "--dtype", "float32", "--max-model-len", "64", "--kv-blocks", "8", "--max-num-seqs", "4",
           "--max-batched-tokens", "64", "--dup", "3"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("token ids:")][0]
    assert [int(x) for x in line.split(":")[1].split()] == ref
    workload = {"name": "tiny", "rounds": [[{"prompt_ids": random_ids(20, 256, 96 + i), "max_tokens": 8} for i in range(3)]] * 2}
    wl = os.path.join(tmp, "workload.json")
    with open(wl, "w") as f:
        json.dump(workload, f)
    out_json = os.path.join(tmp, "bench_out.json")
    cmd = [sys.executable, "-m", "llmgen_b200", "bench", wl, "--model", path, "--max-model-len", "128",
           "--kv-blocks", "32", "--max-num-seqs", "4", "--max-batched-tokens", "128", "--policy", "chunked",
           "--chunk", "16", "--out", out_json]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    summary = json.load(open(out_json))
    assert summary["n_requests"] == 3 and summary["output_tokens"] == 24 and summary["throughput_out"] > 0
    assert summary["policy"] == "chunked" and summary["kv_leak"] is False


@pytest.mark.parametrize("hidden,heads,kv_heads,inter", [(4096, 32, 8, 12288), (5120, 64, 8, 25600)])
def test_layer_sizes_of_the_larger_models(tmp, hidden, heads, kv_heads, inter):
    """One layer with the sizes of the 8B and 32B Qwen3 models (32 or 64 query heads on 8 kv heads of
    128: groups of 4 and 8, a q width that is not the hidden size, intermediate sizes of 12,288 and
    25,600) and a vocabulary that is no multiple of 128: bfloat16 logits of a prompt, of a portion
    beside a decoded token and of decoded tokens against the plain implementation, and graph replay
    against eager steps."""
    from llmgen_b200 import LLM, SamplingParams
    from llmgen_b200.engine.api import write_random_model
    from tests.util import Driver, logits_close
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 1500, "hidden_size": hidden,
           "intermediate_size": inter, "num_hidden_layers": 1, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
           "head_dim": 128, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 1024,
           "tie_word_embeddings": False, "hidden_act": "silu"}
    path = os.path.join(tmp, f"wide_{hidden}")
    write_random_model(path, cfg, 11, 0.02, 0.1, "bfloat16")
    ids = random_ids(300, 1500, 5)
    ids_b = random_ids(60, 1500, 6)
    (ref, bound_a), (ref_b, bound_b) = reference(path, ids), reference(path, ids_b)
    bound = max(bound_a, bound_b)
    from tests.util import forget_plain_models
    forget_plain_models()
    d = Driver(path, "bfloat16", 512, 16)
    got = d.step([("a", ids[:280], range(280))])
    logits_close(got, ref[:280], "bfloat16", bound)
    got = d.step([("b", ids_b[:40], range(40)), ("a", ids[280:281], [0])])       # 41 rows: a portion beside a decoded token
    logits_close(got[:40], ref_b[:40], "bfloat16", bound)
    logits_close(got[40:], ref[280:281], "bfloat16", bound)
    for i in range(19):                                                          # then both decode
        got = d.step([("a", ids[281 + i:282 + i], [0])] + ([("b", ids_b[40 + i:41 + i], [0])] if 40 + i < 60 else []))
        logits_close(got[:1], ref[281 + i:282 + i], "bfloat16", bound)
        if got.shape[0] > 1:
            logits_close(got[1:], ref_b[40 + i:41 + i], "bfloat16", bound)
    outs = {}
    for eager in (False, True):
        llm = LLM(path, dtype="bfloat16", max_model_len=512, max_num_seqs=4, max_batched_tokens=2048, kv_blocks=128, eager=eager)
        outs[eager] = [r["token_ids"] for r in llm.generate([ids[:200], ids[:37]], SamplingParams(0.0, 12, True))]
    assert outs[False] == outs[True]


def test_decode_steps_launched_one_ahead_give_what_steps_read_at_once_give(tmp):
    """The engine launches a decode step before it has read the ids of the step before (the GPU takes
    them from where that step left them).  Same ids as with `run_ahead` off: with requests that end at
    different times (so rows move between steps and batch sizes change), with an end-of-sequence token
    that is only seen after one more step was launched, and with so few pages that requests are preempted."""
    from llmgen_b200 import LLM, SamplingParams
    path = make_folder(tmp, "A")
    prompts = [random_ids(n, 256, 120 + i) for i, n in enumerate((3, 11, 30, 7, 19))]
    params = [SamplingParams(temperature=0.0, max_tokens=m, ignore_eos=True) for m in (5, 23, 9, 30, 16)]
    ref = greedy_reference(path, prompts, 30)
    outs = {}
    for ahead in (True, False):
        llm = LLM(path, dtype="float32", max_model_len=96, max_num_seqs=4, max_batched_tokens=96, kv_blocks=7)
        llm.engine.run_ahead = ahead
        outs[ahead] = [o["token_ids"] for o in llm.generate(prompts, params)]
        assert llm.executor.cache.all_free() and llm.executor.n_graph_steps > 0
        if ahead:
            assert llm.engine.scheduler.num_preemptions > 0
    assert outs[True] == outs[False] == [r[:p.max_tokens] for r, p in zip(ref, params)]
    # an end-of-sequence token: the request's list stops there although the next step had been launched
    stop = ref[1][6]
    first = ref[1].index(stop)
    llm = LLM(path, dtype="float32", max_model_len=128, max_num_seqs=4, max_batched_tokens=128, kv_blocks=32)
    llm.engine.scheduler.config.eos_token_ids = (stop,)
    got = llm.generate(prompts[:3], [SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=(i != 1)) for i in range(3)])
    assert got[1]["token_ids"] == ref[1][:first + 1]
    assert got[0]["token_ids"] == ref[0][:20] and got[2]["token_ids"] == ref[2][:20]
    assert llm.executor.cache.all_free()


def test_decode_launch_takes_ids_from_the_rows_of_the_step_before(tmp):
    """`Executor.decode_launch` with `prev_rows`: the rows change places between steps and one row gets
    its id from the host; compared with steps that are given every id."""
    from llmgen_b200.engine.executor import StepEntry
    from tests.util import Driver
    path = make_folder(tmp, "E")
    prompts = {r: random_ids(n, 290, 130 + i) for i, (r, n) in enumerate((("a", 9), ("b", 21), ("c", 5)))}
    runs = {}
    for fed in (False, True):
        d = Driver(path, "bfloat16", 512, 32)
        d.executor.eager = False
        pos, last = {}, {}
        for r, ids in prompts.items():
            d.step([(r, ids, [])])
            pos[r], last[r] = len(ids), ids[-1] % 7 + 1
        orders = [["a", "b", "c"], ["c", "a", "b"], ["b", "c"], ["c", "b", "a"], ["a", "b", "c"]]
        got, rows_before, pending = [], {}, None
        for order in orders:
            entries, prev = [], []
            for r in order:
                assert d.executor.reserve(r, pos[r], pos[r] + 1)
                row = rows_before.get(r, -1) if fed else -1
                entries.append(StepEntry(r, [None] if row >= 0 else [last[r]], pos[r], [0], 0.0))
                prev.append(row)
                pos[r] += 1
            launched = d.executor.decode_launch(entries, prev if fed else None)
            if pending is not None and fed:
                ids = d.executor.decode_collect(pending[0])           # read only after the next launch
                got.append(dict(zip(pending[1], ids)))
                last.update(got[-1])
            if fed:
                pending, rows_before = (launched, order), {r: i for i, r in enumerate(order)}
            else:
                ids = d.executor.decode_collect(launched)
                got.append(dict(zip(order, ids)))
                last.update(got[-1])
        if fed:
            got.append(dict(zip(pending[1], d.executor.decode_collect(pending[0]))))
        runs[fed] = got
    # "a" sits out the third step: in the fed run its id for the fourth comes from the host (known by then)
    assert runs[True] == runs[False]


@pytest.mark.parametrize("seed", [1, 2, 3])
@pytest.mark.parametrize("policy", ["prefill_first", "chunked"])
def test_random_requests_give_the_same_ids_one_step_ahead_and_not(tmp, seed, policy):
    """Random prompts and lengths, an end-of-sequence token that is hit often, so few pages that requests are
    preempted: greedy ids with decode steps launched one ahead equal those with every step read at once, and
    every completion stops at its first end-of-sequence token or at max_tokens."""
    import random
    from llmgen_b200 import LLM, SamplingParams
    path = make_folder(tmp, "A")
    rng = random.Random(seed)
    prompts = [random_ids(rng.randint(1, 40), 256, 200 + 10 * seed + i) for i in range(9)]
    params = [SamplingParams(temperature=0.0, max_tokens=rng.randint(1, 30), ignore_eos=rng.random() < 0.3) for _ in prompts]
    ref = greedy_reference(path, prompts, 30)
    # an end-of-sequence id that several completions contain
    counts = {}
    for r in ref:
        for t in set(r):
            counts[t] = counts.get(t, 0) + 1
    eos = max(counts, key=lambda t: (counts[t], -t))
    want = []
    for r, p in zip(ref, params):
        out = r[:p.max_tokens]
        if not p.ignore_eos and eos in out:
            out = out[:out.index(eos) + 1]
        want.append(out)
    outs = {}
    for ahead in (True, False):
        llm = LLM(path, dtype="float32", max_model_len=96, max_num_seqs=4, max_batched_tokens=96, kv_blocks=8, policy=policy, chunk=16)
        llm.engine.run_ahead = ahead
        llm.engine.scheduler.config.eos_token_ids = (eos,)
        outs[ahead] = [o["token_ids"] for o in llm.generate(prompts, params)]
        assert llm.executor.cache.all_free()
    assert outs[True] == outs[False] == want


def test_sampled_steps_cut_into_passes_give_the_ids_of_one_pass(tmp):
    """`Executor.step(sample=True)` with more tokens than a pass holds: the step is cut into three passes, want
    lists are out of order, some rows are greedy and some drawn at a temperature.  The ids are those of the same
    step run as one pass (a draw depends on the request and the position, not on the pass or the row)."""
    from llmgen_b200.engine.api import load_model
    from llmgen_b200.engine.executor import EngineLimits, Executor, StepEntry
    path = make_folder(tmp, "B")
    prompts = {"x": random_ids(70, 384, 301), "y": random_ids(45, 384, 302), "z": random_ids(33, 384, 303)}
    wants = {"x": [69, 3, 30], "y": [44, 0], "z": [32]}
    temps = {"x": 0.8, "y": 0.0, "z": 1.3}
    model = load_model(path, "float32")
    got = {}
    for cap in (256, 64):
        ex = Executor(model, EngineLimits(max_num_seqs=4, max_model_len=128, max_step_tokens=cap, page_size=32,
                                          num_pages=16), seed=77, eager=True)
        entries = []
        for r, ids in prompts.items():
            assert ex.admit(r) and ex.reserve(r, 0, len(ids))
            entries.append(StepEntry(r, ids, 0, wants[r], temps[r]))
        assert len(ex._passes(entries)) == (1 if cap == 256 else 3)
        out = ex.step(entries, sample=True, return_logits=True)
        got[cap] = (out.token_ids, out.logits.cpu())
    assert got[256][0] == got[64][0] and len(got[64][0]) == 6
    assert float((got[256][1] - got[64][1]).abs().max()) < 1e-5
    # greedy rows are the plain argmax
    ref = PlainQwen3(path).logits(prompts["y"])
    assert got[64][0][3:5] == [int(ref[44].argmax()), int(ref[0].argmax())]


@pytest.mark.parametrize("n_live,bucket", [(40, 48), (100, 112)])
def test_many_live_sequences_match_plain_greedy_ids(tmp, n_live, bucket):
    """40 and 100 sequences decoding together (graph buckets 48 and 112, padded rows beside live ones, decode
    attention with fewer blocks than sequences x heads would fill twice over) in float32 against plain greedy
    ids; the sequences end at different lengths, so the batch shrinks through smaller buckets."""
    from llmgen_b200 import LLM, SamplingParams
    import random
    path = make_folder(tmp, "A")
    rng = random.Random(n_live)
    prompts = [random_ids(rng.randint(1, 24), 256, 500 + i) for i in range(n_live)]
    lengths = [rng.randint(3, 10) for _ in prompts]
    plain = PlainQwen3(path)
    ref = [plain.greedy(p, n) for p, n in zip(prompts, lengths)]
    llm = LLM(path, dtype="float32", max_model_len=64, max_num_seqs=128, max_batched_tokens=4096, kv_blocks=512)
    assert bucket in llm.executor.buckets()
    outs = llm.generate(prompts, [SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True) for n in lengths])
    assert [o["token_ids"] for o in outs] == ref
    assert llm.executor.n_graph_steps > 0 and bucket in {b for (b, c) in llm.executor.graphs}
    assert llm.executor.cache.all_free()


def test_temperature_ids_do_not_depend_on_steps_launched_ahead_nor_on_the_batch(tmp):
    """A draw's random numbers come from (seed, request, position): the same ids with decode steps launched one
    ahead and not (an end-of-sequence token and preemptions change which rows a step has and how many steps
    run), with the requests submitted alone one after the other, and they are the plain sampler's ids."""
    from llmgen_b200 import LLM, SamplingParams
    from llmgen_b200.engine.executor import SEED_STRIDE
    from tests.plain import qwen3_plain as plain
    path = make_folder(tmp, "B")
    prompts = [random_ids(n, 384, 600 + i) for i, n in enumerate((4, 19, 33, 8, 27))]
    params = [SamplingParams(temperature=t, max_tokens=m, ignore_eos=False) for t, m in ((0.7, 30), (1.1, 40), (0.4, 35), (0.9, 45), (0.7, 38))]
    seed = 4242

    def run(ahead, eos=(), kv_blocks=5):
        llm = LLM(path, dtype="float32", seed=seed, max_model_len=128, max_num_seqs=4, max_batched_tokens=128,
                  block_size=32, kv_blocks=kv_blocks, policy="chunked", chunk=16)
        llm.engine.run_ahead = ahead
        llm.engine.scheduler.config.eos_token_ids = tuple(eos)
        outs = llm.generate(prompts, params)
        assert llm.executor.cache.all_free()
        return [o["token_ids"] for o in outs], llm.engine.scheduler.num_preemptions

    free, _ = run(True, kv_blocks=32)
    eos = free[1][7]                                    # a token the second request draws: it ends there
    a, pre_a = run(True, eos=[eos])
    b, pre_b = run(False, eos=[eos])
    assert a == b and pre_a > 0
    assert a[1] == free[1][:free[1].index(eos) + 1]
    # the plain sampler with the same keys: step seed = seed + stride * (position + 1), row = the request's number
    model = PlainQwen3(path)
    for rid, (prompt, p, ids) in enumerate(zip(prompts, params, a)):
        seq = list(prompt)
        for tok in ids:
            logits = model.logits(seq)[-1]
            step_seed = (seed + SEED_STRIDE * len(seq)) & ((1 << 64) - 1)
            scores = plain.gumbel_scores(logits, p.temperature, step_seed, rid)
            top = scores.topk(2)
            assert tok == int(top.indices[0]) or float(top.values[0] - top.values[1]) < 1e-4
            seq.append(tok)


def test_steps_of_prompts_replay_the_graphs_of_their_shapes(tmp):
    """Every step that is not all single tokens is rounded up to a shape (token rows, sequences) and replays that
    shape's graph: the shapes cover every step up to the limit, all graphs exist once the engine is built (a run
    captures none), chunked prompts beside decoding requests give the ids of the engine that launches kernel by
    kernel, and a reservation beyond max_model_len is refused before it can widen a block table."""
    from llmgen_b200 import LLM, SamplingParams
    from llmgen_b200.engine.executor import StepEntry, StepError
    path = make_folder(tmp, "E")
    prompts = [random_ids(n, 290, 300 + i) for i, n in enumerate((150, 9, 77, 230, 31))]
    params = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    outs = {}
    for eager in (False, True):
        llm = LLM(path, dtype="bfloat16", max_model_len=512, max_num_seqs=4, max_batched_tokens=96, kv_blocks=64, block_size=32,
                  policy="chunked", chunk=40, eager=eager)
        ex = llm.executor
        if not eager:
            shapes = ex.token_shapes()
            assert shapes == sorted(set(shapes)) and shapes[-1] == min(ex.limits.max_step_tokens, ex.SHAPED_TOKENS_MAX)
            assert ex.step_shape([StepEntry("x", [1] * 17, 0)]) == (32, 4)
            assert ex.step_shape([StepEntry("x", [1] * shapes[-1], 0)]) == (shapes[-1], 4)
            assert ex.step_shape([StepEntry("x", [1] * (shapes[-1] + 1), 0)]) is None
            captured = len(ex.shape_graphs)
            assert ex.shaped_steps and captured == len(shapes) * len(ex.seq_shapes()) and llm.graphs_captured >= captured
        outs[eager] = [r["token_ids"] for r in llm.generate(prompts, params)]
        if not eager:
            assert ex.n_shaped_steps > 0 and len(ex.shape_graphs) == captured
            with pytest.raises(StepError, match="max_model_len"):
                ex.admit("far") and ex.reserve("far", 0, 513)
            ex.release("far")
        assert ex.cache.all_free()
    agree = sum(sum(x == y for x, y in zip(a, b)) for a, b in zip(outs[False], outs[True]))
    assert agree >= 0.9 * sum(len(a) for a in outs[True]), (agree, outs)
