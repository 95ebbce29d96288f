"""Command line in the reference's manner (src/cli.zig:1-125, src/llmgen.zig:35-492):

    python -m llmgen_b200 chat  [prompt] [max_new] [options]   generate and print `token ids: ...`
    python -m llmgen_b200 bench <workload.json>    [options]   run a workload, print a JSON summary
    python -m llmgen_b200 workload <out.json>      [options]   write a seeded random workload for `bench`
    python -m llmgen_b200 info --model <dir> | --random <config.json>   sizes, tensors checked, costs; no GPU needed
    python -m llmgen_b200 convert <model.gguf> <out_dir>       the reference's model file as a model folder; no GPU needed

Options keep the reference's names and meanings:
    --model <dir>  --temp <f>  --max-model-len <n>  --max-num-seqs <n>  --max-batched-tokens <n>
    --pass-tokens <n>  --block-size <n>  --gpu-util <f>  --kv-blocks <n>
    --policy prefill_first|chunked  --chunk <n>  --out <path>  --dup <n>  --eager  --sync-each
Added: --dtype bfloat16|float32, --seed <n>, --random <config.json | qwen3-0.6b | qwen3-8b | qwen3-32b> (random
weights drawn from --seed instead of a model folder; --init-on-device draws them on the GPU).  The model is a folder with config.json and model.safetensors
(default: environment variable LLMGEN_MODEL).
Environment, for `chat` (the reference's names): LLMGEN_PROFILE prints the time, FLOP/s and bytes/s
of every kernel by phase (eager steps); LLMGEN_METRICS prints TTFT, inter-token latencies and
throughputs with the model's FLOP and byte rates (shares of LLMGEN_PEAK_TFLOPS / LLMGEN_PEAK_GBPS
when given) and writes them as JSON to the path in LLMGEN_METRICS_JSON.
`workload` takes --scenario single|concurrent8|concurrent32|bench256|longctx (the reference's
bench/gen_workload.py scenarios) and / or --requests <n> --rounds <n> --input <n|lo:hi>
--output <n|lo:hi>, with --vocab <n>, --request-temp <f> and --seed; with --max-model-len given it
shortens outputs that would not fit.  It needs no GPU.

There is no tokenizer here (the engine's contract is token ids in, token ids out): the chat
prompt is a list of token ids, "12,7,99" or "12 7 99", or @file with a JSON list.  The
reference's REPL, --single and --no-kv-cache belong to its text edge and its legacy path and
are not offered.

Workload format (src/bench/workload.zig:6-16):
    {"name": ..., "rounds": [[{"prompt_ids": [...], "max_tokens": n, "temperature": 0.6,
                               "ignore_eos": true}, ...], ...]}
"""
from __future__ import annotations

import argparse
import json
import os
import resource
import statistics
import sys
import time
from typing import List

from .engine.scheduler import CHUNKED, PREFILL_FIRST


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="llmgen_b200", description="Single-GPU inference engine for sm_100a")
    ap.add_argument("cmd", choices=["chat", "bench", "workload", "info", "convert"])
    ap.add_argument("arg0", nargs="?", help="chat: prompt token ids; bench: workload.json; workload: the file to write")
    ap.add_argument("max_new", nargs="?", default=None, help="chat: most tokens to generate (default 2000); convert: the folder to write")
    ap.add_argument("--model", default=os.environ.get("LLMGEN_MODEL"))
    ap.add_argument("--random", metavar="CONFIG_JSON|NAME", help="draw random weights for this config.json (or a named shape: "
                    "qwen3-0.6b, qwen3-8b, qwen3-32b) instead of --model")
    ap.add_argument("--init-on-device", action="store_true", help="with --random: draw the weights on the GPU (other values "
                    "than the host's generator gives; for sizes that would take minutes on the host)")
    ap.add_argument("--seed", type=int, default=0x5EED)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--temp", type=float, default=0.0)
    ap.add_argument("--max-model-len", type=int, default=None, help="default 4096")
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-batched-tokens", type=int, default=16384)
    ap.add_argument("--pass-tokens", type=int, default=8192)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--gpu-util", type=float, default=0.9)
    ap.add_argument("--kv-blocks", type=int, default=0)
    ap.add_argument("--policy", choices=[PREFILL_FIRST, CHUNKED], default=PREFILL_FIRST)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--out")
    ap.add_argument("--dup", type=int, default=1)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--sync-each", action="store_true")
    wl = ap.add_argument_group("workload")
    wl.add_argument("--scenario", help="single, concurrent8, concurrent32, bench256 or longctx")
    wl.add_argument("--requests", type=int, help="requests per round")
    wl.add_argument("--rounds", type=int)
    wl.add_argument("--input", help="prompt length: N or LOW:HIGH")
    wl.add_argument("--output", help="tokens to generate: N or LOW:HIGH")
    wl.add_argument("--vocab", type=int, default=10001, help="token ids are drawn from [0, vocab)")
    wl.add_argument("--request-temp", type=float, default=0.6, help="temperature written into every request")
    return ap


def parse_prompt(text: str) -> List[int]:
    if text.startswith("@"):
        with open(text[1:], "r", encoding="utf-8") as f:
            return [int(t) for t in json.load(f)]
    return [int(t) for t in text.replace(",", " ").split()]


def random_config(text: str, max_model_len=None) -> dict:
    """A config.json file, or the name of a shape (models/shapes.py)."""
    if os.path.isfile(text):
        with open(text, "r", encoding="utf-8") as f:
            return json.load(f)
    from .models.shapes import named_shape
    try:
        return named_shape(text)
    except ValueError as e:
        raise SystemExit(f"--random: {text!r} is no file, and {e}")


def make_llm(args):
    from .engine.api import LLM, random_model
    if args.random:
        model = random_model(random_config(args.random, args.max_model_len), args.seed, args.dtype,
                             init_on_device=args.init_on_device)
    elif args.model:
        model = args.model
    else:
        raise SystemExit("no model: give --model <dir>, set LLMGEN_MODEL, or use --random <config.json>")
    return LLM(model, dtype=args.dtype, seed=args.seed, max_num_seqs=args.max_num_seqs,
               max_model_len=args.max_model_len, max_batched_tokens=args.max_batched_tokens,
               pass_tokens=args.pass_tokens, block_size=args.block_size, gpu_util=args.gpu_util,
               kv_blocks=args.kv_blocks, policy=args.policy, chunk=args.chunk, eager=args.eager,
               sync_each=args.sync_each)


def chat(args) -> int:
    from .sampling import SamplingParams
    if not args.arg0:
        raise SystemExit("chat needs a prompt: token ids such as \"12,7,99\" or @ids.json")
    prompt = parse_prompt(args.arg0)
    # the reference's switches (src/profiler/profiler.zig:95-101, src/profiler/metrics.zig:47-51): a table of
    # kernel times, which needs eager steps, and the latencies of the request with the model's efficiency
    profile = os.environ.get("LLMGEN_PROFILE") is not None
    metrics = None
    if profile:
        args.eager = True
    llm = make_llm(args)
    print(f"[load] {llm.load_seconds:.2f} s", file=sys.stderr)
    if profile:
        from .engine.profiler import OpProfiler
        llm.executor.profiler = OpProfiler().enable()
    if os.environ.get("LLMGEN_METRICS") is not None:
        from .engine.profiler import GenMetrics
        metrics = GenMetrics()
    room = args.max_model_len - len(prompt)
    params = SamplingParams(temperature=args.temp, max_tokens=max(1, min(args.max_new, room)), ignore_eos=False)
    t0 = time.perf_counter()
    if metrics is not None:
        metrics.start(len(prompt), t0)
    requests = [llm.engine.add_request(prompt, params) for _ in range(max(1, args.dup))]
    first = None
    while not llm.engine.is_finished():
        llm.engine.step()
        for r, tok in llm.engine.last_emitted:
            if r is requests[0]:
                now = time.perf_counter()
                if first is None:
                    first = now
                if metrics is not None:
                    metrics.on_token(now)
                print(tok, end=" ", flush=True)
    t1 = time.perf_counter()
    print()
    if metrics is not None:
        from .engine.profiler import ModelCost, efficiency_text
        metrics.finish(t1)
        elem = 2 if args.dtype == "bfloat16" else 4
        print(metrics.text(), file=sys.stderr)
        print(efficiency_text(metrics, ModelCost.from_spec(llm.model.spec, elem, elem)), file=sys.stderr)
        metrics.write_json()
    if profile:
        print(llm.executor.profiler.text(), file=sys.stderr)
        llm.executor.profiler.disable()
        llm.executor.profiler = None
    ids = requests[0].completion
    n = len(ids)
    if first is not None:
        per = (t1 - first) / max(1, n - 1) * 1e3
        print(f"[chat] TTFT {(first - t0) * 1e3:.1f} ms, {per:.2f} ms/token, {n} tokens", file=sys.stderr)
    print("token ids: " + " ".join(str(t) for t in ids))
    if args.dup > 1:
        # the reference's batch-consistency check: copies of one prompt must agree (greedy)
        if any(r.completion != ids for r in requests[1:]):
            print("error: outputs of duplicated requests differ", file=sys.stderr)
            return 1
        print(f"[chat] {args.dup} duplicated requests agree", file=sys.stderr)
    return 0


def percentiles(values: List[float]) -> dict:
    """numpy-style linear percentiles (src/bench/recorder.zig:5-40)."""
    if not values:
        return {"mean": 0.0, "p50": 0.0, "p90": 0.0, "p99": 0.0, "max": 0.0}
    v = sorted(values)

    def pct(p):
        k = (len(v) - 1) * p / 100.0
        lo = int(k)
        hi = min(lo + 1, len(v) - 1)
        return v[lo] + (v[hi] - v[lo]) * (k - lo)
    return {"mean": sum(v) / len(v), "p50": pct(50), "p90": pct(90), "p99": pct(99), "max": v[-1]}


def run_round(llm, reqs, ttft_ms, itl_ms) -> tuple:
    from .sampling import SamplingParams
    t0 = time.perf_counter()
    handles = [llm.engine.add_request(r["prompt_ids"], SamplingParams(
        temperature=float(r.get("temperature", 0.6)), max_tokens=int(r["max_tokens"]),
        ignore_eos=bool(r.get("ignore_eos", True)))) for r in reqs]
    steps = 0
    while not llm.engine.is_finished():
        llm.engine.step()
        steps += 1
    wall = time.perf_counter() - t0
    for h in handles:
        ttft_ms.append((h.first_token_time - h.arrival_time) * 1e3)
        itl_ms += [(b - a) * 1e3 for a, b in zip(h.token_times, h.token_times[1:])]
    llm.engine.release_finished()
    return wall, steps, sum(len(h.completion) for h in handles)


def bench(args) -> int:
    import torch
    from .sampling import SamplingParams
    if not args.arg0:
        raise SystemExit("bench needs a workload.json")
    with open(args.arg0, "r", encoding="utf-8") as f:
        wl = json.load(f)
    rounds = wl.get("rounds") or []
    if not rounds or not rounds[0]:
        raise SystemExit("empty workload")
    llm = make_llm(args)
    reqs0 = rounds[0]
    in_tok = sum(len(r["prompt_ids"]) for r in reqs0)
    print(f"[bench] {wl.get('name', '?')}: {len(reqs0)} requests x {len(rounds)} rounds, input {in_tok} tokens", file=sys.stderr)
    # warm-up, as the reference does: the first ids of request 0, 64 tokens at temperature 1
    warm = min(64, max(1, args.max_model_len - 8))
    llm.generate([reqs0[0]["prompt_ids"][:8]], SamplingParams(temperature=1.0, max_tokens=warm, ignore_eos=True))
    ex = llm.executor
    pre0, graph0, eager0 = llm.engine.scheduler.num_preemptions, ex.n_graph_steps, ex.n_eager_steps
    ttft_ms, itl_ms, walls, steps, out_tok = [], [], [], 0, 0
    for i, reqs in enumerate(rounds):
        wall, n, produced = run_round(llm, reqs, ttft_ms, itl_ms)
        walls.append(wall)
        steps += n
        if i == 0:
            out_tok = produced
        print(f"[bench] round {i + 1}: {wall:.3f} s, {produced / wall:.1f} tok/s", file=sys.stderr)
    leak = not ex.cache.all_free()
    if leak:
        print(f"[bench] cache pages leaked: free {ex.cache.num_free_pages()}", file=sys.stderr)
    wall = statistics.median(walls)
    free, total = torch.cuda.mem_get_info()
    pages = ex.cache.groups[0].pool.num_pages
    summary = {
        "engine": "llmgen_b200", "workload": wl.get("name", "?"), "n_requests": len(reqs0), "repeat": len(rounds),
        "input_tokens": in_tok, "output_tokens": out_tok, "wall_s": wall,
        "throughput_out": out_tok / wall, "throughput_total": (out_tok + in_tok) / wall,
        "ttft_ms": percentiles(ttft_ms), "itl_ms": percentiles(itl_ms),
        "peak_rss_mb": resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 1024.0,
        "device_used_mb": (total - free) / 2 ** 20, "weights_mb": llm.model.weight_bytes() / 2 ** 20,
        "kv_cache_mb": ex.storage.bytes_held() / 2 ** 20, "kv_tokens": pages * ex.limits.page_size,
        "load_s": llm.load_seconds, "graphs_captured": llm.graphs_captured, "preemptions": llm.engine.scheduler.num_preemptions - pre0, "steps": steps,
        "graph_steps": ex.n_graph_steps - graph0, "eager_steps": ex.n_eager_steps - eager0,
        "policy": args.policy, "dtype": args.dtype, "kv_leak": leak,
    }
    text = json.dumps(summary, indent=2)
    print(text)
    if args.out:
        with open(args.out, "w", encoding="utf-8") as f:
            f.write(text + "\n")
    return 0


def workload(args) -> int:
    from . import workload as wl
    if not args.arg0:
        raise SystemExit("workload needs the name of the file to write")
    try:
        name, shape = wl.resolve_shape(args.scenario, args.requests, args.rounds,
                                       wl.parse_range(args.input, "--input") if args.input else None,
                                       wl.parse_range(args.output, "--output") if args.output else None)
        made = wl.make_workload(name, shape, vocab=args.vocab, seed=args.seed, temperature=args.request_temp,
                                max_model_len=args.max_model_len)
    except wl.WorkloadError as e:
        raise SystemExit(f"workload: {e}")
    wl.write_workload(args.arg0, made)
    print(wl.summary(made), file=sys.stderr)
    return 0


def info(args) -> int:
    """The model's sizes and costs, and its tensors checked against what the model declares
    (the reference prints its sizes at start-up, src/models/qwen3.zig:406-419)."""
    from .config.base import ConfigError
    from .info import describe
    from .weights.loader import WeightError
    try:
        if args.random:
            text = describe(config=random_config(args.random), context=args.max_model_len or 4096)
        elif args.model:
            text = describe(model_dir=args.model, context=args.max_model_len or 4096)
        else:
            raise SystemExit("info needs --model <dir> (or LLMGEN_MODEL) or --random <config.json>")
    except (ConfigError, WeightError, OSError, ValueError) as e:
        print(f"info: {e}", file=sys.stderr)
        return 1
    print(text)
    return 0


def convert(args) -> int:
    """A GGUF file of the reference (F32, F16 or BF16 tensors) as config.json + model.safetensors."""
    from .config.base import ConfigError
    from .info import describe
    from .weights.gguf import GGUFError, convert_gguf
    from .weights.loader import WeightError
    if not args.arg0 or not args.max_new:
        raise SystemExit("convert needs the GGUF file and the folder to write")
    try:
        out = convert_gguf(args.arg0, args.max_new)
        print(describe(model_dir=out, context=args.max_model_len or 4096))
    except (GGUFError, ConfigError, WeightError, OSError) as e:
        print(f"convert: {e}", file=sys.stderr)
        return 1
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.cmd == "convert":
        return convert(args)
    try:
        args.max_new = 2000 if args.max_new is None else int(args.max_new)
    except ValueError:
        raise SystemExit(f"the number of tokens to generate must be an integer, not {args.max_new!r}")
    if args.cmd == "workload":
        return workload(args)
    if args.cmd == "info":
        return info(args)
    if args.max_model_len is None:
        args.max_model_len = 4096
    if args.sync_each:
        args.eager = True
    return chat(args) if args.cmd == "chat" else bench(args)
