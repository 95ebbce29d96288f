#!/usr/bin/env python3
"""Benchmark of the engine's decode step and prefill on one B200, at the Qwen3-0.6B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]
                    [--shape 0.6b|8b|32b --layers L]      (other layer sizes, beside the default run)
    python bench.py --kernels [--kernels-out FILE.md]     (kernel by kernel beside the reference's own kernels)

Prints ONE JSON line.  A "step" is one decode step of `--batch` sequences (default 8) whose
prompts are 512 uniform-random token ids; weights are random (seed 2), bfloat16.

  value     decoded tokens per second, timed on the device with CUDA events over exactly K decode
            steps through the executor's launch interface (arrays filled and uploaded, graph
            replayed, ids sampled and handed to the next step on the device, read one step late),
            after W warm-up steps.  Contexts grow from 512 + W upward.
  e2e       the same through the Python entry point (`Engine.step`): every step copies its
            metadata from pinned host memory to the device and reads the sampled ids back.
  prefill   one 2,048-token prompt through one step: tokens/s, ms, and flops / time / the measured
            bf16 peak.
  roofline  the decode step against HBM: bytes it has to read (every weight once, the cache of the
            live requests) / its time / the measured copy bandwidth.
  points    decode tokens/s at batch 1 and 64.
  mixed_step  8 decoded tokens beside a 64-token portion of a prompt in one step (launched kernel by kernel
            from the host): wall ms and the ms between CUDA events.
  load_s    engine construction with cache, workspaces and the capture of every decode graph.

Inputs are larger than L2 (1.19 GB of weights per step against 126 MB), so nothing is flushed
between timed iterations.  The reference (Zig + CUDA for sm_86) cannot be built or installed
here, so `--impl reference` reports that it is unavailable.  Its CUDA kernels, however, are plain
`extern "C"` functions: baseline/build_reference_kernels.py compiles them unmodified for sm_100a, and
`--kernels` times them beside this engine's kernels on the same GPU, shapes and loop
(baseline/kernel_compare.py); that mode prints one JSON line of its own and is no part of the default run.
"""
import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: "Qwen3-0.6B shape ... 28 layers, hidden 1024, 16 q heads, 8 kv heads,
# head_dim 128, intermediate 3072 SwiGLU, vocab 151936, rope_theta 1,000,000, rms_eps 1e-6,
# q/k RMSNorm, tied embeddings, full attention", benchmarked at max_model_len 4096; configs[3] and [4]: the layer
# sizes of Qwen3-8B and Qwen3-32B, for runs beside the default one (`--shape 8b --layers 8`).
from llmgen_b200.models.shapes import QWEN3_SHAPES  # noqa: E402

QWEN3_0_6B = QWEN3_SHAPES["qwen3-0.6b"]
SHAPES = {"0.6b": ("Qwen3-0.6B shape", QWEN3_0_6B), "8b": ("Qwen3-8B shape", QWEN3_SHAPES["qwen3-8b"]),
          "32b": ("Qwen3-32B shape", QWEN3_SHAPES["qwen3-32b"])}
CONTEXT = 4096
PROMPT_TOKENS = 512
PREFILL_TOKENS = 2048
SEED = 2
PUBLISHED_B8 = 1666.0      # the reference's published decode rate nearest to this run: 8 requests, RTX 3090 (tokens/s)


def check_against_baseline_json():
    """The sizes above are those BASELINE.json names; fail loudly if the file says otherwise."""
    path = os.path.join(ROOT, "BASELINE.json")
    if not os.path.isfile(path):
        return
    text = json.load(open(path))["configs"][2]
    pats = {"num_hidden_layers": r"(\d+) layers", "hidden_size": r"hidden (\d+)", "num_attention_heads": r"(\d+) q heads",
            "num_key_value_heads": r"(\d+) kv heads", "head_dim": r"head_dim (\d+)", "intermediate_size": r"intermediate (\d+)",
            "vocab_size": r"vocab (\d+)"}
    for key, pat in pats.items():
        m = re.search(pat, text)
        if m and int(m.group(1)) != QWEN3_0_6B[key]:
            raise SystemExit(f"bench.py: BASELINE.json configs[2] gives {key}={m.group(1)}, bench has {QWEN3_0_6B[key]}")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def mark(self):
        return time.perf_counter()

    def stop(self, windows):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.lines:
            if not any(a <= t <= b + 0.15 for a, b in windows):
                continue
            f = [x.strip() for x in line.split(",")]
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, f[2:]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:      # the timed regions were shorter than a sampling period: use every sample
            for t, line in self.lines:
                f = [x.strip() for x in line.split(",")]
                try:
                    sm.append(float(f[0]))
                    mx.append(float(f[1]))
                except (ValueError, IndexError):
                    pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, n_layers):
    """Bytes and flops of the model as executed (bfloat16)."""
    H, hd, nq, nkv = cfg["hidden_size"], cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    F, V = cfg["intermediate_size"], cfg["vocab_size"]
    per_layer = (nq + 2 * nkv) * hd * H + H * nq * hd + 3 * F * H
    mm_params = n_layers * per_layer
    norm_params = n_layers * (2 * H + 2 * hd) + H
    weight_bytes = 2 * (mm_params + V * H) + 4 * norm_params     # lm_head = the tied table, read whole once
    kv_bytes_per_token = n_layers * 2 * nkv * hd * 2
    return {"mm_params": mm_params, "weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token,
            "per_layer_params": per_layer}


def prefill_flops(cfg, n_layers, P):
    nums = model_numbers(cfg, n_layers)
    gemm = 2 * nums["mm_params"] * P + 2 * cfg["vocab_size"] * cfg["hidden_size"]      # lm_head on one row
    attn = 4 * n_layers * cfg["num_attention_heads"] * cfg["head_dim"] * P * (P + 1) // 2
    return gemm + attn


def kernels_table(args):
    """Kernel by kernel beside the reference's own kernels recompiled for sm_100a; one JSON line."""
    from baseline import reference_kernels as ref
    if not ref.available():
        print(json.dumps({"kernels": None, "unavailable": "baseline/_ref holds no library of the reference's kernels: run "
                          "baseline/build_reference_kernels.py --src <checkout of the reference> first"}))
        return 0
    import torch
    from llmgen_b200.engine.api import require_cuda
    from llmgen_b200.kernels import build as kernel_build
    from baseline import kernel_compare
    require_cuda()
    kernel_build.ensure_built(["elementwise", "attn_prep", "attention_decode", "attention_tc", "gemm_skinny", "gemm_tc"])
    sampler = ClockSampler()
    sampler.start()
    w0 = sampler.mark()
    rows = kernel_compare.run_all()
    clocks = sampler.stop([(w0, sampler.mark())])
    table = kernel_compare.as_markdown(rows)
    if args.kernels_out:
        os.makedirs(os.path.dirname(os.path.abspath(args.kernels_out)), exist_ok=True)
        with open(args.kernels_out, "w") as f:
            f.write(table + "\n")
    print(table, file=sys.stderr)
    print(json.dumps({"kernels": rows, "gpu": torch.cuda.get_device_name(0), "clocks": clocks}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (named in config)")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="0.6b",
                    help="layer sizes of another model than the default run's (use with --layers where time needs it)")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--prompt-tokens", type=int, default=PROMPT_TOKENS,
                    help="for other context lengths than the default run's: the prompts' length (prompts of a batch are "
                         "then computed one by one)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="the engine's longest sequence")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true", help="for profiling runs: leave the prefill measurement out")
    ap.add_argument("--skip-e2e", action="store_true", help="for profiling runs: leave the end-to-end measurement out")
    ap.add_argument("--rates", action="store_true",
                    help="print the device's tcgen05.mma, TMA and exponential rates (baseline/device_rates.py) and exit")
    ap.add_argument("--lazy-graphs", action="store_true",
                    help="for profiling runs: capture each CUDA graph when it is first used, not all of them at start")
    ap.add_argument("--mixed", default="", metavar="DECODING,PORTION,REPEATS",
                    help="for profiling runs: only steps of DECODING single tokens beside a portion of PORTION tokens")
    ap.add_argument("--kernels", action="store_true",
                    help="time this engine's kernels beside the reference's (baseline/_ref, built by baseline/build_reference_kernels.py)")
    ap.add_argument("--kernels-out", default="", help="with --kernels: also write the table as markdown to this file")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "AIxSpace/llmgen is a Zig 0.15 + CUDA (sm_86) program: no Zig "
                          "compiler is installed and pip reports 'Neither setup.py nor pyproject.toml found', so it "
                          "cannot be installed or run here; its CUDA kernels alone are compiled for sm_100a and timed "
                          "beside this engine's by `bench.py --kernels` (profiles/reference_kernels_on_b200.md)"}))
        return 0
    if args.kernels:
        return kernels_table(args)
    if args.rates:
        from baseline import device_rates
        sys.stdout.write(device_rates.run())
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.shape == "0.6b":
        check_against_baseline_json()
    warmup = max(3, args.warmup)
    K = max(1, args.steps)

    import numpy as np
    import torch
    from llmgen_b200.engine.api import LLM, random_model
    from llmgen_b200.engine.executor import StepEntry
    from llmgen_b200.kernels import ops
    from llmgen_b200.sampling import SamplingParams

    shape_name, shape_cfg = SHAPES[args.shape]
    cfg = dict(shape_cfg)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n_layers = cfg["num_hidden_layers"]
    pk = peaks()
    nums = model_numbers(cfg, n_layers)
    rng = np.random.default_rng(SEED)
    model = random_model(cfg, SEED, "bfloat16")
    llm = LLM(model, max_num_seqs=64, max_model_len=args.context, max_batched_tokens=16384, pass_tokens=8192,
              block_size=args.block_size, gpu_util=0.5, seed=SEED,
              capture_at_start=not (args.mixed or args.lazy_graphs))
    ex = llm.executor
    V = cfg["vocab_size"]
    sampler = ClockSampler()
    sampler.start()
    windows = []

    def device_decode(batch, warm, steps):
        """K decode steps through the executor's launch interface, timed with CUDA events: every step fills and
        uploads its arrays, replays its graph, samples, and hands its ids to the next step on the device (the
        step after is launched before this one's ids are read, as the engine does).  Returns (ms per step, mean
        context, launches per step)."""
        reqs = [f"dev{batch}_{i}" for i in range(batch)]
        P = args.prompt_tokens
        total = P + warm + steps + 1
        prompts = [rng.integers(0, V, P).tolist() for _ in range(batch)]
        for r in reqs:
            assert ex.admit(r) and ex.reserve(r, 0, total)
        if P * batch <= 65536:
            first_ids = ex.step([StepEntry(r, p, 0, [P - 1], 0.6) for r, p in zip(reqs, prompts)], sample=True, return_logits=False).token_ids
        else:
            first_ids = [ex.step([StepEntry(r, p, 0, [P - 1], 0.6)], sample=True, return_logits=False).token_ids[0]
                         for r, p in zip(reqs, prompts)]
        state = {"pos": P, "pending": None}
        rows = list(range(batch))
        launches_before, graph_steps_before = ex.launch_count, ex.n_graph_steps

        def one():
            pos = state["pos"]
            if state["pending"] is None:
                entries = [StepEntry(r, [t], pos, [0], 0.6) for r, t in zip(reqs, first_ids)]
                launched = ex.decode_launch(entries, None)
            else:
                entries = [StepEntry(r, [None], pos, [0], 0.6) for r in reqs]
                launched = ex.decode_launch(entries, rows)
                ex.decode_collect(state["pending"])          # the ids of the step before, read one step late
            state["pending"], state["pos"] = launched, pos + 1
        for _ in range(warm):
            one()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = sampler.mark()
        start.record()
        first = state["pos"]
        for _ in range(steps):
            one()
        end.record()
        torch.cuda.synchronize()
        windows.append((w0, sampler.mark()))
        ex.decode_collect(state["pending"])
        ms = start.elapsed_time(end) / steps
        # kernels of this package that every replayed step launches (counted when its graph was recorded)
        per_step = (ex.launch_count - launches_before) // max(1, ex.n_graph_steps - graph_steps_before)
        for r in reqs:
            ex.release(r)
        return ms, (first + 1 + state["pos"]) / 2.0, per_step

    def mixed_step(decoding=8, portion=64, repeats=20):
        """A step of the kind the chunked policy makes: `decoding` single tokens beside one portion of a prompt.
        The layers of such a step are replayed from the CUDA graph of its shape; wall time against device time shows
        what the host costs."""
        reqs = [f"mix{i}" for i in range(decoding)]
        if decoding + 1 > ex.limits.max_num_seqs:
            raise SystemExit(f"--mixed: {decoding} single tokens and a portion are {decoding + 1} sequences; "
                             f"--batch {ex.limits.max_num_seqs} admits no more than that many")
        for r in reqs:
            assert ex.admit(r) and ex.reserve(r, 0, 512 + repeats + 3)
        assert ex.admit("mixp") and ex.reserve("mixp", 0, (repeats + 3) * portion)
        ex.step([StepEntry(r, rng.integers(0, V, 512).tolist(), 0, [511], 0.6) for r in reqs], sample=True, return_logits=False)
        dev, wall = [], []
        for i in range(repeats + 3):
            entries = [StepEntry(r, [7], 512 + i, [0], 0.6) for r in reqs]
            entries.append(StepEntry("mixp", rng.integers(0, V, portion).tolist(), i * portion, [], 0.6))
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            start.record()
            ex.step(entries, sample=True, return_logits=False)
            end.record()
            torch.cuda.synchronize()
            if i >= 3:
                wall.append((time.perf_counter() - t0) * 1e3)
                dev.append(start.elapsed_time(end))
        for r in reqs + ["mixp"]:
            ex.release(r)
        return {"tokens": decoding + portion, "ms": statistics.median(wall), "ms_device_events": statistics.median(dev)}

    if args.mixed:
        d, p, r = (int(x) for x in args.mixed.split(","))
        print(json.dumps({"mixed_step": mixed_step(d, p, r), "shaped_steps": ex.n_shaped_steps}))
        return 0

    # ---- prefill: one 2,048-token prompt, one step
    def prefill_once():
        ids = rng.integers(0, V, PREFILL_TOKENS).tolist()
        assert ex.admit("prefill") and ex.reserve("prefill", 0, PREFILL_TOKENS)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        w0 = sampler.mark()
        start.record()
        ex.step([StepEntry("prefill", ids, 0, [PREFILL_TOKENS - 1], 0.6)], sample=True, return_logits=False)
        end.record()
        torch.cuda.synchronize()
        windows.append((w0, sampler.mark()))
        ex.release("prefill")
        return start.elapsed_time(end)
    prefill = None
    if not args.skip_prefill:
        for _ in range(3):
            prefill_once()
        prefill_ms = statistics.median(prefill_once() for _ in range(5))
        pf = prefill_flops(cfg, n_layers, PREFILL_TOKENS)
        prefill = {"value": PREFILL_TOKENS / (prefill_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": prefill_ms,
                   "frac": pf / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12)}

    # ---- the decode step on the device
    ms_step, mean_ctx, launches_per_step = device_decode(args.batch, warmup, K)
    value = args.batch / (ms_step / 1e3)
    step_bytes = nums["weight_bytes"] + args.batch * mean_ctx * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"]}

    # ---- end to end through the entry point: host token ids in, host token ids out, every step
    e2e = None
    if not args.skip_e2e:
        prompts = [rng.integers(0, V, args.prompt_tokens).tolist() for _ in range(args.batch)]
        params = SamplingParams(temperature=0.6, max_tokens=warmup + K + 2, ignore_eos=True)
        for p in prompts:
            llm.engine.add_request(p, params)
        llm.engine.step()                       # the prompts
        for _ in range(warmup):
            llm.engine.step()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = sampler.mark()
        t0 = time.perf_counter()
        start.record()
        emitted = 0
        for _ in range(K):
            llm.engine.step()
            emitted += len(llm.engine.last_emitted)
        end.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        windows.append((w0, sampler.mark()))
        e2e_ms = max(start.elapsed_time(end), wall * 1e3)
        llm.engine.run_until_done()
        llm.engine.release_finished()
        # every step copies its packed arrays up (ids, positions, lengths, slots, block tables, sampler keys ...) and its
        # sampled ids and the kernels' two status flags down
        e2e = {"value": emitted / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": ex.last_upload_bytes,
               "d2h_bytes_per_step": 4 * args.batch + 8}

    points = {}
    mixed = None
    if not args.skip_points:
        for b in (1, 64):
            ms_b, _, _ = device_decode(b, warmup, K)
            points[f"decode_b{b}"] = b / (ms_b / 1e3)
        mixed = mixed_step()
    clocks = sampler.stop(windows)

    line = {
        "metric": f"decode tok/s at batch {args.batch} ({shape_name}, bf16, random weights, {args.prompt_tokens}-token prompts)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": value / PUBLISHED_B8 if args.shape == "0.6b" else None,
        "vs_baseline_note": "the published numbers are the reference's on an RTX 3090 (8 requests end to end: 1,666 tokens/s); "
                            "another machine, not a same-hardware ratio",
        "dtype": "bf16",
        "data": "synthetic: seeded uniform-random token ids, random-init weights (seed 2)",
        "config": {"model": shape_name, "global_batch": args.batch, "seq_len": args.context, "parallelism": "single GPU",
                   "layers": n_layers, "layers_in_config": full_layers, "hidden": cfg["hidden_size"],
                   "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": V, "tied_embeddings": bool(cfg["tie_word_embeddings"]),
                   "prompt_tokens": args.prompt_tokens, "mean_context": mean_ctx, "page_size": args.block_size,
                   "l2": f"inputs larger than L2 ({nums['weight_bytes'] / 1e9:.2f} GB of weights per step), no flush", "peaks": pk["source"]},
        "e2e": e2e, "gpu_launches": launches_per_step * K, "prefill": prefill, "roofline": roofline, "points": points,
        "mixed_step": mixed, "load_s": llm.load_seconds, "clocks": clocks, "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
