"""Measurement helpers of the engine: per-request latency metrics, a cost model of the
architecture, and a per-kernel profile of eager steps.

The reference has the same three under src/profiler/: `GenMetrics` (TTFT, inter-token
latencies, throughputs; switched on by LLMGEN_METRICS, written as JSON to the path in
LLMGEN_METRICS_JSON, src/profiler/metrics.zig:29-189, src/profiler/reporter.zig:3-27),
`ModelCost` (FLOPs and bytes of a prompt and of decode steps from the model's sizes, compared
with LLMGEN_PEAK_TFLOPS / LLMGEN_PEAK_GBPS, src/profiler/metrics.zig:202-266) and `OpProfiler`
(time, FLOPs and bytes per operation and phase; switched on by LLMGEN_PROFILE, forces eager
steps, src/profiler/profiler.zig:46-180).  The reference times each graph node on the host with
a device synchronisation around it; here every kernel binding of `llmgen_b200.kernels.ops` is
bracketed by two CUDA events on the launching stream, which are read after the pass has ended,
so the pass itself runs without a synchronisation.

Nothing in this file is on the path of a step unless a profiler was enabled.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

PREFILL, DECODE, MIXED = "prefill", "decode", "mixed"


def percentile(sorted_values: Sequence[float], p: float) -> float:
    """Linear interpolation between the two nearest ranks (src/profiler/common.zig, numpy's default)."""
    if not sorted_values:
        return 0.0
    k = (len(sorted_values) - 1) * p / 100.0
    lo = int(k)
    hi = min(lo + 1, len(sorted_values) - 1)
    return sorted_values[lo] + (sorted_values[hi] - sorted_values[lo]) * (k - lo)


def env_number(name: str) -> Optional[float]:
    try:
        return float(os.environ[name])
    except (KeyError, ValueError):
        return None


# ------------------------------------------------------------------------------ GenMetrics
@dataclass
class GenMetrics:
    """Latencies of one request from the host's clock: `start()` when it is submitted,
    `on_token(now)` for every token that reaches the caller, `finish(now)` at the end."""
    prompt_tokens: int = 0
    t0: float = 0.0
    first: Optional[float] = None
    last: float = 0.0
    end: float = 0.0
    itl: List[float] = field(default_factory=list)      # seconds between consecutive tokens

    def start(self, prompt_tokens: int, now: float) -> None:
        self.prompt_tokens, self.t0, self.first, self.last, self.end = prompt_tokens, now, None, now, now
        self.itl.clear()

    def on_token(self, now: float) -> None:
        if self.first is None:
            self.first = now
        else:
            self.itl.append(now - self.last)
        self.last = now

    def finish(self, now: float) -> None:
        self.end = now

    @property
    def gen_tokens(self) -> int:
        return 0 if self.first is None else 1 + len(self.itl)

    def decode_seconds(self) -> float:
        """First token to last token."""
        return 0.0 if self.first is None else self.last - self.first

    def report(self, backend: str = "llmgen_b200") -> dict:
        """The fields of the reference's JSON report (src/profiler/reporter.zig:3-15).  The time to
        the first token stands for the prompt's time: the step that computes the prompt also
        samples the first token."""
        ttft = 0.0 if self.first is None else self.first - self.t0
        itl = sorted(self.itl)
        dec = self.decode_seconds()
        return {
            "backend": backend,
            "prompt_tokens": self.prompt_tokens,
            "gen_tokens": self.gen_tokens,
            "prefill_ms": ttft * 1e3,
            "ttft_ms": ttft * 1e3,
            "tpot_ms": dec / len(itl) * 1e3 if itl else 0.0,
            "itl_p50_ms": percentile(itl, 50) * 1e3,
            "itl_p99_ms": percentile(itl, 99) * 1e3,
            "prefill_tps": self.prompt_tokens / ttft if ttft > 0 else 0.0,
            "decode_tps": len(itl) / dec if dec > 0 else 0.0,
            "e2e_ms": (self.end - self.t0) * 1e3,
        }

    def text(self) -> str:
        r = self.report()
        lines = ["=== generation metrics ===",
                 f"prompt tokens : {r['prompt_tokens']}",
                 f"gen tokens    : {r['gen_tokens']}",
                 f"TTFT          : {r['ttft_ms']:.2f} ms",
                 f"E2E           : {r['e2e_ms']:.2f} ms"]
        if self.itl:
            itl = sorted(self.itl)
            k = max(len(self.itl) // 10, 1)
            lines += [f"TPOT          : {r['tpot_ms']:.3f} ms",
                      f"ITL first 10% : {sum(self.itl[:k]) / k * 1e3:.3f} ms   last 10%: {sum(self.itl[-k:]) / k * 1e3:.3f} ms",
                      f"ITL p50/p90/p99/max : {r['itl_p50_ms']:.3f} / {percentile(itl, 90) * 1e3:.3f} / "
                      f"{r['itl_p99_ms']:.3f} / {itl[-1] * 1e3:.3f} ms",
                      f"decode        : {r['decode_tps']:.1f} tok/s"]
        lines.append(f"prefill       : {r['prefill_tps']:.1f} tok/s")
        total = r["prompt_tokens"] + r["gen_tokens"]
        lines.append(f"total         : {total / (r['e2e_ms'] / 1e3) if r['e2e_ms'] > 0 else 0.0:.1f} tok/s")
        return "\n".join(lines)

    def write_json(self, path: Optional[str] = None) -> Optional[str]:
        """Write the report to `path`, or to the path in LLMGEN_METRICS_JSON; nothing if neither is given."""
        path = path or os.environ.get("LLMGEN_METRICS_JSON")
        if not path:
            return None
        with open(path, "w", encoding="utf-8") as f:
            json.dump(self.report(), f, indent=2)
            f.write("\n")
        return path


# ------------------------------------------------------------------------------- ModelCost
@dataclass(frozen=True)
class AttentionTerm:
    q_dim: int                  # query heads x head size
    kv_dim: int                 # key/value heads x head size
    window: int                 # 0: every key


@dataclass(frozen=True)
class ModelCost:
    """FLOPs and bytes that the model's sizes imply, run item by run item: what a step has to
    compute and to read at least.  `n_mm` counts the weights that take part in matrix products
    (the output projection included, the embedding table only where it is that projection)."""
    n_mm: int
    head_params: int            # hidden x vocabulary, part of n_mm
    attention: Tuple[AttentionTerm, ...]
    w_elem: int                 # bytes per weight
    kv_elem: int                # bytes per cached value
    complete: bool = True       # False: a part of unknown kind was counted as nothing

    @classmethod
    def from_spec(cls, spec, w_elem: int = 2, kv_elem: int = 2) -> "ModelCost":
        n_mm, terms, complete = 0, [], True
        for item in spec.run_order:
            block = spec.layers[item.layer]
            mixer, ffn = getattr(block, "mixer", None), getattr(block, "ffn", None)
            if getattr(mixer, "kind", None) == "attention":
                q_dim, kv_dim = mixer.num_heads * mixer.head_dim, mixer.num_kv_heads * mixer.head_dim
                n_mm += 2 * mixer.hidden_size * q_dim
                if item.writes_cache:                       # an item that reads another's cache projects no k, v
                    n_mm += 2 * mixer.hidden_size * kv_dim
                terms.append(AttentionTerm(q_dim, kv_dim, int(mixer.window or 0)))
            elif mixer is not None:
                complete = False
            if getattr(ffn, "kind", None) == "gated_mlp":
                n_mm += 3 * ffn.hidden_size * ffn.intermediate_size
            elif ffn is not None:
                complete = False
        head = spec.hidden_size * spec.vocab_size
        return cls(n_mm + head, head, tuple(terms), w_elem, kv_elem, complete)

    @staticmethod
    def _visible_sum(first_ctx: int, n: int, window: int) -> int:
        """Sum over the context lengths first_ctx .. first_ctx + n - 1 of the keys a query sees."""
        if n <= 0:
            return 0
        if not window:
            return n * first_ctx + n * (n - 1) // 2
        below = max(0, min(n, window - first_ctx + 1))     # context lengths that are still inside the window
        return below * first_ctx + below * (below - 1) // 2 + (n - below) * window

    def kv_bytes_per_token(self) -> int:
        return sum(2 * t.kv_dim * self.kv_elem for t in self.attention)

    def prefill_flops(self, p: int, logits_rows: int = 1) -> int:
        """A prompt of p tokens under the causal mask, the output projection on `logits_rows` rows
        (the reference's formula projects every row, src/profiler/metrics.zig:228-230)."""
        attn = sum(4 * t.q_dim * self._visible_sum(1, p, t.window) for t in self.attention)
        return 2 * (self.n_mm - self.head_params) * p + 2 * self.head_params * logits_rows + attn

    def decode_flops(self, c0: int, n: int) -> int:
        """n steps of one sequence whose context (the new token included) is c0, c0 + 1, ..."""
        return 2 * self.n_mm * n + sum(4 * t.q_dim * self._visible_sum(c0, n, t.window) for t in self.attention)

    def decode_bytes(self, c0: int, n: int) -> int:
        """Every weight once a step, and the keys and values the new token sees."""
        kv = sum(2 * t.kv_dim * self.kv_elem * self._visible_sum(c0, n, t.window) for t in self.attention)
        return self.n_mm * self.w_elem * n + kv


def efficiency_text(metrics: GenMetrics, cost: ModelCost, peak_tflops: Optional[float] = None,
                    peak_gbps: Optional[float] = None) -> str:
    """Achieved FLOP/s of the prompt and bytes/s of the decode steps of one request, and their
    shares of the peaks given (default: LLMGEN_PEAK_TFLOPS and LLMGEN_PEAK_GBPS)."""
    peak_tflops = peak_tflops if peak_tflops is not None else env_number("LLMGEN_PEAK_TFLOPS")
    peak_gbps = peak_gbps if peak_gbps is not None else env_number("LLMGEN_PEAK_GBPS")
    r = metrics.report()
    lines = ["=== hardware efficiency ===", f"N_mm          : {cost.n_mm / 1e6:.1f} M weights in matrix products"
             + ("" if cost.complete else " (parts of unknown kind not counted)")]
    prefill_s = r["prefill_ms"] / 1e3
    if prefill_s > 0:
        pf = cost.prefill_flops(metrics.prompt_tokens)
        lines.append(f"prefill       : {pf / 1e9:.1f} GFLOP, {pf / prefill_s / 1e12:.3f} TFLOP/s")
        if peak_tflops:
            lines.append(f"MFU (prefill) : {pf / prefill_s / (peak_tflops * 1e12) * 100:.1f} %")
    n, dec_s = len(metrics.itl), metrics.decode_seconds()
    if n and dec_s > 0:
        c0 = metrics.prompt_tokens + 1
        lines.append(f"decode        : {cost.decode_flops(c0, n) / dec_s / 1e12:.3f} TFLOP/s, "
                     f"{cost.decode_bytes(c0, n) / dec_s / 1e9:.1f} GB/s")
        if peak_gbps:
            lines.append(f"MBU (decode)  : {cost.decode_bytes(c0, n) / dec_s / (peak_gbps * 1e9) * 100:.1f} %")
    return "\n".join(lines)


# ------------------------------------------------------------------------------ OpProfiler
def _nbytes(x) -> int:
    """Bytes of an operand: an array, the slices of a product cut along K, or nothing."""
    if x is None:
        return 0
    tensor = getattr(x, "tensor", None)                    # ops.Partials
    if tensor is not None:
        return tensor.numel() * tensor.element_size()
    if hasattr(x, "numel") and hasattr(x, "element_size"):
        return x.numel() * x.element_size()
    return 0


@dataclass
class PassInfo:
    """What the profiler knows of the pass that is running: its phase and, per sequence, where its
    tokens start and how many there are."""
    phase: str = PREFILL
    starts: Tuple[int, ...] = ()
    q_lens: Tuple[int, ...] = ()

    def visible_keys(self, window: int) -> int:
        """Sum over the pass's tokens of the keys each one sees."""
        return sum(ModelCost._visible_sum(s + 1, n, window) for s, n in zip(self.starts, self.q_lens))

    def keys_read(self, window: int) -> int:
        """Keys that the pass's sequences read when each is read once."""
        if not window:
            return sum(s + n for s, n in zip(self.starts, self.q_lens))
        return sum(min(s + n, window + n - 1) for s, n in zip(self.starts, self.q_lens))


def _cost_product(a, info: PassInfo) -> Tuple[int, int]:
    w = a["w"]
    x = a.get("a", a.get("x"))
    out = a.get("out", a.get("slices"))
    M, N, K = int(x.shape[0]), int(w.shape[0]), int(w.shape[1])
    return 2 * M * N * K, _nbytes(w) + _nbytes(x) + _nbytes(out)


def _cost_attention(a, info: PassInfo) -> Tuple[int, int]:
    nq, nkv, hd, window = int(a["nq"]), int(a["nkv"]), int(a["hd"]), int(a["window"] or 0)
    elem = a["kcache"].element_size()
    tokens = sum(info.q_lens)
    flops = 4 * nq * hd * info.visible_keys(window)
    bytes_ = 2 * nkv * hd * elem * info.keys_read(window) + 2 * tokens * nq * hd * elem
    packed = a.get("packed")
    if packed is not None:                                 # the kernel also reads the projection and stores k, v
        bytes_ += _nbytes(packed) + 2 * tokens * int(a.get("nk") or 0) * hd * elem
    return flops, bytes_


def _cost_attn_prep(a, info: PassInfo) -> Tuple[int, int]:
    n_rows = int(getattr(a["qkv"], "rows", None) or a["qkv"].shape[0])
    nq, nk, hd = int(a["nq"]), int(a["nk"]), int(a["hd"])
    elem = a["kcache"].element_size() if a.get("kcache") is not None else 2
    written = n_rows * (nq + 2 * nk) * hd * elem            # q in place or to q_out, k and v into the cache
    tables = 2 * n_rows * int(a["rot"]) * 4 if a.get("cos") is not None else 0
    return n_rows * (nq + nk) * hd * 6, _nbytes(a["qkv"]) + written + tables


def _cost_embed(a, info: PassInfo) -> Tuple[int, int]:
    out = a["out"]
    return 0, _nbytes(a["ids"]) + _nbytes(out) + out.numel() * a["table"].element_size()


def _cost_norm(a, info: PassInfo) -> Tuple[int, int]:
    out = a["out"]
    rows, H = int(out.shape[0]), int(out.shape[-1])
    resid = rows * H * 4 * (2 if (a.get("write_resid", True) and a.get("rows") is None and a.get("delta") is not None) else 1)
    return 5 * rows * H, resid + _nbytes(a.get("delta")) + _nbytes(out) + _nbytes(a["weight"])


def _cost_all_operands(a, info: PassInfo) -> Tuple[int, int]:
    out = a.get("out", a.get("out_ids"))
    flops = out.numel() if hasattr(out, "numel") else 0
    return flops, sum(_nbytes(v) for k, v in a.items() if k != "scratch")


# kernel bindings of `ops` that launch work, and how each one's FLOPs and bytes are counted
OP_COSTS: Dict[str, Callable] = {
    "embed_rows": _cost_embed, "add_rmsnorm": _cost_norm, "silu_mul": _cost_all_operands, "widen": _cost_all_operands,
    "attn_prep": _cost_attn_prep, "gemm_simt": _cost_product, "gemv_bf16": _cost_product, "gemm_tc": _cost_product,
    "gemm_skinny": _cost_product, "gemm_rows8": _cost_product, "gemm_rows8_gated": _cost_product, "paged_attention": _cost_attention, "attention_decode": _cost_attention,
    "attention_tc": _cost_attention, "sample": _cost_all_operands,
}


class CudaEventClock:
    """Marks on the current CUDA stream; `elapsed_ms` is valid after `wait()`."""

    def __init__(self):
        import torch
        self._torch = torch
        self._spare: List[object] = []

    def mark(self):
        if self._torch.cuda.is_current_stream_capturing():
            return None                                    # launches recorded into a graph are not timed
        ev = self._spare.pop() if self._spare else self._torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def wait(self) -> None:
        self._torch.cuda.current_stream().synchronize()

    def elapsed_ms(self, a, b) -> float:
        return a.elapsed_time(b)

    def give_back(self, marks) -> None:
        self._spare.extend(marks)


@dataclass
class OpStat:
    calls: int = 0
    ms: float = 0.0
    flops: int = 0
    bytes: int = 0


class OpProfiler:
    """Device time, FLOPs and bytes of every kernel binding, by phase, while enabled.

    `enable()` puts a timed wrapper around each binding listed in `OP_COSTS` (they are module
    attributes of `llmgen_b200.kernels.ops`, looked up at every call), `disable()` takes it away.
    Only launches made directly are seen, so the engine has to run eager steps; a replayed graph
    makes no calls.  The executor calls `begin_pass` before every eager pass.  The marks between
    kernels keep a kernel from starting before the one before has ended, so the times are those of
    serialised launches, as under a profiler; the phase total runs from a pass's first mark to its
    last and `(between kernels)` is what the kernels do not account for.
    """
    _active: Optional["OpProfiler"] = None

    def __init__(self, ops_module=None, clock=None):
        if ops_module is None:
            from ..kernels import ops as ops_module
        self.ops = ops_module
        self.clock = clock
        self.stats: Dict[Tuple[str, str], OpStat] = {}
        self.phase_ms: Dict[str, float] = {}
        self.passes: Dict[str, int] = {}
        self.info = PassInfo()
        self._saved: Dict[str, Callable] = {}
        self._open: List[tuple] = []           # (phase, op, mark before, mark after) of the pass not yet read

    # -- switching
    def enable(self) -> "OpProfiler":
        if OpProfiler._active is not None:
            raise RuntimeError("another OpProfiler is enabled")
        if self.clock is None:
            self.clock = CudaEventClock()
        for name in OP_COSTS:
            fn = getattr(self.ops, name, None)
            if fn is not None:
                self._saved[name] = fn
                setattr(self.ops, name, self._timed(name, fn))
        OpProfiler._active = self
        return self

    def disable(self) -> None:
        if OpProfiler._active is self:
            self.collect()
            for name, fn in self._saved.items():
                setattr(self.ops, name, fn)
            self._saved.clear()
            OpProfiler._active = None

    def __enter__(self):
        return self.enable()

    def __exit__(self, *exc):
        self.disable()

    def _timed(self, name: str, fn: Callable) -> Callable:
        import inspect
        signature = inspect.signature(fn)
        cost = OP_COSTS[name]

        def timed(*args, **kwargs):
            before = self.clock.mark()
            if before is None:
                return fn(*args, **kwargs)
            result = fn(*args, **kwargs)
            after = self.clock.mark()
            bound = signature.bind(*args, **kwargs)
            bound.apply_defaults()
            try:
                flops, bytes_ = cost(bound.arguments, self.info)
            except (AttributeError, KeyError, TypeError, IndexError):
                flops, bytes_ = 0, 0                       # an operand of a kind the model does not know
            stat = self.stats.setdefault((self.info.phase, name), OpStat())
            stat.calls += 1
            stat.flops += int(flops)
            stat.bytes += int(bytes_)
            self._open.append((self.info.phase, name, before, after))
            return result
        timed.__name__ = name
        timed.__wrapped__ = fn
        return timed

    # -- what the executor reports
    def begin_pass(self, starts: Sequence[int], q_lens: Sequence[int]) -> None:
        """A pass over these sequences is about to be launched; the pass before is read now."""
        self.collect()
        if all(n == 1 for n in q_lens):
            phase = DECODE
        elif any(n == 1 and s > 0 for s, n in zip(starts, q_lens)):
            phase = MIXED
        else:
            phase = PREFILL
        self.info = PassInfo(phase, tuple(int(s) for s in starts), tuple(int(n) for n in q_lens))

    def collect(self) -> None:
        """Read the marks of the launches so far (waits for the stream)."""
        if not self._open:
            return
        self.clock.wait()
        phase = self._open[0][0]
        for ph, name, before, after in self._open:
            self.stats[(ph, name)].ms += self.clock.elapsed_ms(before, after)
        self.phase_ms[phase] = self.phase_ms.get(phase, 0.0) + self.clock.elapsed_ms(self._open[0][2], self._open[-1][3])
        self.passes[phase] = self.passes.get(phase, 0) + 1
        give_back = getattr(self.clock, "give_back", None)
        if give_back is not None:
            give_back([m for rec in self._open for m in rec[2:]])
        self._open.clear()

    # -- results
    def op_ms(self, phase: str) -> float:
        return sum(s.ms for (ph, _), s in self.stats.items() if ph == phase)

    def rows(self, phase: str) -> List[dict]:
        """One row per binding that ran in `phase`, the longest first."""
        self.collect()
        total = self.phase_ms.get(phase, 0.0)
        out = []
        for (ph, name), s in self.stats.items():
            if ph != phase or s.calls == 0:
                continue
            ns = max(s.ms * 1e6, 1.0)
            out.append({"op": name, "calls": s.calls, "total_ms": s.ms, "avg_us": s.ms * 1e3 / s.calls,
                        "pct": s.ms / total * 100 if total > 0 else 0.0, "gflops": s.flops / ns, "gbps": s.bytes / ns,
                        "intensity": s.flops / max(s.bytes, 1)})
        out.sort(key=lambda r: -r["total_ms"])
        return out

    def text(self) -> str:
        self.collect()
        lines = []
        for phase in (PREFILL, MIXED, DECODE):
            rows = self.rows(phase)
            if not rows:
                continue
            total = self.phase_ms.get(phase, 0.0)
            lines.append(f"=== kernel time [{phase}] ({self.passes.get(phase, 0)} passes, {total:.2f} ms) ===")
            lines.append(f"{'op':<20} {'calls':>8} {'total_ms':>10} {'avg_us':>9} {'pct':>6} {'GFLOP/s':>10} {'GB/s':>9} {'FLOP/B':>8}")
            for r in rows:
                lines.append(f"{r['op']:<20} {r['calls']:>8} {r['total_ms']:>10.3f} {r['avg_us']:>9.2f} {r['pct']:>5.1f}% "
                             f"{r['gflops']:>10.1f} {r['gbps']:>9.1f} {r['intensity']:>8.2f}")
            other = max(total - self.op_ms(phase), 0.0)
            lines.append(f"{'(between kernels)':<20} {'':>8} {other:>10.3f} {'':>9} {other / total * 100 if total > 0 else 0.0:>5.1f}%")
        return "\n".join(lines)
