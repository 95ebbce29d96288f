"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

One `Executor.step(entries)` runs exactly the tokens it is given, as one batch, against the
cache that earlier steps left: portions of prompts beside single decoded tokens, cut
anywhere.  It is the reference's `Executor.forward(entries)` (src/executor.zig:530-590) with
two differences: the caller may pass token ids directly (replay) and gets float32 logits at the
rows it names (the reference returns only sampled ids, src/executor.zig:669-677).

Host work per step: fill one pinned metadata buffer (`StepMetaBuilder`), ONE host-to-device
copy, the launches (or one graph replay for a pure-decode step), one device-to-host copy of
the sampled ids.  A step with more tokens than `max_step_tokens` is cut into passes
(src/executor.zig:986-1043).

Pages must have been reserved for every position the step writes (`reserve`); the scheduler
or the replay program does that, as the reference's scheduler calls `ensure`.
"""
from __future__ import annotations

import array
import ctypes
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheError, CacheManager
from ..cache.manager import runtime as cache_runtime
from ..cache.storage import CacheStorage, bytes_per_page, plan_groups
from ..kernels import ops
from .context import GroupView, StepContext, StepMetaBuilder, Workspace
from .model import DecoderModel

SEED_STRIDE = 0x9E3779B97F4A7C15
DEFAULT_SEED = 0x5EED
MASK64 = (1 << 64) - 1


class StepError(ValueError):
    pass


@dataclass
class PendingIds:
    """The sampled ids of a launched decode step: a pinned host buffer that is valid once `event` has passed,
    and beside it the kernels' two status flags as they stood after the step."""
    host: torch.Tensor
    event: object
    flags: Optional[torch.Tensor] = None


@dataclass
class EngineLimits:
    """Engine-side limits (command-line options in the reference, src/cli.zig:33-62)."""
    max_num_seqs: int = 256          # sequences per step
    max_model_len: int = 4096        # longest sequence; width of the block tables
    max_step_tokens: int = 8192      # tokens per forward pass (`--pass-tokens`)
    page_size: int = 16              # tokens per cache page (`--block-size`)
    num_pages: Optional[int] = None  # pages per group (`--kv-blocks`); None: from free memory
    gpu_util: float = 0.9            # share of device memory the process may use

    def __post_init__(self):
        if self.max_num_seqs <= 0 or self.max_model_len <= 0 or self.page_size <= 0:
            raise StepError("engine limits must be positive")
        self.max_step_tokens = max(self.max_step_tokens, self.max_num_seqs)


@dataclass
class StepEntry:
    req: Hashable
    tokens: Sequence[int]
    start: int                              # position of tokens[0] in its sequence
    want: Sequence[int] = ()                # indices into `tokens` whose logits are wanted
    temperature: float = 0.0                # for sampled ids


@dataclass
class StepOutput:
    logits: Optional[torch.Tensor] = None   # float32 [wanted, vocab], device
    token_ids: Optional[List[int]] = None   # one per wanted row, host


def _model_parts(model):
    """Every part object of a model: its blocks, what they hold (norms, mixer, feed-forward) and the final norm."""
    parts = [model.final_norm]
    for layer in model.layers:
        parts.append(layer)
        parts += [v for v in vars(layer).values() if hasattr(v, "forward") or hasattr(v, "add_norm")]
    return parts


class Executor:
    def __init__(self, model: DecoderModel, limits: EngineLimits, seed: int = DEFAULT_SEED,
                 eager: bool = False, sync_each: bool = False):
        self.model = model
        self.limits = limits
        self.device = model.device
        self.dtype = model.dtype
        # a part whose `forward` cannot be recorded into a CUDA graph (it reads a result back on the host, or its
        # launches depend on the data) says so with a class attribute `capturable = False`; every step of a model
        # with such a part is launched kernel by kernel
        self.uncapturable = sorted({type(p).__name__ for p in _model_parts(model) if getattr(p, "capturable", True) is False})
        self.eager = eager or sync_each or bool(self.uncapturable)
        self.sync_each = sync_each
        self.seed = seed & MASK64
        self.n_graph_steps = 0
        self.n_eager_steps = 0
        self.launch_count = 0
        self.last_upload_bytes = 0       # bytes of the last step's arrays copied to the device
        self.profiler = None             # an `engine.profiler.OpProfiler`: told of every eager pass
        if limits.max_model_len > model.max_positions():
            raise StepError(f"max_model_len {limits.max_model_len} exceeds the model's "
                            f"{model.max_positions()} positions")
        self.max_blocks = (limits.max_model_len + limits.page_size - 1) // limits.page_size

        # caches: one request per cache number of the run list
        kv_requests, state_requests = {}, {}
        for item in model.spec.run_order:
            if item.cache is None:
                continue
            mixer = model.layers[item.layer].mixer
            kv = mixer.cache_request()
            st = mixer.state_request()
            for table, req in ((kv_requests, kv), (state_requests, st)):
                if req is None:
                    continue
                if item.cache in table and table[item.cache] != req:
                    raise StepError(f"run items sharing cache {item.cache} ask for different geometries")
                table[item.cache] = req
        self.kv_requests, self.state_requests = kv_requests, state_requests
        self.group_specs, self.group_index = plan_groups(kv_requests)
        pages = self._pages_per_group()
        self.cache = CacheManager(self.group_specs, pages, limits.page_size, limits.max_num_seqs)
        self.storage = CacheStorage(kv_requests, state_requests, self.group_index, pages, limits.page_size,
                                    limits.max_num_seqs, self.dtype, self.device)
        self.layer_caches = [self.storage.layer_cache(item.cache, item.writes_cache) for item in model.spec.run_order]
        # one mixer for every set of step arrays: mixers that say, by `step_arrays_key()`, that they add the
        # same arrays are asked once
        self._unique_mixers = []
        keys = set()
        for layer in model.layers:
            m = getattr(layer, "mixer", None)
            if m is not None and hasattr(m, "prepare_step"):
                key = m.step_arrays_key() if hasattr(m, "step_arrays_key") else id(m)
                if key not in keys:
                    keys.add(key)
                    self._unique_mixers.append(m)

        # mixers whose own step arrays depend only on the batch's shape let decode steps reuse them
        self._static_step_arrays = all(getattr(m, "step_arrays_follow_shapes", False) for m in self._unique_mixers)
        self.workspace = Workspace(self.device, limits.max_step_tokens)
        Tm, Sm, G = limits.max_step_tokens, limits.max_num_seqs, len(self.group_specs)
        words = 64 + 12 * Tm + 12 * Sm + G * (Tm + Sm * self.max_blocks + 8)
        self.meta_host = [torch.empty(words, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.meta_events = [None, None]
        self.meta_dev = torch.zeros(words, dtype=torch.int32, device=self.device)
        self._meta_turn = 0
        self.sample_scratch = ops.sample_scratch(max(Sm, 64), self.device)
        self.ids_host = torch.empty(max(Tm, Sm), dtype=torch.int32).pin_memory()
        # decode steps replayed from a graph leave their sampled ids here; the next step may take its
        # input ids from it on the device (`decode_launch`), before the host has read them
        self.sampled_dev = torch.zeros(Sm, dtype=torch.int32, device=self.device)
        self._ids_hosts = [torch.empty(Sm, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._ids_events = [torch.cuda.Event(), torch.cuda.Event()]
        # what the kernels report beside their results (a wait that ran out, a sequence beyond a launch's bound,
        # a token id outside the vocabulary): read with every step's ids, never by a synchronisation of its own
        self.status_dev = ops.status_flags(self.device)
        self._status_hosts = [torch.zeros(2, dtype=torch.int32).pin_memory() for _ in range(3)]
        self._ids_turn = 0
        self.graphs: Dict[Tuple[int, int], dict] = {}     # (batch-size bucket, context-length class) -> graph
        # steps of any other kind (portions of prompts, with or without single tokens beside them) replay a graph
        # captured for their shape, (token rows, sequences) rounded up: see `step_shape`
        self.shape_graphs: Dict[Tuple[int, int], dict] = {}
        self.shaped_steps = not self.eager and all(getattr(m, "replay_any_step", False) for m in self._unique_mixers)
        self.n_shaped_steps = 0
        self._token_shapes, self._seq_shapes = self.token_shapes(), self.seq_shapes()
        self._graph_logits = None                         # float32 [max_num_seqs, vocab], shared by the graphs
        # decode steps rewrite only what changed in a host buffer that the same bucket filled last
        self._host_owner = [None, None]                   # per pinned buffer: (bucket, layout) of its last fill
        self._host_rows = [None, None]                    # per pinned buffer: per group and row, (request, table stamp)
        self._runtime = cache_runtime()
        top = self.limits.max_num_seqs
        self._decode_args = ((ctypes.c_longlong * top)(), (ctypes.c_int * top)(), (ctypes.c_int * top)(),
                             (ctypes.c_float * top)(), (ctypes.c_int * top)())
        # ... requests, tokens, positions, temperatures of a decode step, and the rows of the step before its ids come from

    # ------------------------------------------------------------------ sizing
    def _pages_per_group(self) -> List[int]:
        lim = self.limits
        if lim.num_pages is not None:
            if lim.num_pages * lim.page_size < lim.max_model_len:
                raise StepError(f"{lim.num_pages} pages of {lim.page_size} tokens cannot hold one sequence of "
                                f"max_model_len {lim.max_model_len}")
            return [lim.num_pages] * len(self.group_specs)
        # From free memory, as the reference does (src/graph/scheduler.zig:386-403):
        # (total * util - used - activations reserve) / bytes per page over all layers.
        free, total = torch.cuda.mem_get_info(self.device)
        used = total - free
        budget = int(total * lim.gpu_util) - used - self._activation_reserve()
        per_page = sum(bytes_per_page(self.kv_requests, self.group_index, g, lim.page_size, self.dtype)
                       for g in range(len(self.group_specs)))
        if per_page == 0:
            return [0] * len(self.group_specs)
        n = budget // per_page
        cap = lim.max_num_seqs * self.max_blocks   # more than every sequence at full length is never used
        n = int(min(n, cap))
        if n * lim.page_size < lim.max_model_len:
            raise StepError(f"the memory budget leaves {max(n, 0)} pages, fewer than one sequence of "
                            f"max_model_len {lim.max_model_len} needs")
        return [n] * len(self.group_specs)

    def _activation_reserve(self) -> int:
        """Device memory to leave beside the cache pages for a step's activations: what the widest layer says it
        keeps in the workspace (`workspace_bytes(tokens)`; a layer that does not say is counted by its hidden
        width alone), the float32 residual, and the logits of a batch of decoded tokens."""
        spec = self.model.spec
        tokens = self.limits.max_step_tokens
        elem = 2 if self.dtype == torch.bfloat16 else 4
        widest = 0
        for layer in self.model.layers:
            ask = getattr(layer, "workspace_bytes", None)
            widest = max(widest, ask(tokens) if ask is not None else 6 * tokens * spec.hidden_size * elem)
        rows = max(64, self.limits.max_num_seqs)
        return widest + tokens * spec.hidden_size * 4 + 2 * rows * spec.vocab_size * 4 + (64 << 20)

    # ------------------------------------------------------------------ cache front
    def admit(self, req: Hashable) -> bool:
        slot = self.cache.admit(req)
        self._reset_fresh_state()
        return slot is not None

    def _reset_fresh_state(self) -> None:
        """Zero the per-request state of slots that new requests received since the last look
        (through `admit` here or through the scheduler, which admits on the native side)."""
        if self.cache.fresh_state:
            self.storage.reset_state(list(self.cache.fresh_state))
            self.cache.fresh_state.clear()

    def reserve(self, req: Hashable, start: int, end: int) -> bool:
        if end > self.limits.max_model_len:
            raise StepError(f"request {req!r}: positions up to {end} exceed max_model_len {self.limits.max_model_len}")
        return self.cache.reserve(req, start, end)

    def can_reserve(self, req: Hashable, start: int, end: int) -> bool:
        return self.cache.can_reserve(req, start, end)

    def release(self, req: Hashable) -> None:
        self.cache.release(req)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], sample: bool = False, return_logits: bool = True) -> StepOutput:
        """Run the entries' tokens as one batch.  Logits rows (and sampled ids) come in the order
        of the entries and, inside an entry, of its `want` list."""
        entries = [e for e in entries]
        arrays = self._validate(entries)
        # a portion's ids were turned into an array for the check: the step's arrays are filled from it
        entries = [e if a is None else StepEntry(e.req, a, e.start, e.want, e.temperature) for e, a in zip(entries, arrays)]
        self._reset_fresh_state()
        n_tokens = sum(len(e.tokens) for e in entries)
        if n_tokens == 0:
            return StepOutput(torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.device)
                              if return_logits else None, [] if sample else None)
        pure_decode = all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        if pure_decode and sample and not return_logits:
            if not self.eager:
                return self._graph_step(entries)
            # eager generation runs exactly what the graph of this step would replay (the batch
            # padded to its bucket), so that both give the same bits
            out = self._eager_pass(entries, True, False, pad_to=self._bucket_for(len(entries)))
            self.n_eager_steps += 1
            return out
        passes = self._passes(entries)
        logits_parts, ids_parts, order = [], [], []
        for sub, keys in passes:
            shape = self.step_shape(sub) if self.shaped_steps and self.profiler is None else None
            if shape is not None:
                out = self._shaped_pass(sub, sample, return_logits or len(passes) > 1, shape)
            else:
                out = self._eager_pass(sub, sample, return_logits or len(passes) > 1)
            if return_logits or len(passes) > 1:
                logits_parts.append(out.logits)
            if sample:
                ids_parts += out.token_ids
            order += keys
        self.n_eager_steps += 1
        result = StepOutput()
        # restore the order (entry, k-th want) when passes or want lists permuted it
        wanted = [(i, k) for i, e in enumerate(entries) for k in range(len(e.want))]
        perm = None
        if order != wanted:
            where = {key: r for r, key in enumerate(order)}
            perm = [where[key] for key in wanted]
        if return_logits:
            logits = logits_parts[0] if len(logits_parts) == 1 else torch.cat(logits_parts, dim=0)
            if perm is not None:
                logits = logits.index_select(0, torch.as_tensor(perm, dtype=torch.long, device=self.device))
            result.logits = logits
        if sample:
            result.token_ids = [ids_parts[r] for r in perm] if perm is not None else ids_parts
        return result

    def _validate(self, entries: Sequence[StepEntry], prev_rows: Optional[Sequence[int]] = None) -> List[Optional[np.ndarray]]:
        """Raise `StepError` for a step that cannot run.  Returns, per entry, its token ids as an integer
        array where the check made one (None for a single token)."""
        lim = self.limits
        arrays: List[Optional[np.ndarray]] = []
        V = self.model.spec.vocab_size
        if len(entries) > lim.max_num_seqs:
            raise StepError(f"{len(entries)} sequences in one step, the limit is {lim.max_num_seqs}")
        seen = set()
        for i, e in enumerate(entries):
            if e.req in seen:
                raise StepError(f"request {e.req!r} appears twice in one step")
            seen.add(e.req)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.req!r} brings no tokens")
            if e.start < 0 or e.start + n > lim.max_model_len:
                raise StepError(f"request {e.req!r}: positions [{e.start}, {e.start + n}) exceed max_model_len "
                                f"{lim.max_model_len}")
            if n == 1 and prev_rows is not None and prev_rows[i] >= 0:
                toks = None                                    # its token is still on the device
            elif n == 1 and type(e.tokens[0]) is int and 0 <= e.tokens[0] < V:
                toks = None                                    # the common case of a decoded token, checked without numpy
            else:
                toks = None
                if type(e.tokens) is list:
                    try:                                       # several times faster than numpy on a list of ints
                        toks = np.frombuffer(array.array("i", e.tokens), dtype=np.int32)
                    except (TypeError, OverflowError):
                        toks = None                            # numpy's conversion below names the fault
                if toks is None:
                    toks = np.asarray(e.tokens)
            if toks is not None and (toks.dtype.kind not in "iu" or int(toks.min()) < 0 or int(toks.max()) >= V):
                bad = [int(t) for t in toks.tolist() if not (isinstance(t, int) and 0 <= t < V)][:1]
                raise StepError(f"request {e.req!r}: token id {bad[0] if bad else '?'} outside the vocabulary [0, {V})")
            arrays.append(toks if n > 1 else None)
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.req!r}: wanted place {w} outside its {n} tokens")
            why = self.cache.check_step(e.req, e.start, n)
            if why:
                raise StepError(why)
        return arrays

    def _passes(self, entries: Sequence[StepEntry]):
        """Cut the entries into passes of at most `max_step_tokens` tokens.  Each pass is a list of
        entries plus the (entry index, k-th want) key of each of its wanted rows, in row order."""
        cap = self.limits.max_step_tokens
        passes, cur, keys, room = [], [], [], cap
        for i, e in enumerate(entries):
            off = 0
            n = len(e.tokens)
            while off < n:
                take = min(n - off, room)
                want_here = [(k, w - off) for k, w in enumerate(e.want) if off <= w < off + take]
                cur.append(StepEntry(e.req, e.tokens[off:off + take], e.start + off, [w for _, w in want_here],
                                     e.temperature))
                keys += [(i, k) for k, _ in want_here]
                off += take
                room -= take
                if room == 0:
                    passes.append((cur, keys))
                    cur, keys, room = [], [], cap
        if cur:
            passes.append((cur, keys))
        return passes

    # -- metadata
    def _build_meta(self, entries: Sequence[StepEntry], pad_to: int = 0, ctx_bound: int = 0,
                    ids_from: Optional[Sequence[int]] = None, shape: Optional[Tuple[int, int]] = None):
        """Fill and upload the step's metadata; returns (StepContext, want rows view, temps view,
        view of the sampler's row keys, number of wanted rows).  A batch of single tokens padded to a graph's
        shape (`pad_to` sequences) also gets `ids_from`: for each row the row of the step before whose sampled id
        is its token, or -1.  `shape` = (token rows, sequences) lays any other step out for the graph of that
        shape: token rows beyond the step's own belong to no sequence and are written nowhere, and the sequences
        beyond its own have no tokens."""
        lim = self.limits
        ps = lim.page_size
        S_real = len(entries)
        S = max(S_real, pad_to, shape[1] if shape else 0)
        q_lens = [len(e.tokens) for e in entries] + [0 if shape else 1] * (S - S_real)
        starts = [e.start for e in entries] + [0] * (S - S_real)
        T = max(sum(q_lens), shape[0] if shape else 0)
        pure_decode = all(n == 1 for n in q_lens) and not shape
        b = StepMetaBuilder(q_lens, starts, pure_decode, lim.page_size, token_bound=shape[0] if shape else 0)
        ids = np.zeros(T, dtype=np.int32)
        pos = np.zeros(T, dtype=np.int32)
        seq_of = np.zeros(T, dtype=np.int32)
        cu_q = np.zeros(S + 1, dtype=np.int32)
        ctx_len = np.zeros(S, dtype=np.int32)
        state_slots = np.full(S, -1, dtype=np.int32)
        want_rows, temps, keys = [], [], []
        t = 0
        for s, e in enumerate(entries):
            n = q_lens[s]
            ids[t:t + n] = np.asarray([0 if tok is None else tok for tok in e.tokens] if n == 1 else e.tokens, dtype=np.int32)
            pos[t:t + n] = np.arange(e.start, e.start + n, dtype=np.int32)
            seq_of[t:t + n] = s
            ctx_len[s] = e.start + n
            state_slots[s] = self.cache.state.slot(e.req)
            want_rows += [t + w for w in e.want]
            temps += [e.temperature] * len(e.want)
            keys += [self.row_key(e.req, e.start + w) for w in e.want]
            t += n
            cu_q[s + 1] = t
        for s in range(S_real, S):          # padding rows: one token, no keys, written nowhere
            if shape:
                cu_q[s + 1] = t
                continue
            seq_of[t] = s
            t += 1
            cu_q[s + 1] = t
            want_rows.append(t - 1)
            temps.append(0.0)
            keys.append(0)
        b.add("ids", ids)
        if pad_to > 0:
            src = np.full(T, -1, dtype=np.int32)
            if ids_from is not None:
                src[:S_real] = np.asarray(ids_from, dtype=np.int32)
            b.add("ids_from", src)
        b.add("positions", pos)
        b.add("seq_of_token", seq_of)
        b.add("cu_q", cu_q)
        b.add("ctx_len", ctx_len)
        b.add("state_slots", state_slots)
        for gi, g in enumerate(self.cache.groups):
            slots = np.full(T, -1, dtype=np.int32)
            bt = np.zeros((S, self.max_blocks), dtype=np.int32)
            t = 0
            for s, e in enumerate(entries):
                table = g.table(e.req)
                n = q_lens[s]
                tab = np.asarray(table, dtype=np.int32)
                bt[s, :len(table)] = tab
                p = np.arange(e.start, e.start + n)
                slots[t:t + n] = tab[p // ps] * ps + p % ps
                t += n
            b.add(f"slots_{gi}", slots)
            b.add(f"block_tables_{gi}", bt)
        for m in self._unique_mixers:
            m.prepare_step(b)
        # what only the sampler and the gather of the wanted rows read comes last: its size is the one thing that a
        # step's shape does not fix, and nothing that a replayed graph reads lies behind it
        b.add("want_rows", np.asarray(want_rows, dtype=np.int32))
        b.add("temps", np.asarray(temps, dtype=np.float32), dtype=np.float32)
        b.add("row_keys", np.asarray(keys, dtype=np.uint64).view(np.int32))

        turn = self._meta_turn
        self._meta_turn ^= 1
        if self.meta_events[turn] is not None:
            self.meta_events[turn].synchronize()
        layout, total = b.pack_into(self.meta_host[turn])
        self._host_owner[turn] = None
        self._last_fill = (turn, layout, total)
        self.meta_dev[:total].copy_(self.meta_host[turn][:total], non_blocking=True)
        self.last_upload_bytes = 4 * total
        ev = torch.cuda.Event()
        ev.record()
        self.meta_events[turn] = ev

        def view(name):
            off, size, dt = layout[name]
            v = self.meta_dev[off:off + size]
            return v.view(torch.float32) if dt == np.float32 else v

        views = {n: view(n) for n in layout}
        longest = int(ctx_len.max()) if S else 0
        ctx = StepContext(
            n_tokens=T, n_seqs=S, dtype=self.dtype, device=self.device, workspace=self.workspace,
            requests=[e.req for e in entries], starts=starts, q_lens=q_lens, pure_decode=pure_decode,
            # a step laid out for the graph of its shape is bounded by the longest sequence the engine takes: the
            # graph's launches must hold for every step of that shape
            max_ctx=longest, max_ctx_bound=ctx_bound or (lim.max_model_len if shape else self.context_class(longest)),
            max_seqs_bound=lim.max_num_seqs,
            ids=views["ids"], ids_from=views.get("ids_from"),
            prev_sampled=self.sampled_dev if "ids_from" in layout else None,
            positions=views["positions"], cu_q=views["cu_q"], ctx_len=views["ctx_len"],
            state_slots=views["state_slots"], seq_of_token=views["seq_of_token"],
            groups=[GroupView(views[f"slots_{gi}"], views[f"block_tables_{gi}"], self.max_blocks)
                    for gi in range(len(self.cache.groups))],
            extra=views)
        return ctx, views["want_rows"], views["temps"], views["row_keys"], len(want_rows)

    def row_key(self, req: Hashable, position: int) -> int:
        """The sampler's 64-bit key of the row that samples the token after `position` of `req`:
        (seed + stride * (position + 1)) ^ (request << 40), the reference's step_seed ^ (row << 40)
        (src/backend/cpu/sample.zig:28, seed stride src/executor.zig:717-753) with the position in the step's
        place and the request's number in the row's.  A draw then depends on the request and the position
        alone: not on what else is in the batch, on how many steps ran before, on whether steps are launched
        ahead, nor on a preemption that computes the position a second time."""
        return ((self.seed + SEED_STRIDE * (position + 1)) & MASK64) ^ ((self.cache.key(req) << 40) & MASK64)

    def _raise_status(self, flags_host: torch.Tensor) -> None:
        kernel_error, bad_token = int(flags_host[0]), int(flags_host[1])
        if kernel_error or bad_token:
            self.status_dev.zero_()
            raise StepError(ops.status_message(kernel_error, bad_token))

    def _maybe_sync(self):
        if self.sync_each:
            torch.cuda.synchronize(self.device)

    def _eager_pass(self, entries: Sequence[StepEntry], sample: bool, return_logits: bool, pad_to: int = 0) -> StepOutput:
        if self.profiler is not None:
            self.profiler.begin_pass([e.start for e in entries], [len(e.tokens) for e in entries])
        ctx, want_rows, temps, keys, n_want = self._build_meta(entries, pad_to=pad_to)
        ctx.fixed_shapes = pad_to > 0      # the launch shapes a captured graph of this step would have
        resid, delta = self.model.hidden_states(ctx, self.layer_caches)
        return self._finish_pass(entries, ctx, resid, delta, want_rows, temps, keys, n_want, sample, return_logits)

    def _shaped_pass(self, entries: Sequence[StepEntry], sample: bool, return_logits: bool, shape: Tuple[int, int]) -> StepOutput:
        """What `_eager_pass` gives, with the layers replayed from the graph of the step's shape."""
        g = self.shape_graphs.get(shape) or self._capture_shape(shape)
        ctx, want_rows, temps, keys, n_want = self._build_meta(entries, shape=shape)
        if self._shape_layout() != g["layout"]:
            # a part laid its arrays out by the step's lengths, not by its shape: such a model's steps cannot be
            # replayed; launch this one and all later ones kernel by kernel
            self.shaped_steps = False
            return self._eager_pass(entries, sample, return_logits)
        g["graph"].replay()
        self.launch_count += g["launches"]
        self.n_shaped_steps += 1
        return self._finish_pass(entries, ctx, g["resid"], g["delta"], want_rows, temps, keys, n_want, sample, return_logits)

    def _finish_pass(self, entries, ctx, resid, delta, want_rows, temps, keys, n_want, sample, return_logits) -> StepOutput:
        """Logits of the wanted rows of a pass whose layers have run (or are in the stream), and their sampled ids."""
        n_real = sum(len(e.want) for e in entries)
        out = StepOutput()
        if n_want == 0:
            if return_logits:
                out.logits = torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.device)
            if sample:
                out.token_ids = []
            return out
        logits = self.model.logits(ctx, resid, delta, want_rows, n_want)
        if sample:
            ids_dev = self.workspace.flat("sampled_ids", max(n_want, self.limits.max_num_seqs), torch.int32)[:n_want]
            if ops.sample_scratch_bytes(n_want) > self.sample_scratch.numel() * 4:
                self.sample_scratch = ops.sample_scratch(n_want, self.device)
            ops.sample(ids_dev, logits, temps, None, self.sample_scratch, row_keys=keys)
            host = self.ids_host[:n_want] if n_want <= self.ids_host.numel() else torch.empty(n_want, dtype=torch.int32).pin_memory()
            host.copy_(ids_dev, non_blocking=True)
            self._status_hosts[2].copy_(self.status_dev, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            self._raise_status(self._status_hosts[2])
            out.token_ids = host.tolist()[:n_real]
        if return_logits:
            out.logits = logits[:n_real]
        return out

    # ------------------------------------------------------------------ CUDA graphs
    def buckets(self) -> List[int]:
        """Batch sizes with a captured graph: 1, 2, 4, 8, 16, then steps of 16, and max_num_seqs
        (src/executor.zig:613-626)."""
        top = self.limits.max_num_seqs
        out = [b for b in (1, 2, 4, 8, 16) if b <= top]
        out += list(range(32, top + 1, 16))
        if top not in out:
            out.append(top)
        return out

    def _bucket_for(self, n: int) -> int:
        for b in self.buckets():
            if b >= n:
                return b
        raise StepError(f"{n} sequences exceed max_num_seqs {self.limits.max_num_seqs}")

    def context_class(self, max_ctx: int) -> int:
        """Captured graphs fix their launch shapes, and how the keys of a sequence are best cut into
        parts depends on how many there are: graphs are kept per class of context length (512,
        1024, 2048, ... up to max_model_len) and a step replays the graph of the smallest class
        that holds its longest sequence."""
        bound = 512
        while bound < max_ctx:
            bound *= 2
        return min(bound, self.limits.max_model_len)

    def decode_graph(self, n_seqs: int, max_ctx: int) -> Tuple[int, dict]:
        """(bucket, captured graph) for a step of `n_seqs` single tokens whose longest sequence
        has `max_ctx` keys; captured on first use."""
        bucket = self._bucket_for(n_seqs)
        bound = self.context_class(max_ctx)
        return bucket, (self.graphs.get((bucket, bound)) or self._capture(bucket, bound))

    def _capture(self, bucket: int, ctx_bound: int = 0) -> dict:
        """Warm up once with an all-padding batch (loads kernels, lets the library pick its
        algorithms, creates the workspaces), then record the same launches into a graph
        (src/executor.zig:609-660)."""
        ctx_bound = ctx_bound or self.limits.max_model_len
        V = self.model.spec.vocab_size
        # one array of logits for all graphs (they never run at the same time): a graph of its own per bucket and
        # class would hold gigabytes at a large vocabulary
        if self._graph_logits is None:
            self._graph_logits = torch.empty((self.limits.max_num_seqs, V), dtype=torch.float32, device=self.device)
        logits = self._graph_logits[:bucket]
        ids_dev = self.sampled_dev[:bucket]
        # the warm-up runs sample elsewhere: a step in flight may have left ids in `sampled_dev` that the
        # step this graph is captured for takes its tokens from
        ids_warm = torch.zeros(bucket, dtype=torch.int32, device=self.device)

        def run():
            ctx, want_rows, temps, keys, n_want = self._build_meta([], pad_to=bucket, ctx_bound=ctx_bound)
            ctx.fixed_shapes = True
            self.model.forward(ctx, self.layer_caches, want_rows, n_want, out=logits)
            ops.sample(ids_warm, logits, temps, None, self.sample_scratch, row_keys=keys)

        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            run()
            run()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        # the metadata upload stays outside the graph: build it first, then capture the launches
        ctx, want_rows, temps, keys, n_want = self._build_meta([], pad_to=bucket, ctx_bound=ctx_bound)
        ctx.fixed_shapes = True
        torch.cuda.synchronize(self.device)
        self.workspace.frozen = True
        launches_before = ops.launches()
        try:
            with torch.cuda.graph(graph, stream=stream):
                self.model.forward(ctx, self.layer_caches, want_rows, n_want, out=logits)
                ops.sample(ids_dev, logits, temps, None, self.sample_scratch, row_keys=keys)
        finally:
            self.workspace.frozen = False
        entry = {"graph": graph, "ids": ids_dev, "logits": logits, "launches": ops.launches() - launches_before}
        self.graphs[(bucket, ctx_bound)] = entry
        return entry

    def context_classes(self) -> List[int]:
        """Every class of context length a decode graph is kept for, up to max_model_len."""
        out, bound = [], 512
        while bound < self.limits.max_model_len:
            out.append(bound)
            bound *= 2
        return out + [self.limits.max_model_len]

    def capture_all(self) -> int:
        """Capture the decode graph of every batch-size bucket and context class, as the reference does for its
        buckets when it starts (src/executor.zig:609-660), and the graph of every shape of the other steps, so that
        no step of a run pays for a capture.  Returns how many graphs were captured."""
        made = 0
        for bound in self.context_classes():
            for b in self.buckets():
                if (b, bound) not in self.graphs:
                    self._capture(b, bound)
                    made += 1
        if self.shaped_steps:
            for seqs in self._seq_shapes:
                for rows in self._token_shapes:
                    if (rows, seqs) not in self.shape_graphs:
                        self._capture_shape((rows, seqs))
                        made += 1
        return made

    # ------------------------------------------------------------------ graphs for steps of any kind
    SHAPED_TOKENS_MAX = 2048      # steps of more tokens are launched kernel by kernel: the GPU then lags the host anyway

    def token_shapes(self) -> List[int]:
        """Token rows that a step which is not all single tokens is padded to before it replays a graph: 16 to 256
        in the few-rows products' own steps, then multiples of 128 up to 1,024 (the tiled product's tile: padding
        costs it nothing) and of 256 up to 2,048.  Above that a step's kernels take longer than its launches, and
        capturing a graph for it would cost more than it saves."""
        top = min(self.limits.max_step_tokens, self.SHAPED_TOKENS_MAX)
        out = [16, 32, 48, 64, 96, 128, 192, 256] + list(range(384, 1025, 128)) + list(range(1280, 2049, 256))
        out = [t for t in out if t < top]
        return out + [top]

    def seq_shapes(self) -> List[int]:
        top = self.limits.max_num_seqs
        return [b for b in (8, 64) if b < top] + [top]

    def step_shape(self, entries: Sequence[StepEntry]) -> Optional[Tuple[int, int]]:
        """(token rows, sequences) of the graph that this step replays."""
        n_tokens = sum(len(e.tokens) for e in entries)
        rows = next((t for t in self._token_shapes if t >= n_tokens), None)
        seqs = next((b for b in self._seq_shapes if b >= len(entries)), None)
        if rows is None or seqs is None:
            return None
        return rows, seqs

    def _capture_shape(self, shape: Tuple[int, int]) -> dict:
        """Record the launches of all layers for a step of `shape` into a graph.  They depend on the shape alone:
        the step's arrays have fixed places and sizes in the uploaded block (lists of tiles are padded to the most
        the shape can have) and every kernel runs over all token rows of the shape.  The gather of the wanted rows,
        the output projection and the sampler stay outside: how many rows are wanted is not part of the shape."""
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            ctx = self._build_meta([], shape=shape)[0]      # loads kernels, creates the workspaces
            ctx.fixed_shapes = True
            self.model.hidden_states(ctx, self.layer_caches)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        self.workspace.frozen = True
        launches_before = ops.launches()
        try:
            # the upload of the arrays stays outside the graph
            ctx = self._build_meta([], shape=shape)[0]
            ctx.fixed_shapes = True
            layout = self._shape_layout()
            torch.cuda.synchronize(self.device)
            with torch.cuda.graph(graph, stream=stream):
                resid, delta = self.model.hidden_states(ctx, self.layer_caches)
        finally:
            self.workspace.frozen = False
        entry = {"graph": graph, "resid": resid, "delta": delta, "layout": layout,
                 "launches": ops.launches() - launches_before}
        self.shape_graphs[shape] = entry
        return entry

    def _shape_layout(self) -> dict:
        """Places and sizes of the arrays of the step just laid out, without those that no graph reads."""
        return {k: v for k, v in self._last_fill[1].items() if k not in ("want_rows", "temps", "row_keys")}

    def _graph_step(self, entries: Sequence[StepEntry]) -> StepOutput:
        return StepOutput(None, self.decode_collect(self._decode_launch(entries, None)))

    def decode_launch(self, entries: Sequence[StepEntry], prev_rows: Optional[Sequence[int]] = None) -> "PendingIds":
        """Launch a step of single tokens with sampling and return at once; `decode_collect` waits for
        its ids.  `prev_rows[i] >= 0` says that entry i's token is the id that the step launched just
        before this one sampled in that row (its `tokens` may then be `[None]`): the GPU takes it
        from there, so the host need not have read it.  Only with captured graphs (not `eager`)."""
        entries = [e for e in entries]
        if self.eager:
            raise StepError("decode_launch needs captured graphs (the engine was built with eager=True)")
        if prev_rows is not None and len(prev_rows) != len(entries):
            raise StepError("one previous row (or -1) per entry is required")
        for i, e in enumerate(entries):
            if len(e.tokens) != 1 or list(e.want) != [0]:
                raise StepError("decode_launch takes single tokens whose logits are sampled")
            if e.tokens[0] is None and (prev_rows is None or not 0 <= prev_rows[i] < self.limits.max_num_seqs):
                raise StepError(f"request {e.req!r}: no token and no row of the step before to take it from")
        self._validate(entries, prev_rows)
        self._reset_fresh_state()
        return self._decode_launch(entries, prev_rows)

    def _decode_launch(self, entries, prev_rows) -> "PendingIds":
        n = len(entries)
        bucket, g = self.decode_graph(n, max(e.start for e in entries) + 1)
        self._fill_decode_meta(entries, bucket, prev_rows)
        g["graph"].replay()
        self.launch_count += g["launches"]
        turn = self._ids_turn
        self._ids_turn ^= 1
        host = self._ids_hosts[turn][:n]
        host.copy_(self.sampled_dev[:n], non_blocking=True)
        flags = self._status_hosts[turn]
        flags.copy_(self.status_dev, non_blocking=True)
        self._ids_events[turn].record()
        self.n_graph_steps += 1
        return PendingIds(host, self._ids_events[turn], flags)

    def decode_collect(self, pending: "PendingIds") -> List[int]:
        """The sampled ids of a launched step, in the order of its entries."""
        pending.event.synchronize()
        if pending.flags is not None:
            self._raise_status(pending.flags)
        return pending.host.tolist()

    def _fill_decode_meta(self, entries: Sequence[StepEntry], bucket: int, prev_rows: Optional[Sequence[int]] = None) -> None:
        """The metadata of a step of single tokens.  The first fill of a pinned buffer for a bucket
        goes through `_build_meta`; later ones rewrite only what a decode step changes (tokens,
        positions, lengths, slots, the sampler's keys, and block-table rows whose table grew), with the
        layout of that first fill."""
        turn = self._meta_turn
        owner = self._host_owner[turn]
        if not self._static_step_arrays:
            self._build_meta(entries, pad_to=bucket, ids_from=prev_rows)
            return
        if owner is None or owner[0] != bucket:
            self._build_meta(entries, pad_to=bucket, ids_from=prev_rows)
            t, layout, total = self._last_fill
            names = ["ids", "positions", "ctx_len", "state_slots", "temps", "ids_from", "row_keys"]
            for gi in range(len(self.cache.groups)):
                names += [f"slots_{gi}", f"block_tables_{gi}"]
            offs = (ctypes.c_int * len(names))(*[layout[name][0] for name in names])
            self._host_owner[t] = (bucket, layout, total, offs)
            # (request, table stamp) per group and row; -1 = unknown, so the first native fill writes every row
            stamps = (ctypes.c_longlong * (2 * bucket * len(self.cache.groups)))()
            for i in range(len(stamps)):
                stamps[i] = -1
            self._host_rows[t] = stamps
            return
        _, layout, total, offs = owner
        self._meta_turn ^= 1
        if self.meta_events[turn] is not None:
            self.meta_events[turn].synchronize()
        host = self.meta_host[turn]
        n = len(entries)
        a = self._decode_args
        key = self.cache.key
        a[0][:n] = [key(e.req) for e in entries]
        if prev_rows is None:
            a[1][:n] = [e.tokens[0] for e in entries]
            a[4][:n] = [-1] * n
        else:
            a[1][:n] = [e.tokens[0] if r < 0 else 0 for e, r in zip(entries, prev_rows)]
            a[4][:n] = list(prev_rows)
        a[2][:n] = [e.start for e in entries]
        a[3][:n] = [e.temperature for e in entries]
        rc = self._runtime.llmr_fill_decode(self.cache.native_handle, ctypes.c_void_p(host.data_ptr()), offs,
                                            ctypes.c_int(n), ctypes.c_int(bucket), ctypes.c_int(self.max_blocks),
                                            a[0], a[1], a[4], a[2], a[3], ctypes.c_ulonglong(self.seed), self._host_rows[turn])
        if rc != 0:
            self._host_owner[turn] = None
            raise StepError(self._runtime.llmr_last_error().decode("utf-8", "replace"))
        self.meta_dev[:total].copy_(self.meta_host[turn][:total], non_blocking=True)
        self.last_upload_bytes = 4 * total
        ev = torch.cuda.Event()
        ev.record()
        self.meta_events[turn] = ev
