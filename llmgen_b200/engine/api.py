"""The Python entry point: load a model folder (or draw random weights) and generate.

    llm = LLM(model_dir, dtype="bfloat16", max_model_len=4096, ...)
    outputs = llm.generate(list_of_prompt_ids, SamplingParams(temperature=0, max_tokens=32))
    # outputs[i]["token_ids"] are the generated ids of prompt i

The reference has no Python API; the keyword names are its command-line options
(src/cli.zig:33-62): max_num_seqs, max_model_len, max_batched_tokens, pass_tokens,
block_size, gpu_util, kv_blocks, policy, chunk, eager, sync_each.
"""
from __future__ import annotations

import contextlib
import os
import tempfile
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..parts.registry import model_weight_decls
from ..registry import config_from_dict, config_from_folder
from ..sampling.params import SamplingParams
from ..weights import open_weights, random_tensors, weights_from_dict, write_model_folder
from .engine import Engine
from .executor import DEFAULT_SEED, EngineLimits, Executor
from .model import DecoderModel
from .scheduler import PREFILL_FIRST, SchedulerConfig

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, not {dtype!r}") from None


def require_cuda(device="cuda:0") -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("llmgen_b200 runs on a CUDA device (sm_100a); none is visible and there is no CPU path")
    dev = torch.device(device)
    torch.cuda.set_device(dev)
    # true float32 and exact bfloat16 accumulation in any library product
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    return dev


def load_model(model_dir: str, dtype=torch.bfloat16, device="cuda:0") -> DecoderModel:
    """config.json chooses the architecture; tensors are checked against what it declares."""
    dev = require_cuda(device)
    arch, cfg = config_from_folder(model_dir)
    spec = arch.build_spec(cfg)
    weights = open_weights(model_dir, model_weight_decls(spec), spec.ignorable_tensors, spec.same_as)
    return DecoderModel(spec, weights, resolve_dtype(dtype), dev)


def write_random_model(model_dir: str, config: dict, seed: int, sigma: Optional[float] = None,
                       sigma_norm: Optional[float] = None, store_dtype=torch.bfloat16) -> str:
    """The random-weights mode: a model folder (config.json, model.safetensors) from a
    configuration dict and a seed."""
    arch, cfg = config_from_dict(config)
    spec = arch.build_spec(cfg)
    tensors = random_tensors(model_weight_decls(spec), seed,
                             spec.init_sigma if sigma is None else sigma,
                             spec.init_sigma_norm if sigma_norm is None else sigma_norm,
                             resolve_dtype(store_dtype))
    out_cfg = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(config)
    out_cfg["torch_dtype"] = "bfloat16" if resolve_dtype(store_dtype) == torch.bfloat16 else "float32"
    return write_model_folder(model_dir, out_cfg, tensors)


def random_model(config: dict, seed: int, dtype=torch.bfloat16, device="cuda:0", sigma: Optional[float] = None,
                 sigma_norm: Optional[float] = None, store_dtype=torch.bfloat16, init_on_device: bool = False) -> DecoderModel:
    """A model with random weights without touching the disk (same values as `write_random_model` with the
    same arguments, unless `init_on_device`: the tensors are then drawn by the GPU's generator, which is what
    benchmarks of models of tens of gigabytes use)."""
    dev = require_cuda(device)
    arch, cfg = config_from_dict(config)
    spec = arch.build_spec(cfg)
    decls = model_weight_decls(spec)
    tensors = random_tensors(decls, seed, spec.init_sigma if sigma is None else sigma,
                             spec.init_sigma_norm if sigma_norm is None else sigma_norm, resolve_dtype(store_dtype),
                             device=dev if init_on_device else "cpu")
    return DecoderModel(spec, weights_from_dict(tensors, decls), resolve_dtype(dtype), dev)


class LLM:
    def __init__(self, model: Union[str, DecoderModel], dtype="bfloat16", device="cuda:0", seed: int = DEFAULT_SEED,
                 max_num_seqs: int = 256, max_model_len: int = 4096, max_batched_tokens: int = 16384,
                 pass_tokens: int = 8192, block_size: int = 16, gpu_util: float = 0.9, kv_blocks: int = 0,
                 policy: str = PREFILL_FIRST, chunk: int = 2048, eager: bool = False, sync_each: bool = False,
                 capture_at_start: bool = True):
        """`capture_at_start`: record the CUDA graph of every decode batch size and context class now (unless
        `eager`), as the reference does when it starts; `load_seconds` then includes it.  False leaves each
        graph to the first step that needs it."""
        t0 = time.perf_counter()
        self.model = model if isinstance(model, DecoderModel) else load_model(model, dtype, device)
        limits = EngineLimits(max_num_seqs=max_num_seqs, max_model_len=max_model_len, max_step_tokens=pass_tokens,
                              page_size=block_size, num_pages=kv_blocks or None, gpu_util=gpu_util)
        self.executor = Executor(self.model, limits, seed=seed, eager=eager, sync_each=sync_each)
        self.engine = Engine(self.executor, SchedulerConfig(
            max_num_seqs=max_num_seqs, max_num_batched_tokens=max_batched_tokens, policy=policy,
            chunk_tokens=chunk, eos_token_ids=tuple(self.model.spec.eos_token_ids)))
        self.graphs_captured = 0
        if capture_at_start and not self.executor.eager:
            self.graphs_captured = self.executor.capture_all()
            torch.cuda.synchronize(self.executor.device)
        self.load_seconds = time.perf_counter() - t0      # weights, cache, workspaces and graph capture

    @contextlib.contextmanager
    def profile(self):
        """`with llm.profile() as prof: llm.generate(...)`, then `prof.text()` or `prof.rows(phase)`: device time,
        FLOPs and bytes of every kernel by phase (`engine.profiler.OpProfiler`).  Only launches made directly
        are seen, so the engine must have been built with `eager=True`."""
        from .profiler import OpProfiler
        if not self.executor.eager:
            raise ValueError("profiling needs eager steps: build the LLM with eager=True")
        prof = OpProfiler().enable()
        self.executor.profiler = prof
        try:
            yield prof
        finally:
            prof.disable()
            self.executor.profiler = None

    def generate(self, prompts: Sequence[Sequence[int]], params: Union[SamplingParams, Sequence[SamplingParams], None] = None
                 ) -> List[Dict]:
        """Token ids in, token ids out: submits all prompts together and runs until done."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        requests = [self.engine.add_request(p, sp) for p, sp in zip(prompts, params)]
        self.engine.run_until_done()
        outs = [{"request_id": r.id, "prompt_token_ids": r.token_ids[:r.num_prompt_tokens],
                 "token_ids": r.completion, "num_preemptions": r.num_preemptions} for r in requests]
        self.engine.release_finished()
        return outs
