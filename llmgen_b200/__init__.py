"""llmgen_b200: a single-GPU inference engine for sm_100a (B200), built from parts.

    from llmgen_b200 import LLM, SamplingParams
    llm = LLM("/path/to/model_folder")              # config.json + model.safetensors
    outs = llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=16))
"""
__version__ = "0.1.0"


# public names and the modules they live in; imported on first use, so that `import llmgen_b200`
# (and the commands that need no GPU) do not load torch
_EXPORTS = {
    "LLM": "engine.api", "load_model": "engine.api", "random_model": "engine.api", "write_random_model": "engine.api",
    "SamplingParams": "sampling.params", "Engine": "engine.engine", "SchedulerConfig": "engine.scheduler",
    "Executor": "engine.executor", "EngineLimits": "engine.executor", "StepEntry": "engine.executor",
    "register_architecture": "registry",
}


def __getattr__(name):
    module = _EXPORTS.get(name)
    if module is None:
        raise AttributeError(f"module 'llmgen_b200' has no attribute {name!r}")
    import importlib
    return getattr(importlib.import_module("." + module, __name__), name)


def __dir__():
    return sorted(list(globals()) + list(_EXPORTS))
