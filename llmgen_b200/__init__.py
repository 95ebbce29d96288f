"""llmgen_b200: a single-GPU inference engine for sm_100a (B200), built from parts.

    from llmgen_b200 import LLM, SamplingParams
    llm = LLM("/path/to/model_folder")              # config.json + model.safetensors
    outs = llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=16))
"""
__version__ = "0.1.0"


def __getattr__(name):
    if name in ("LLM", "SamplingParams", "Engine", "EngineConfig"):
        from .engine import api
        return getattr(api, name)
    raise AttributeError(name)
