"""Sampling: per-request parameters here, the GPU sampler in `csrc/sampling.cu`
(`llmgen_b200.kernels.ops.sample`): greedy and temperature (Gumbel-max) sampling, the two the
reference's engine path offers (src/backend/cuda/sample/sample.cu:33-77)."""
from .params import SamplingParams

__all__ = ["SamplingParams"]
