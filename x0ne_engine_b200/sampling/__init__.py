"""Sampling options; the device sampler itself is `csrc/sampling.cu` (called through csrc.ops.sample)."""
from .params import GREEDY_BELOW, PromptTooLong, SamplingParams, fresh_seed, generation_budget

__all__ = ["GREEDY_BELOW", "PromptTooLong", "SamplingParams", "fresh_seed", "generation_budget"]
