"""Sampling: parameters, seeds, and the sampler that turns logits into tokens."""

from ayaka_b200.sampling.params import SamplingParams

__all__ = ["SamplingParams"]
