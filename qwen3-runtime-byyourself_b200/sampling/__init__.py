"""Sampling: options, the per-sequence random stream, and the GPU sampler."""
from .params import SamplingParams, uniform_for

__all__ = ["SamplingParams", "uniform_for", "Sampler", "NonFiniteLogits"]


def __getattr__(name):  # the sampler needs torch and the CUDA extension; the options do not
    if name in ("Sampler", "NonFiniteLogits"):
        from . import sampler
        return getattr(sampler, name)
    raise AttributeError(name)
