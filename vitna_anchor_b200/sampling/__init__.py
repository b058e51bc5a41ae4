from .params import SamplingParams, SplitMix64  # noqa: F401
