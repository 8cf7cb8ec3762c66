from .host import HostSampler, SplitMix64, argmax
from .params import SamplingParams

__all__ = ["HostSampler", "SplitMix64", "argmax", "SamplingParams"]
