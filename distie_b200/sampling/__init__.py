"""Token selection: greedy and temperature sampling."""

from .sampler import Sampler, uniform

__all__ = ["Sampler", "uniform"]
