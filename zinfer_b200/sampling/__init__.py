from .params import SamplingParams
from .sampler import Sampler
from .stop import StopAnalysis, analyze_generated

__all__ = ["Sampler", "SamplingParams", "StopAnalysis", "analyze_generated"]
