from .params import SamplingParams
from .uniform import uniform

__all__ = ["SamplingParams", "uniform"]
