"""fieldrun_b200: a small model library with generation of its own for one B200.

From a model folder (config.json + safetensors) to generated tokens, for the
MiniMax-M2 architecture: typed configuration and a registry, weights by tensor
name, layers put together from parts, a paged cache with a slot per sequence, one
step function for batches of unequal lengths, a generation loop with greedy and
temperature sampling, and hand-written CUDA kernels for sm_100a underneath.
"""
from .api import LanguageModel, build_model, load, random_model, write_random_model
from .config import (ConfigError, MiniMaxM2Config, ModelConfig, load_config, register_architecture,
                     registered_architectures)
from .weights import RandomInit, WeightError

__version__ = "0.1.0"

__all__ = ["ConfigError", "LanguageModel", "MiniMaxM2Config", "ModelConfig", "RandomInit", "WeightError",
           "build_model", "load", "load_config", "random_model", "register_architecture",
           "registered_architectures", "write_random_model"]
