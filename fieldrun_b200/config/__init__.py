from .base import ConfigError, KeyReader, ModelConfig, read_config_json
from .minimax_m2 import MiniMaxM2Config
from .plan import LayerSpec, ModelPlan, PartSpec, RunSpec, default_run_order
from .registry import (Architecture, architecture_for, load_config, register_architecture,
                       registered_architectures)

__all__ = [
    "Architecture", "ConfigError", "KeyReader", "LayerSpec", "MiniMaxM2Config", "ModelConfig", "ModelPlan",
    "PartSpec", "RunSpec", "architecture_for", "default_run_order", "load_config", "read_config_json",
    "register_architecture", "registered_architectures",
]
