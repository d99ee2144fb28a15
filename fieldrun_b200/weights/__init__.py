from .loader import (MATRIX, TABLE, VECTOR, FolderSource, MemorySource, TensorNeed, TensorSource, WeightError,
                     check_needs, held_dtype)
from .random_init import RandomInit, write_model_folder
from .safetensors_io import ModelFolder, TensorToWrite, WeightFileError, read_header, write_safetensors

__all__ = [
    "MATRIX", "TABLE", "VECTOR", "FolderSource", "MemorySource", "ModelFolder", "RandomInit", "TensorNeed",
    "TensorSource", "TensorToWrite", "WeightError", "WeightFileError", "check_needs", "held_dtype", "read_header",
    "write_model_folder", "write_safetensors",
]
