"""Weights: the safetensors container, the checked loader, the random-weights writer."""

from .loader import DictSource, WeightStore, WeightsError, check_checkpoint, open_weights
from .random_init import RandomSource, random_tensors, write_random_model
from .safetensors_io import ModelTensors, SafetensorsError, SafetensorsFile, save_file

__all__ = [
    "DictSource",
    "ModelTensors",
    "RandomSource",
    "SafetensorsError",
    "SafetensorsFile",
    "WeightStore",
    "WeightsError",
    "check_checkpoint",
    "open_weights",
    "random_tensors",
    "save_file",
    "write_random_model",
]
