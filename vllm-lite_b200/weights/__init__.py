"""Weights: the safetensors container, binding by name, random initialisation."""
from .loader import WeightError, find_weight_files, load_weights, resident_dtype  # noqa: F401
from .random_init import random_tensors, write_model_dir  # noqa: F401
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors  # noqa: F401
