"""Weights: the safetensors container, loading by tensor name, random initialisation."""

from .loader import bind_tensors, check_tensors, inspect_folder, load_model, parse_dtype
from .random_init import random_tensors, write_model_folder
from .safetensors_io import SafetensorsFolder, write_safetensors
