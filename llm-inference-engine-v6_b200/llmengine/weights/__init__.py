"""Checkpoint reading (safetensors by tensor name) and the random-weights mode."""
from .loader import Checkpoint, WeightError, load_tensors, merge_needs
from .random_init import model_tensor_needs, random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, list_safetensors, write_safetensors

__all__ = ["Checkpoint", "WeightError", "load_tensors", "merge_needs", "model_tensor_needs", "random_tensors",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "list_safetensors", "write_safetensors"]
