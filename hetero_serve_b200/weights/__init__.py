from .loader import (WeightError, canonical_names, check_tensors, load_checkpoint,
                     random_weights, write_model_dir)
from .safetensors_io import SafetensorsError, read_safetensors, write_safetensors

__all__ = ["SafetensorsError", "WeightError", "canonical_names", "check_tensors",
           "load_checkpoint", "random_weights", "read_safetensors", "write_model_dir",
           "write_safetensors"]
