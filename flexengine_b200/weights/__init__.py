from .loader import CheckpointError, check_against_plan, load_model, random_model
from .random_init import checkpoint_tensors, random_tensor, write_random_model
from .safetensors_io import CheckpointFormatError, CheckpointReader, write_safetensors

__all__ = ["CheckpointError", "check_against_plan", "load_model", "random_model", "checkpoint_tensors",
           "random_tensor", "write_random_model", "CheckpointFormatError", "CheckpointReader", "write_safetensors"]
