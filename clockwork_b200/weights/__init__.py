from .decl import TensorDecl
from .loader import WeightMismatchError, check_declarations, load_checkpoint_into
from .random_init import fill_model_on_device, write_random_model
from .safetensors_io import CheckpointIndex, SafetensorsError, SafetensorsFile, save_safetensors

__all__ = [
    "TensorDecl", "WeightMismatchError", "check_declarations", "load_checkpoint_into",
    "fill_model_on_device", "write_random_model",
    "CheckpointIndex", "SafetensorsError", "SafetensorsFile", "save_safetensors",
]
