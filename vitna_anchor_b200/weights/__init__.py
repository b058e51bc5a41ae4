from .loader import WeightMismatch, WeightSpec, load_weights  # noqa: F401
from .random_init import random_weights, write_model_folder  # noqa: F401
from .safetensors_io import CheckpointError, SafetensorsFile, write_safetensors  # noqa: F401
