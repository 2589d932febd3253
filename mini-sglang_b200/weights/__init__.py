from .loader import CheckpointSource, RandomSource, TensorDecl, WeightsError, check_index, kept_dtype
from .random_init import write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_dir, write_safetensors

__all__ = ["CheckpointSource", "RandomSource", "TensorDecl", "WeightsError", "check_index", "kept_dtype",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "open_model_dir", "write_safetensors"]
