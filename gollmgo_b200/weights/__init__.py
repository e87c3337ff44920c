from .loader import WeightError, WeightSpec, check_manifest, checkpoint_source, storage_dtype
from .random_init import random_source, random_tensor, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, save_file

__all__ = ["WeightError", "WeightSpec", "check_manifest", "checkpoint_source", "storage_dtype",
           "random_source", "random_tensor", "write_random_model", "SafetensorsError",
           "SafetensorsFile", "open_model_files", "save_file"]
