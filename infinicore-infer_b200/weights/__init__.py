"""Weights: safetensors by tensor name, one error for everything that does not fit, random mode."""
from .loader import (KEEP, MATRIX, TABLE, VECTOR, DictWeights, FileWeights, TensorDecl,
                     UnusedTensorsWarning, WeightError, WeightSource, check_manifest, stored_dtype)
from .random_init import DeviceRandomWeights, random_tensors, write_model_folder
from .safetensors_io import (SafetensorsError, TensorInfo, index_directory, read_header,
                             read_tensor, write_file)

__all__ = [
    "KEEP", "MATRIX", "TABLE", "VECTOR", "DictWeights", "FileWeights", "TensorDecl", "WeightError", "UnusedTensorsWarning",
    "WeightSource", "check_manifest", "stored_dtype", "DeviceRandomWeights", "random_tensors",
    "write_model_folder", "SafetensorsError", "TensorInfo", "index_directory", "read_header",
    "read_tensor", "write_file",
]
