from .loader import WeightError, WeightStore, open_weights, weights_from_dict
from .random_init import random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, TensorDirectory, write_safetensors

__all__ = ["WeightError", "WeightStore", "open_weights", "weights_from_dict", "random_tensors",
           "write_model_folder", "SafetensorsError", "TensorDirectory", "write_safetensors"]
