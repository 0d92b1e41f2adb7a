"""Weights: the safetensors container, loading by tensor name, and the random-weights mode."""
from .loader import TensorDecl, WeightsError, load_weights  # noqa: F401
from .random_init import normal_values, random_tensors, random_tensors_on_device, write_random_model  # noqa: F401
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors  # noqa: F401
