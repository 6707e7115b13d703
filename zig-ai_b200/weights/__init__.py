from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .loader import WeightError, load_tensors
from .random_init import random_tensors, write_random_model
