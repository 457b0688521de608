from .loader import WeightError, load_weights
from .random_init import init_random, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_checkpoint, write_safetensors
