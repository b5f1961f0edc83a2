from .loader import load_tensors, open_folder
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors, write_streamed
