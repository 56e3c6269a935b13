from .loader import (WeightsError, check_and_bind, load_checkpoint, place_on_device,
                     strip_wrapper_prefixes)
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, load_file, read_header, save_file

__all__ = [n for n in dir() if not n.startswith("_")]
