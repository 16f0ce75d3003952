from .loader import PlacedSource, WeightError, check_checkpoint
from .random_init import random_tensor, random_tensors, random_tensors_on_device, write_random_model
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, open_model_dir, save_file
