from .safetensors_io import SafetensorsFile, SafetensorsError, write_safetensors, open_model_files
from .loader import WeightError, load_model_weights, check_and_load, held_dtype
from .random_init import write_random_model, random_state_dict, random_tensors_on_device
