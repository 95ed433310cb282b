from .safetensors_io import SafetensorsFile, write_safetensors, SafetensorsFormatError
from .loader import WeightError, load_tensors, check_against_specs, WEIGHT_FILE
from .random_init import write_random_model, random_tensors
