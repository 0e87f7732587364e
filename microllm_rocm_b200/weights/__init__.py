from .safetensors import SafetensorsFile, SafetensorsError, save_file, inspect_file, open_model_files
from .loader import load_weights, WeightLoadError, LoadReport, check_names
from .random_init import write_random_model, init_random, random_tensors
