from .safetensors_io import SafetensorsFile, write_safetensors, open_model_files
from .loader import load_weights, check_tensors
