from .safetensors_io import FolderReader, WeightError, folder_index, read_header, save_tensors
from .loader import check_names, load_folder
from .random_init import random_tensor, random_tensors, write_random_model

__all__ = ["FolderReader", "WeightError", "folder_index", "read_header", "save_tensors", "check_names",
           "load_folder", "random_tensor", "random_tensors", "write_random_model"]
