from .loader import FolderSource, check_names_and_shapes, load_into
from .random_init import InitSpec, RandomSource, parameter_specs, write_model_folder
from .safetensors_io import open_model_folder, read_header, read_tensor, write_safetensors

__all__ = ["FolderSource", "check_names_and_shapes", "load_into", "InitSpec", "RandomSource", "parameter_specs",
           "write_model_folder", "open_model_folder", "read_header", "read_tensor", "write_safetensors"]
