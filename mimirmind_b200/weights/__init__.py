from .safetensors_io import SafetensorsError, SafetensorsFolder, write_safetensors
from .store import (WeightsError, expected_tensors, load_spec, load_tensors, parse_dtype, random_tensors,
                    write_random_model)

__all__ = ["SafetensorsError", "SafetensorsFolder", "write_safetensors", "WeightsError", "expected_tensors",
           "load_spec", "load_tensors", "parse_dtype", "random_tensors", "write_random_model"]
