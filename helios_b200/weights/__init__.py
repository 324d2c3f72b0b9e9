from .loader import WeightsError, bind_tensors, expected_tensors, load_weights, shard_files
from .random_init import (bind_random_weights, random_tensors, write_byte_tokenizer,
                          write_model_folder)

__all__ = ["WeightsError", "bind_tensors", "expected_tensors", "load_weights", "shard_files",
           "bind_random_weights", "random_tensors", "write_byte_tokenizer", "write_model_folder"]
