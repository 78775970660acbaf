from .loader import WeightsError, check_names_and_shapes, find_shards, load_tensors
from .random_init import expected_tensors, random_state, random_tensors_on_device, write_random_model
from .specs import TensorSpec

__all__ = ["TensorSpec", "WeightsError", "check_names_and_shapes", "expected_tensors", "find_shards",
           "load_tensors", "random_state", "random_tensors_on_device", "write_random_model"]
