from .model import KVGroup, Model, StateGroup, load_model, tensor_table
from .spec import LayerCall, ModelSpec

__all__ = ["KVGroup", "LayerCall", "Model", "ModelSpec", "StateGroup", "load_model", "tensor_table"]
