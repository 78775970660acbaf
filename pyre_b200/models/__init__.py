from .model import KVGroup, Model, StateGroup, tensor_table
from .spec import LayerCall, ModelSpec

__all__ = ["KVGroup", "LayerCall", "Model", "ModelSpec", "StateGroup", "tensor_table"]
