from . import attention, block, embedding, mlp, norm, rotary  # noqa: F401  (register the built-in parts)
from .base import (BoundCall, HeadGeometry, PagedKVSpec, Part, PartSpec, PositionEncoding, StateSpec, all_graph_safe, collect_libraries, collect_tensors,
                   load_part, make_part, register_part, registered_parts)

__all__ = ["BoundCall", "HeadGeometry", "PagedKVSpec", "Part", "PartSpec", "PositionEncoding", "StateSpec", "collect_libraries", "collect_tensors",
           "load_part", "make_part", "register_part", "registered_parts"]
