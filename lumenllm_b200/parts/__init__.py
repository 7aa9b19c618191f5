from .base import (CATEGORIES, Runtime, build_part, part_class, part_tensors, register_part)
from . import norm, position, attention, mlp, block, embed_head  # noqa: F401  (registration)
from .linear import Linear

__all__ = ["CATEGORIES", "Runtime", "build_part", "part_class", "part_tensors", "register_part",
           "Linear"]
