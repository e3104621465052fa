from . import attention, block, embedding, latent_attention, loop, mlp, moe, norm, position, wkv  # noqa: F401  (registration)
from .base import CATEGORIES, Part, Runtime, build_part, part_class, register_part

__all__ = ["CATEGORIES", "Part", "Runtime", "build_part", "part_class", "register_part"]
