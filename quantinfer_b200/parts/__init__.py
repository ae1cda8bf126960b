from . import (attention, block, embedding, ffn, gated_attention, gated_delta, latent_attention, lightning_attention, mamba2, mingru, moe, norm,
               parallel_mixers, position, reentry, short_conv, time_mix)  # noqa: F401  (registers the built-in kinds)
from .base import Part, Runtime, build_part, part_class, register_part
from .linear import Linear

__all__ = ["Part", "Runtime", "build_part", "part_class", "register_part", "Linear"]
