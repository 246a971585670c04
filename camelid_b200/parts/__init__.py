from .base import Part, TensorSpec, build_block, build_part, known_parts, register_part
from . import (norm, position, attention, feedforward, embedding, block, shift, loop, window_attention,  # noqa: F401
               recurrent, parallel, experts, side_input, latent_attention)                                                                    # (registers the parts)

__all__ = ["Part", "TensorSpec", "build_block", "build_part", "known_parts", "register_part"]
