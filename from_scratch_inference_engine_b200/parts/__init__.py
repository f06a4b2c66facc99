from .base import (LayerCache, Mixer, Part, StateNeed, build_part, register_part,
                   registered_parts, unregister_part)
from . import (norm, rope, attention, lightning, talking_attention, mlp, block, mingru,   # registers
               scaled_attention, latent_attention, routed_experts, inlet, state_space,  # the built-in
               parallel_mixers)                                                       # kinds
from .model import DecoderModel, tensor_specs

__all__ = ["LayerCache", "Mixer", "Part", "StateNeed", "build_part", "register_part",
           "registered_parts", "unregister_part", "DecoderModel", "tensor_specs"]
