from . import bilipel, lazilorn, lodalix, qwen2, zisesun  # noqa: F401  (register Qwen2ForCausalLM, Zisesun, Lodalix, Lazilorn and Bilipel)
from .decoder import CacheNeed, DecoderModel, LayerParts

__all__ = ["CacheNeed", "DecoderModel", "LayerParts"]
