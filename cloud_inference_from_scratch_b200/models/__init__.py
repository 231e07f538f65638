from . import lazilorn, lodalix, qwen2, zisesun  # noqa: F401  (register Qwen2ForCausalLM, Zisesun, Lodalix and Lazilorn)
from .decoder import CacheNeed, DecoderModel, LayerParts

__all__ = ["CacheNeed", "DecoderModel", "LayerParts"]
