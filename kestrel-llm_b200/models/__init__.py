from .decoder import DecoderModel, LayerCall
from . import qwen3  # registers "Qwen3ForCausalLM"
from . import zidivik  # registers "Zidivik"

__all__ = ["DecoderModel", "LayerCall", "qwen3", "zidivik"]
