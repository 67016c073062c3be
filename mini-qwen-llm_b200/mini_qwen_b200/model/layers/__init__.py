from .linear_w4a16 import LinearW4A16
from .moe import Qwen3MoEBlock

__all__ = ["LinearW4A16", "Qwen3MoEBlock"]
