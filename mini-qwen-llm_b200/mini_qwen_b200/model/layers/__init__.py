from .linear_w4a16 import LinearW4A16
from .moe import Qwen3MoEBlock
from .rms_norm import RMSNorm, rms_norm

__all__ = ["LinearW4A16", "Qwen3MoEBlock", "RMSNorm", "rms_norm"]
