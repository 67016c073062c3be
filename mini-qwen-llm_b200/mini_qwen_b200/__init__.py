"""B200-native MoE block for mini-qwen-llm: the reference's Python call signatures over
libmqmoe.so (hand-written sm_100a kernels behind a C ABI).

The sub-packages mirror the reference's ``mini_qwen`` layout:
``kernels`` (moe_router, moe_permute, moe_grouped_gemm, moe_unpermute, w4a16_gemm),
``model.layers`` (Qwen3MoEBlock, LinearW4A16), ``quantization`` (pack_int4, unpack_int4,
_per_group_minmax_quantize), ``config`` (Qwen3MoEConfig).
"""
from .config import Qwen3MoEConfig

__all__ = ["Qwen3MoEConfig"]
__version__ = "0.1.0"
