"""Kernel entry points with the call signatures of the reference's ``mini_qwen.kernels``."""
from .moe_router import moe_router
from .moe_permute import moe_permute, moe_permute_plan
from .moe_unpermute import moe_unpermute
from .moe_grouped_gemm import moe_grouped_gemm, moe_grouped_swiglu, moe_grouped_swiglu_gather
from .w4a16_gemm import w4a16_gemm, w4a16_grouped_gemm, w4a16_grouped_swiglu

__all__ = ["moe_router", "moe_permute", "moe_permute_plan", "moe_unpermute", "moe_grouped_gemm",
           "moe_grouped_swiglu", "moe_grouped_swiglu_gather", "w4a16_gemm", "w4a16_grouped_gemm", "w4a16_grouped_swiglu"]
