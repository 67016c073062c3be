"""The configuration fields the MoE block reads (the reference's ``mini_qwen/config.py:50-69``)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class Qwen3MoEConfig:
    """Defaults are the Qwen3-30B-A3B MoE layer."""
    hidden_size: int = 2048
    intermediate_size: int = 768      # per expert (HF: moe_intermediate_size)
    num_experts: int = 128
    num_experts_per_tok: int = 8
    norm_topk_prob: bool = True       # divide the K routing weights by their sum

    @classmethod
    def from_hf_config(cls, hf_config) -> "Qwen3MoEConfig":
        inter = getattr(hf_config, "moe_intermediate_size", None)
        if inter is None:
            inter = hf_config.intermediate_size
        return cls(
            hidden_size=hf_config.hidden_size,
            intermediate_size=inter,
            num_experts=getattr(hf_config, "num_experts", 128),
            num_experts_per_tok=getattr(hf_config, "num_experts_per_tok", 8),
            norm_topk_prob=getattr(hf_config, "norm_topk_prob", True),
        )
