"""Selector with the reference's signature (dot_production_attention/__init__.py:4-26).
There is one implementation here — the CUDA kernels — whatever the flag says."""
from typing import Tuple

from .cuda_impl import CudaMultiStageDotProductionAttention


def get_multi_stage_dot_production_attention(flash_attn=False) -> Tuple[type, bool]:
    return CudaMultiStageDotProductionAttention, True


__all__ = ["CudaMultiStageDotProductionAttention", "get_multi_stage_dot_production_attention"]
