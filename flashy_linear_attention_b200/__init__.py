"""B200-native (sm_100a) causal linear attention behind the `flashlinear` Python API.

Public surface (same names as the reference package, flashlinear/__init__.py:1-2 and
flashlinear/kernels/__init__.py:1-5):
    LinearAttention, LinearAttentionSmallVHD,
    linear_flash_wrapper_fwd, linear_flash_wrapper_bwd,
    linear_flash_wrapper_fwd_smallv_hd, linear_flash_wrapper_bwd_smallv_hd
plus the lower-level causal_dot_product_fwd / causal_dot_product_bwd (running-state arguments),
LinearAttentionResumable (state carried across calls), LinearAttentionNormalized (the README's
denominator fused into streaming kernels) and host.HostPipeline (pinned host tensors).
"""
from .functions import (
    LinearAttention,
    LinearAttentionNormalized,
    LinearAttentionResumable,
    LinearAttentionSmallVHD,
    TaylorLinearAttention,
)
from .ops import (
    causal_dot_product_bwd,
    causal_dot_product_fwd,
    check_status,
    chunk_state,
    linear_flash_wrapper_bwd,
    linear_flash_wrapper_bwd_smallv_hd,
    linear_flash_wrapper_fwd,
    linear_flash_wrapper_fwd_smallv_hd,
)

__all__ = [
    "LinearAttention",
    "LinearAttentionSmallVHD",
    "LinearAttentionResumable",
    "LinearAttentionNormalized",
    "TaylorLinearAttention",
    "linear_flash_wrapper_fwd",
    "linear_flash_wrapper_bwd",
    "linear_flash_wrapper_fwd_smallv_hd",
    "linear_flash_wrapper_bwd_smallv_hd",
    "causal_dot_product_fwd",
    "causal_dot_product_bwd",
    "check_status",
    "chunk_state",
]
