"""Drop-in for the reference's flashlinear/kernels/__init__.py:1-5 (the four launch wrappers)."""
from flashy_linear_attention_b200.ops import (
    linear_flash_wrapper_bwd,
    linear_flash_wrapper_bwd_smallv_hd,
    linear_flash_wrapper_fwd,
    linear_flash_wrapper_fwd_smallv_hd,
)

__all__ = [
    "linear_flash_wrapper_fwd",
    "linear_flash_wrapper_bwd",
    "linear_flash_wrapper_fwd_smallv_hd",
    "linear_flash_wrapper_bwd_smallv_hd",
]
