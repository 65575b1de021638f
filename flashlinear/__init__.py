"""Drop-in import name: ``from flashlinear import LinearAttention, LinearAttentionSmallVHD``
(the reference's flashlinear/__init__.py:1-2), served by the sm_100a kernels of
flashy_linear_attention_b200."""
from flashy_linear_attention_b200.functions import LinearAttention, LinearAttentionSmallVHD

__all__ = ["LinearAttention", "LinearAttentionSmallVHD"]
