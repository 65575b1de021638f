"""`torch.autograd.Function`s with the interface of the reference's
``flashlinear.LinearAttention`` (flashlinear/linear_attn.py:11-31) and
``flashlinear.LinearAttentionSmallVHD`` (flashlinear/linear_attn_smallv_hd.py:14-36):
``.apply(q, k, v)`` returns the unnormalised causal ``(Q K^T (.) M) V`` in bf16, saves q, k, v and
returns three bf16 gradients from backward. Under autocast the inputs are cast to bf16 exactly as
the reference's ``custom_fwd(cast_inputs=torch.bfloat16)`` does.
"""
from __future__ import annotations

from typing import Any, Tuple

import torch
from torch.autograd import Function

from .ops import (
    linear_flash_wrapper_bwd,
    linear_flash_wrapper_bwd_smallv_hd,
    linear_flash_wrapper_fwd,
    linear_flash_wrapper_fwd_smallv_hd,
)


class LinearAttention(Function):
    """Causal linear attention with dk == dv."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx: Any, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        out = linear_flash_wrapper_fwd(q, k, v)
        ctx.save_for_backward(q, k, v)
        return out

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx: Any, grad_output: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        query, key, value = ctx.saved_tensors
        gradq, gradk, gradv = linear_flash_wrapper_bwd(grad_output, query, key, value)
        return gradq, gradk, gradv


class LinearAttentionSmallVHD(Function):
    """Causal linear attention where q/k have head dim hd_qk and v has a smaller hd_v."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx: Any, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        out = linear_flash_wrapper_fwd_smallv_hd(q, k, v)
        ctx.save_for_backward(q, k, v)
        return out

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx: Any, grad_output: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        query, key, value = ctx.saved_tensors
        gradq, gradk, gradv = linear_flash_wrapper_bwd_smallv_hd(grad_output, query, key, value)
        return gradq, gradk, gradv
