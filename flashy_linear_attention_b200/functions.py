"""`torch.autograd.Function`s with the interface of the reference's
``flashlinear.LinearAttention`` (flashlinear/linear_attn.py:11-31) and
``flashlinear.LinearAttentionSmallVHD`` (flashlinear/linear_attn_smallv_hd.py:14-36):
``.apply(q, k, v)`` returns the unnormalised causal ``(Q K^T (.) M) V`` in bf16, saves q, k, v (plus
the small fp32 final state when the backward can use it) and returns three bf16 gradients from
backward. Under autocast the inputs are cast to bf16 exactly as
the reference's ``custom_fwd(cast_inputs=torch.bfloat16)`` does.
"""
from __future__ import annotations

from typing import Any, Tuple

import torch
from torch.autograd import Function

from . import ops
from .ops import (
    linear_flash_wrapper_bwd,
    linear_flash_wrapper_bwd_smallv_hd,
    linear_flash_wrapper_fwd,
    linear_flash_wrapper_fwd_smallv_hd,
)


def _forward_with_state(ctx: Any, q, k, v, smallv: bool):
    """Forward through the reference-named wrapper's checks; when a backward will follow and can
    use it, also keeps the final state S = sum k^T v (fp32, batch*heads x dk x dv), which lets the
    backward read q, k, v, dO from HBM once instead of twice."""
    want_state = any(ctx.needs_input_grad[:3]) and q.is_cuda and ops.backward_uses_final_state(q, v)
    if not want_state:
        out = linear_flash_wrapper_fwd_smallv_hd(q, k, v) if smallv else linear_flash_wrapper_fwd(q, k, v)
        ctx.save_for_backward(q, k, v)
        ctx.has_state = False
        return out
    ops.check_forward_preconditions(q, v, smallv)
    B, H, _, dk = q.shape
    s_final = torch.empty(B * H, dk, v.shape[-1], dtype=torch.float32, device=q.device)
    out = ops.causal_dot_product_fwd(q, k, v, s_final=s_final)
    ctx.save_for_backward(q, k, v, s_final)
    ctx.has_state = True
    return out


def _backward_with_state(ctx: Any, grad_output, smallv: bool):
    if not ctx.has_state:
        query, key, value = ctx.saved_tensors
        fn = linear_flash_wrapper_bwd_smallv_hd if smallv else linear_flash_wrapper_bwd
        return fn(grad_output, query, key, value)
    query, key, value, s_final = ctx.saved_tensors
    return ops.causal_dot_product_bwd(grad_output, query, key, value, s_last=s_final)


class LinearAttention(Function):
    """Causal linear attention with dk == dv."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx: Any, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        return _forward_with_state(ctx, q, k, v, smallv=False)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx: Any, grad_output: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        gradq, gradk, gradv = _backward_with_state(ctx, grad_output, smallv=False)
        return gradq, gradk, gradv


class LinearAttentionSmallVHD(Function):
    """Causal linear attention where q/k have head dim hd_qk and v has a smaller hd_v."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx: Any, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        return _forward_with_state(ctx, q, k, v, smallv=True)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx: Any, grad_output: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        gradq, gradk, gradv = _backward_with_state(ctx, grad_output, smallv=True)
        return gradq, gradk, gradv
