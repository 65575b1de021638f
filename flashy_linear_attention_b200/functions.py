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
    ctx.keep_padded = False
    if smallv and q.is_cuda and q.shape[-1] % 8 != 0 and any(ctx.needs_input_grad[:3]):
        # Head dims such as 273 have rows the kernels cannot address in place. Repack q and k once,
        # keep the repacked views for the backward, and let the backward return dQ and dK as views
        # of row-padded tensors (same values and shape as the reference's gradients, which are
        # contiguous, linear_attn_kernels_smallv_hd.py:384-386; one copy pass per tensor less).
        ops.check_forward_preconditions(q, v, smallv)
        q, k = ops.kernel_view(q), ops.kernel_view(k)
        ctx.keep_padded = True
    if not want_state:
        out = linear_flash_wrapper_fwd_smallv_hd(q, k, v) if smallv else linear_flash_wrapper_fwd(q, k, v)
        ctx.save_for_backward(q, k, v)
        ctx.has_state = False
        return out
    ops.check_forward_preconditions(q, v, smallv)
    B, H, _, dk = q.shape
    s_final = torch.empty(B * H, dk, v.shape[-1], dtype=torch.float32, device=q.device)
    # few heads per GPU: the forward is split into segments and also hands the state at the segment
    # boundaries to the backward
    seg_states = ops.segment_states_buffer(q, v)
    out = ops.causal_dot_product_fwd(q, k, v, s_final=s_final, seg_states=seg_states)
    if seg_states is None:
        ctx.save_for_backward(q, k, v, s_final)
    else:
        ctx.save_for_backward(q, k, v, s_final, seg_states)
    ctx.has_state = True
    return out


def _backward_with_state(ctx: Any, grad_output, smallv: bool):
    if not ctx.has_state:
        query, key, value = ctx.saved_tensors
        if ctx.keep_padded:
            return ops.causal_dot_product_bwd(grad_output, query, key, value, keep_padded=True)
        fn = linear_flash_wrapper_bwd_smallv_hd if smallv else linear_flash_wrapper_bwd
        return fn(grad_output, query, key, value)
    query, key, value, s_final = ctx.saved_tensors[:4]
    seg_states = ctx.saved_tensors[4] if len(ctx.saved_tensors) > 4 else None
    return ops.causal_dot_product_bwd(grad_output, query, key, value, s_last=s_final, seg_states=seg_states)


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


class LinearAttentionResumable(Function):
    """Causal linear attention that carries its running state across calls.

    ``out, s_final = LinearAttentionResumable.apply(q, k, v, s_init)`` where ``s_init`` /
    ``s_final`` are fp32 ``[batch, heads, dk, dv]`` (sum of k_j^T v_j over the tokens before /
    up to the end of this call; ``s_init=None`` starts from zero). Feeding ``s_final`` of one call
    as ``s_init`` of the next gives what one call over the concatenated tokens gives: chunked
    prefill, decoding a few tokens at a time, or training on a long sequence piece by piece. Any
    number of tokens per call is accepted (the reference's multiple-of-64 rule,
    linear_attn_kernels.py:323-325, is a property of its tiling; a call of one token still costs a
    whole 128-token tile here, so decode in blocks where possible). The state is
    differentiable: the backward returns the gradient of ``s_init`` and accepts one for ``s_final``.

    Not part of the reference, whose Functions (flashlinear/linear_attn.py:11-31) always start from
    an empty state. Head dims up to 128.
    """

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx: Any, q, k, v, s_init=None):
        assert q.shape[-1] <= ops.KERNEL_HEAD_DIM and v.shape[-1] <= ops.KERNEL_HEAD_DIM, \
            f"Only head_dims <= {ops.KERNEL_HEAD_DIM} are supported."
        B, H, _, dk = q.shape
        dv = v.shape[-1]
        if s_init is not None:
            # autocast's cast_inputs also turns the fp32 state to bf16; the state stays fp32
            s_init = s_init.to(torch.float32).contiguous()
            if tuple(s_init.shape) != (B, H, dk, dv):
                raise ValueError(f"s_init must have shape {(B, H, dk, dv)}")
        s_final = torch.empty(B, H, dk, dv, dtype=torch.float32, device=q.device)
        out = ops.causal_dot_product_fwd(
            q, k, v, s_init=None if s_init is None else s_init.view(B * H, dk, dv),
            s_final=s_final.view(B * H, dk, dv))
        ctx.save_for_backward(q, k, v, s_init, s_final)
        return out, s_final

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx: Any, grad_output, grad_s_final):
        q, k, v, s_init, s_final = ctx.saved_tensors
        B, H, _, dk = q.shape
        dv = v.shape[-1]
        flat = (B * H, dk, dv)
        if grad_output is None:
            grad_output = torch.zeros_like(v)
        r_init = None if grad_s_final is None else grad_s_final.to(torch.float32).contiguous().view(flat)
        r_final = torch.empty(flat, dtype=torch.float32, device=q.device) if ctx.needs_input_grad[3] else None
        s_last = s_final.view(flat) if ops.backward_uses_final_state(q, v) else None
        dq, dk_, dv_ = ops.causal_dot_product_bwd(
            grad_output.contiguous(), q, k, v,
            s_init=None if s_init is None else s_init.view(flat),
            r_init=r_init, r_final=r_final, s_last=s_last)
        return dq, dk_, dv_, None if r_final is None else r_final.view(B, H, dk, dv)


class LinearAttentionNormalized(Function):
    """Causal linear attention WITH its denominator:
    ``out_i = sum_{j<=i} (q_i . k_j) v_j / (q_i . sum_{j<=i} k_j + eps)``, i.e. the whole recipe of
    the reference's README (README.md:27-30) in one Function. The product runs in the same kernels
    as LinearAttention / LinearAttentionSmallVHD; the denominator, the division and their
    gradients run in three streaming kernels with an fp32 running sum instead of PyTorch's
    cumsum / multiply / sum / divide passes. ``apply(q, k, v, eps=1e-5)``; dv a multiple of 8.
    """

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx: Any, q, k, v, eps: float = 1e-5):
        ops.check_forward_preconditions(q, v, smallv=q.shape[-1] != v.shape[-1])
        if v.shape[-1] % 8 != 0:
            raise NotImplementedError("LinearAttentionNormalized needs a value head dim that is a multiple of 8")
        q, k = ops.kernel_view(q), ops.kernel_view(k)  # repacked once if the rows are not 16-byte multiples
        B, H, _, dk = q.shape
        need_grad = any(ctx.needs_input_grad[:3])
        s_final = None
        if need_grad and ops.backward_uses_final_state(q, v):
            s_final = torch.empty(B * H, dk, v.shape[-1], dtype=torch.float32, device=q.device)
        out = ops.causal_dot_product_fwd(q, k, v, s_final=s_final)
        if not out.is_contiguous():
            out = out.contiguous()
        den = ops.normalize_fwd(q, k, out, eps)
        ctx.has_state = s_final is not None
        if ctx.has_state:
            ctx.save_for_backward(q, k, v, out, den, s_final)
        else:
            ctx.save_for_backward(q, k, v, out, den)
        return out

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx: Any, grad_output):
        q, k, v, out, den = ctx.saved_tensors[:5]
        s_final = ctx.saved_tensors[5] if ctx.has_state else None
        dnum, dden = ops.normalize_bwd_prepare(grad_output, out, den)
        dq, dk, dv = ops.causal_dot_product_bwd(dnum, q, k, v, s_last=s_final, keep_padded=True)
        ops.normalize_bwd_sweep(q, k, dq, dk, dden)
        return dq, dk, dv, None


class TaylorLinearAttention(Function):
    """Causal linear attention on second-order Taylor features of RAW q, k:
    ``apply(xq, xk, v)`` with xq, xk ``[B, H, N, d]`` (d = 8 or 16) and v ``[B, H, N, dv]`` (dv <= 64)
    returns ``sum_{j<=i} (phi(xq_i) . phi(xk_j)) v_j`` with ``phi(x) = [1, x / d^(1/4),
    vec(x x^T) / (sqrt(2) sqrt(d))]`` (benchmark configuration 4: d = 16 -> 273 features), and its
    backward returns gradients with respect to the raw xq, xk and v.

    The feature map runs in its own kernels and writes rows the attention kernels read in place,
    so the pad passes of ``LinearAttentionSmallVHD`` on contiguous 273-wide tensors disappear and the
    273-wide tensors never have to exist on the caller's side. The reference has no counterpart.
    """

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
    def forward(ctx: Any, xq, xk, v):
        pq, pk = ops.taylor_features(xq), ops.taylor_features(xk)
        ops.check_forward_preconditions(pq, v, smallv=True)
        out = ops.causal_dot_product_fwd(pq, pk, v)
        ctx.save_for_backward(xq, xk, v, pq, pk)
        return out

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx: Any, grad_output):
        xq, xk, v, pq, pk = ctx.saved_tensors
        dpq, dpk, dv = ops.causal_dot_product_bwd(grad_output, pq, pk, v, keep_padded=True)
        return ops.taylor_features_bwd(dpq, xq), ops.taylor_features_bwd(dpk, xk), dv
