"""Parity at the benchmark's full sizes: whole heads against the naive path.

The reference's naive path (flashlinear/test_attn.py:49-62) needs an N x N score matrix per head;
oracle.torch_naive.naive_rows_blocked evaluates the same sums in blocks of query rows, in float64
on the GPU, so that heads of 8192, 2048 and 65536 tokens can be checked in full. Inputs are the
benchmark's seeded distributions. Tolerances as everywhere: max-rel <= 2e-2, Frobenius < 1e-2.
"""
import pytest
import torch

from oracle import torch_naive

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
MAX_REL_TOL = 2e-2
FROB_TOL = 1e-2


def _elu1(shape, gen):
    return (torch.nn.functional.elu(torch.randn(shape, device=DEV, generator=gen)) + 1).to(torch.bfloat16)


def _normal(shape, gen):
    return torch.randn(shape, device=DEV, generator=gen).to(torch.bfloat16)


def _taylor(x):
    """[1, x / d^(1/4), vec(x x^T) / (sqrt(2) sqrt(d))], the feature map of configuration 4, fp32."""
    d = x.shape[-1]
    quad = (x.unsqueeze(-1) * x.unsqueeze(-2)).flatten(-2) / (2.0 ** 0.5 * d ** 0.5)
    return torch.cat([torch.ones_like(x[..., :1]), x / d ** 0.25, quad], dim=-1)


def _check_heads(heads, q, k, v, dy, got, block=2048):
    """got = (out, dq, dk, dv) of the library; every listed (b, h) head against the oracle."""
    for b, h in heads:
        want = torch_naive.naive_rows_blocked(*(t[b, h].double() for t in (q, k, v, dy)), block=block)
        for name, g, w in zip(("out", "dq", "dk", "dv"), got, want):
            g = g[b, h].double()
            max_rel = ((g - w).abs().max() / w.abs().max()).item()
            frob = (torch.linalg.norm(g - w) / torch.linalg.norm(w)).item()
            assert max_rel <= MAX_REL_TOL and frob < FROB_TOL, \
                f"{name}[{b},{h}]: max-rel {max_rel:.3e}, frobenius {frob:.3e}"


def _three_heads(B, H):
    return [(0, 0), (B // 2, H // 2), (B - 1, H - 1)]


def test_configuration_3_three_heads_through_the_function():
    """B4 H32 N8192 D128 through LinearAttention.apply + autograd: first, middle and last head."""
    from flashlinear import LinearAttention

    B, H, N, D = 4, 32, 8192, 128
    gen = torch.Generator(device=DEV).manual_seed(3)
    q, k = _elu1((B, H, N, D), gen).requires_grad_(True), _elu1((B, H, N, D), gen).requires_grad_(True)
    v, dy = _normal((B, H, N, D), gen).requires_grad_(True), _normal((B, H, N, D), gen)
    out = LinearAttention.apply(q, k, v)
    grads = torch.autograd.grad(out, (q, k, v), dy)
    _check_heads(_three_heads(B, H), q.detach(), k.detach(), v.detach(), dy, (out.detach(),) + grads)


def test_configuration_4_full_size_smallv_function():
    """B8 H16 N2048, 273 Taylor features of 16 raw dims, dv 64, through LinearAttentionSmallVHD.apply
    on contiguous 273-wide tensors (the layout a caller of the reference would hold)."""
    from flashlinear import LinearAttentionSmallVHD

    B, H, N, dv = 8, 16, 2048, 64
    gen = torch.Generator(device=DEV).manual_seed(4)
    q = _taylor(torch.randn(B, H, N, 16, device=DEV, generator=gen)).to(torch.bfloat16).requires_grad_(True)
    k = _taylor(torch.randn(B, H, N, 16, device=DEV, generator=gen)).to(torch.bfloat16).requires_grad_(True)
    v, dy = _normal((B, H, N, dv), gen).requires_grad_(True), _normal((B, H, N, dv), gen)
    assert q.shape[-1] == 273 and q.is_contiguous()
    out = LinearAttentionSmallVHD.apply(q, k, v)
    grads = torch.autograd.grad(out, (q, k, v), dy)
    assert tuple(grads[0].shape) == (B, H, N, 273) and tuple(grads[2].shape) == (B, H, N, dv)
    _check_heads(_three_heads(B, H), q.detach(), k.detach(), v.detach(), dy, (out.detach(),) + grads)


def test_configuration_4_full_size_from_raw_inputs():
    """The same shape through TaylorLinearAttention.apply on the RAW 16-dim q, k: output and the
    gradients with respect to the raw inputs, against autograd through the fp64 feature map and the
    naive path."""
    from flashy_linear_attention_b200.functions import TaylorLinearAttention

    B, H, N, dv = 8, 16, 2048, 64
    gen = torch.Generator(device=DEV).manual_seed(5)
    xq, xk = _normal((B, H, N, 16), gen).requires_grad_(True), _normal((B, H, N, 16), gen).requires_grad_(True)
    v, dy = _normal((B, H, N, dv), gen).requires_grad_(True), _normal((B, H, N, dv), gen)
    out = TaylorLinearAttention.apply(xq, xk, v)
    gxq, gxk, gv = torch.autograd.grad(out, (xq, xk, v), dy)
    for b, h in _three_heads(B, H):
        rq = xq[b, h].detach().double().requires_grad_(True)
        rk = xk[b, h].detach().double().requires_grad_(True)
        rv = v[b, h].detach().double().requires_grad_(True)
        # the kernels consume bf16 features: round them the same way, with a straight-through gradient
        fq, fk = _taylor(rq), _taylor(rk)
        fq = fq + (fq.detach().to(torch.bfloat16).double() - fq.detach())
        fk = fk + (fk.detach().to(torch.bfloat16).double() - fk.detach())
        want = torch_naive.naive_rows_blocked(fq, fk, rv)
        wq, wk, wv = torch.autograd.grad(want, (rq, rk, rv), dy[b, h].double())
        for name, g, w in (("out", out[b, h], want.detach()), ("dxq", gxq[b, h], wq), ("dxk", gxk[b, h], wk),
                           ("dv", gv[b, h], wv)):
            g = g.detach().double()
            max_rel = ((g - w).abs().max() / w.abs().max()).item()
            frob = (torch.linalg.norm(g - w) / torch.linalg.norm(w)).item()
            assert max_rel <= MAX_REL_TOL and frob < FROB_TOL, f"{name}[{b},{h}]: {max_rel:.3e} {frob:.3e}"


def test_configuration_5_full_length_on_one_gpu():
    """B1 H32 N65536 D128 on one GPU: two whole heads against the row-blocked oracle, and the
    single-sweep backward (dQ as total-minus-suffix, where fp32 states of size ~sqrt(N) are
    subtracted) against the two-direction backward."""
    from flashy_linear_attention_b200 import ops

    B, H, N, D = 1, 32, 65536, 128
    gen = torch.Generator(device=DEV).manual_seed(6)
    q, k = _elu1((B, H, N, D), gen), _elu1((B, H, N, D), gen)
    v, dy = _normal((B, H, N, D), gen), _normal((B, H, N, D), gen)
    s_state = torch.empty(B * H, D, D, dtype=torch.float32, device=DEV)
    out = ops.causal_dot_product_fwd(q, k, v, s_final=s_state)
    # segments=1 keeps the backward unsegmented, the form that uses the forward's final state
    dq, dk, dv = ops.causal_dot_product_bwd(dy, q, k, v, s_last=s_state, segments=1)
    dq2, dk2, dv2 = ops.causal_dot_product_bwd(dy, q, k, v, segments=1)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    rel = (torch.linalg.norm(dq.float() - dq2.float()) / torch.linalg.norm(dq2.float())).item()
    assert rel < FROB_TOL, rel
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2)
    heads = [(0, 0), (0, H - 1)]
    _check_heads(heads, q, k, v, dy, (out, dq, dk, dv), block=4096)
    _check_heads(heads[:1], q, k, v, dy, (out, dq2, dk2, dv2), block=4096)
    # the default call (automatic segments) as well
    dq3, dk3, dv3 = ops.causal_dot_product_bwd(dy, q, k, v, s_last=s_state)
    _check_heads(heads[1:], q, k, v, dy, (out, dq3, dk3, dv3), block=4096)
