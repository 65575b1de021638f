"""float16 inputs. The reference is bf16-only in practice (its kernels cast the score tile with
tl.bfloat16, flashlinear/kernels/linear_attn_kernels.py:82,187,197,299); here the same kernels run
with fp16 tensor-core operands and fp16 outputs when every tensor of a call is float16 and the head
dims are at most 128. Oracle: the naive path in float64 on the fp16-rounded inputs; same bounds as
for bf16 (fp16 has three more mantissa bits, so they are met with room to spare)."""
import numpy as np
import pytest
import torch

from oracle import linear_attention_oracle as orc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
MAX_REL_TOL = 2e-2
FROB_TOL = 1e-2


def _inputs(shape, seed):
    B, H, N, dk, dv = shape
    rng = np.random.default_rng(seed)
    q = orc.elu_plus_one(rng.standard_normal((B, H, N, dk))).astype(np.float16)
    k = orc.elu_plus_one(rng.standard_normal((B, H, N, dk))).astype(np.float16)
    v = rng.standard_normal((B, H, N, dv)).astype(np.float16)
    dy = rng.standard_normal((B, H, N, dv)).astype(np.float16)
    return q, k, v, dy


def _check(name, got, want):
    g = got.detach().float().cpu().numpy()
    mr, fr = orc.max_rel_error(g, want), orc.frobenius_rel_error(g, want)
    assert mr <= MAX_REL_TOL and fr < FROB_TOL, f"{name}: max-rel {mr:.3e}, frobenius {fr:.3e}"


@pytest.mark.parametrize("shape", [(2, 3, 512, 64, 64), (1, 2, 1024, 128, 128), (1, 2, 320, 96, 32), (1, 1, 200, 40, 40),
                                   (1, 4, 4096, 128, 128)],
                         ids=lambda s: "x".join(map(str, s)))
def test_fp16_forward_and_backward_against_oracle(shape):
    from flashy_linear_attention_b200 import ops

    q, k, v, dy = _inputs(shape, seed=sum(shape))
    tq, tk, tv, tdy = (torch.from_numpy(t).to(DEV) for t in (q, k, v, dy))
    out = ops.causal_dot_product_fwd(tq, tk, tv)
    dq, dk_, dv_ = ops.causal_dot_product_bwd(tdy, tq, tk, tv)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert out.dtype == torch.float16 and dq.dtype == torch.float16
    q64, k64, v64, dy64 = (t.astype(np.float64) for t in (q, k, v, dy))
    if shape[2] > 2048:  # one head is enough at this length
        q64, k64, v64, dy64 = (t[:, -1:] for t in (q64, k64, v64, dy64))
        out, dq, dk_, dv_ = (t[:, -1:] for t in (out, dq, dk_, dv_))
    _check("out", out, orc.linear_ref(q64, k64, v64))
    rq, rk, rv = orc.linear_ref_grads(q64, k64, v64, dy64)
    _check("dq", dq, rq)
    _check("dk", dk_, rk)
    _check("dv", dv_, rv)


def test_fp16_through_the_function_and_dtype_rules():
    from flashlinear import LinearAttention
    from flashy_linear_attention_b200 import ops

    q, k, v, dy = _inputs((1, 2, 384, 64, 64), seed=3)
    tq, tk, tv = (torch.from_numpy(t).to(DEV).requires_grad_(True) for t in (q, k, v))
    out = LinearAttention.apply(tq, tk, tv)          # no autocast: fp16 stays fp16
    assert out.dtype == torch.float16
    out.backward(torch.from_numpy(dy).to(DEV))
    torch.cuda.synchronize()
    ops.check_status(DEV)
    rq, rk, rv = orc.linear_ref_grads(*(t.astype(np.float64) for t in (q, k, v, dy)))
    _check("dq", tq.grad, rq)
    _check("dk", tk.grad, rk)
    _check("dv", tv.grad, rv)
    with pytest.raises(TypeError):                   # mixed 16-bit types are refused
        ops.causal_dot_product_fwd(tq.detach(), tk.detach().to(torch.bfloat16), tv.detach())
    wide = torch.zeros(1, 1, 128, 256, dtype=torch.float16, device=DEV)
    with pytest.raises(TypeError):                   # head dims above 128 are bf16 only
        ops.causal_dot_product_fwd(wide, wide, wide)
