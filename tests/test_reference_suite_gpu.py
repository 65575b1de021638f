"""The reference's own eight acceptance tests (flashlinear/test_attn.py:65-176 and
flashlinear/test_attn_smallv_hd.py:69-184), restated against this library's `flashlinear` API:
same input recipe (softplus q, k; q / sqrt(hd); dy = 0.1 randn resp. randn), same shape ranges
drawn from a seeded numpy RNG, same expected value (the naive PyTorch path evaluated in bf16 on the
GPU) and the same bound: Frobenius relative error < 1e-2."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

NUM_TEST = 3
BFLOAT16_MAX_TOL = 1e-2
DEV = "cuda:0"
_rng = np.random.RandomState(0)


def rel_error(x, y):
    return torch.linalg.norm(x.float() - y.float()) / torch.linalg.norm(y.float())


def make_input_qkv(bs, nh, sq, hd_qk, hd_v=None):
    hd_v = hd_qk if hd_v is None else hd_v
    q = torch.randn((bs, nh, sq, hd_qk), device=DEV, dtype=torch.bfloat16)
    k = torch.randn((bs, nh, sq, hd_qk), device=DEV, dtype=torch.bfloat16)
    v = torch.randn((bs, nh, sq, hd_v), device=DEV, dtype=torch.bfloat16)
    q = torch.nn.functional.softplus(q)
    k = torch.nn.functional.softplus(k)
    q *= 1.0 / math.sqrt(hd_qk)
    for t in (q, k, v):
        t.requires_grad_(True)
    return q, k, v


def naive_causal_product(q, k, v):
    """(q k^T * tril) v in the dtype of the inputs (the reference tests' expected value)."""
    scores = torch.matmul(q, k.transpose(-2, -1))
    n = q.size(-2)
    scores = scores * torch.ones(1, 1, n, n, dtype=torch.bool, device=q.device).tril(diagonal=0)
    return torch.matmul(scores, v)


def _dims_equal(standard):
    hd = (lambda: _rng.choice([32, 64, 128], size=NUM_TEST, replace=True)) if standard else (lambda: _rng.randint(16, 128, size=NUM_TEST))
    return [
        (int(b), int(nh), int(sq), int(h))
        for b in _rng.randint(1, 4, size=NUM_TEST)
        for nh in _rng.randint(1, 32, size=NUM_TEST)
        for sq in 64 * _rng.randint(1, 32, size=NUM_TEST)
        for h in hd()
    ]


def _dims_smallv(standard):
    hd = (lambda: _rng.choice([32, 64, 128], size=NUM_TEST, replace=True)) if standard else (lambda: _rng.randint(32, 128, size=NUM_TEST))
    return [
        (int(b), int(nh), int(sq), int(hqk), int(hv))
        for b in _rng.randint(1, 4, size=NUM_TEST)
        for nh in _rng.randint(1, 32, size=NUM_TEST)
        for sq in 64 * _rng.randint(1, 32, size=NUM_TEST)
        for hqk in hd()
        for hv in _rng.choice([16, 32], size=NUM_TEST, replace=True)
    ]


def _fwd_case(fn, dims):
    q, k, v = make_input_qkv(*dims)
    with torch.no_grad():
        ref_out = naive_causal_product(q, k, v)
        out = fn.apply(q, k, v)
    assert out.shape == ref_out.shape and out.dtype == torch.bfloat16
    assert rel_error(out, ref_out) < BFLOAT16_MAX_TOL


def _bwd_case(fn, dims, dy_scale):
    q, k, v = make_input_qkv(*dims)
    ref_out = naive_causal_product(q, k, v)
    dy = dy_scale * torch.randn_like(ref_out)
    ref_out.backward(dy, retain_graph=True)
    dQ_t, dK_t, dV_t = [t.grad.clone() for t in (q, k, v)]
    q.grad, k.grad, v.grad = None, None, None
    out = fn.apply(q, k, v)
    out.backward(dy, retain_graph=True)
    assert rel_error(q.grad, dQ_t) < BFLOAT16_MAX_TOL
    assert rel_error(k.grad, dK_t) < BFLOAT16_MAX_TOL
    assert rel_error(v.grad, dV_t) < BFLOAT16_MAX_TOL


@pytest.mark.parametrize("dims", _dims_equal(True))
def test_attn_fwd(dims):
    from flashlinear import LinearAttention
    _fwd_case(LinearAttention, dims)


@pytest.mark.parametrize("dims", _dims_equal(True))
def test_attn_bwd(dims):
    from flashlinear import LinearAttention
    _bwd_case(LinearAttention, dims, 0.1)


@pytest.mark.parametrize("dims", _dims_equal(False))
def test_attn_fwd_masked_hd(dims):
    from flashlinear import LinearAttention
    _fwd_case(LinearAttention, dims)


@pytest.mark.parametrize("dims", _dims_equal(False))
def test_attn_bwd_masked_hd(dims):
    from flashlinear import LinearAttention
    _bwd_case(LinearAttention, dims, 0.1)


@pytest.mark.parametrize("dims", _dims_smallv(True))
def test_smallv_attn_fwd(dims):
    from flashlinear import LinearAttentionSmallVHD
    _fwd_case(LinearAttentionSmallVHD, dims)


@pytest.mark.parametrize("dims", _dims_smallv(True))
def test_smallv_attn_bwd(dims):
    from flashlinear import LinearAttentionSmallVHD
    _bwd_case(LinearAttentionSmallVHD, dims, 1.0)


@pytest.mark.parametrize("dims", _dims_smallv(False))
def test_smallv_attn_fwd_masked_hd(dims):
    from flashlinear import LinearAttentionSmallVHD
    _fwd_case(LinearAttentionSmallVHD, dims)


@pytest.mark.parametrize("dims", _dims_smallv(False))
def test_smallv_attn_bwd_masked_hd(dims):
    from flashlinear import LinearAttentionSmallVHD
    _bwd_case(LinearAttentionSmallVHD, dims, 1.0)
