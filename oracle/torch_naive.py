"""The reference's naive PyTorch path restated with torch ops, for CPU timing and GPU-side checks
-- TEST / BENCHMARK INFRASTRUCTURE, not a product path (the library never imports it).

Follows flashlinear/test_attn.py:49-62 (`linear_ref_torch`: q k^T, multiply by a lower-triangular
boolean mask, times v) and README.md:27-30 (denominator with eps = 1e-5); gradients come from
autograd as in flashlinear/test_attn.py:107-111. Pinned against the reference's own outputs in
tests/test_oracle.py::test_torch_naive_matches_reference_fixture.
"""
from __future__ import annotations

import time

import torch


def naive_causal_product(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    scores = torch.matmul(q, k.transpose(-2, -1))
    n_q, n_k = q.size(-2), k.size(-2)
    mask = torch.ones(1, 1, n_q, n_k, dtype=torch.bool, device=q.device).tril(diagonal=0)
    scores = scores * mask
    return torch.matmul(scores, v)


def naive_linear_attention(q, k, v, eps: float = 1e-5, normalise: bool = True):
    out = naive_causal_product(q, k, v)
    if not normalise:
        return out
    denom = (q * k.cumsum(-2)).sum(dim=-1, keepdim=True) + eps
    return out / denom


def naive_rows_blocked(q, k, v, dy=None, block: int = 2048):
    """The same naive path for ONE head ([N, d] tensors), evaluated in blocks of query rows so that
    the N x N score matrix (flashlinear/test_attn.py:52) never exists as a whole: rows r0..r1 only
    meet keys 0..r1, exactly what the lower-triangular mask (:54-60) keeps. Returns out, or
    (out, dq, dk, dv) when `dy` is given: the closed form of what autograd returns for
    sum(out * dy) (flashlinear/test_attn.py:107-111). Runs in the dtype and on the device of its
    inputs (float64 for parity checks of long sequences)."""
    n = q.shape[0]
    out = torch.empty(n, v.shape[1], dtype=q.dtype, device=q.device)
    if dy is not None:
        dq = torch.empty_like(q)
        dk = torch.zeros_like(k)
        dv = torch.zeros_like(v)
    for r0 in range(0, n, block):
        r1 = min(n, r0 + block)
        rows = torch.arange(r0, r1, device=q.device).unsqueeze(1)
        cols = torch.arange(0, r1, device=q.device).unsqueeze(0)
        mask = cols <= rows
        p = (q[r0:r1] @ k[:r1].T) * mask
        out[r0:r1] = p @ v[:r1]
        if dy is not None:
            dp = (dy[r0:r1] @ v[:r1].T) * mask
            dq[r0:r1] = dp @ k[:r1]
            dk[:r1] += dp.T @ q[r0:r1]
            dv[:r1] += p.T @ dy[r0:r1]
    if dy is None:
        return out
    return out, dq, dk, dv


def time_fwd_bwd_cpu(batch, heads, seqlen, dk, dv, steps=1, warmup=0, threads=None, seed=0, normalise=False):
    """Times forward + autograd backward of the naive path in fp32 on the host cores.
    Returns (seconds per step, threads used)."""
    if threads:
        torch.set_num_threads(int(threads))
    gen = torch.Generator().manual_seed(seed)
    q = (torch.nn.functional.elu(torch.randn(batch, heads, seqlen, dk, generator=gen)) + 1).requires_grad_(True)
    k = (torch.nn.functional.elu(torch.randn(batch, heads, seqlen, dk, generator=gen)) + 1).requires_grad_(True)
    v = torch.randn(batch, heads, seqlen, dv, generator=gen).requires_grad_(True)
    dy = torch.randn(batch, heads, seqlen, dv, generator=gen)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        out = naive_linear_attention(q, k, v, normalise=normalise)
        torch.autograd.grad(out, (q, k, v), dy)
        t1 = time.perf_counter()
        if it >= warmup:
            times.append(t1 - t0)
    return sum(times) / len(times), torch.get_num_threads()
