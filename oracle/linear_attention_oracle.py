"""CPU oracle for causal linear attention -- TEST INFRASTRUCTURE, not a product path.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference legs may import this
module; the library itself never does (it has no CPU fallback).

Parity pin: every function here is checked in tests/test_oracle.py against fixtures under
tests/golden/ that were produced by importing and running the reference's own naive PyTorch path
(`linear_ref_torch`, flashlinear/test_attn.py:49-62, gradients by autograd as in :107-111) with
tests/golden/make_golden.py.

Restated reference behaviour (numpy, any float dtype):
  linear_ref            flashlinear/test_attn.py:49-62       out = ((q k^T) * tril) v
  linear_ref_grads      flashlinear/test_attn.py:107-111     autograd of the above, in closed form
  denominator           README.md:27-30                      (q * cumsum(k)).sum(-1) + eps
  normalised_ref        README.md:27-30                      out / denominator
  bf16_round            flashlinear/kernels/linear_attn_kernels.py:82,98   P and outputs go to bf16
  kernel_numerics_*     flashlinear/kernels/linear_attn_kernels.py:74-82,179-197,291-299
                        the Triton kernels' rounding points: fp32 scores -> mask -> bf16 -> fp32
                        second product -> bf16 output
  chunked_fwd / chunked_bwd   the chunk + running-state formulation the CUDA kernels use; the same
                        sums as linear_ref in another order (no counterpart in the reference)
  taylor_feature_map    no counterpart in the reference (README.md:3 links a description only):
                        x in R^16 -> [1, x / 16^(1/4), vec(x x^T) / (sqrt(2) * sqrt(16))] in R^273
"""
from __future__ import annotations

import numpy as np


# ------------------------------------------------------------------------------------------------
# bf16 emulation (numpy has no bfloat16)
# ------------------------------------------------------------------------------------------------
def bf16_round(x: np.ndarray) -> np.ndarray:
    """Rounds float32 values to the nearest bfloat16 (ties to even) and returns them as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = rounded.view(np.float32).copy()
    nan = np.isnan(x)
    if nan.any():
        out[nan] = np.nan
    return out.reshape(x.shape)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns (uint16) of float32 values that are exactly representable."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    return (x.view(np.uint32) >> 16).astype(np.uint16).reshape(x.shape)


def bf16_from_bits(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32).reshape(b.shape)


# ------------------------------------------------------------------------------------------------
# The reference's naive path (flashlinear/test_attn.py:49-62)
# ------------------------------------------------------------------------------------------------
def _tril(n: int, dtype) -> np.ndarray:
    return np.tril(np.ones((n, n), dtype=dtype))


def linear_ref(q: np.ndarray, k: np.ndarray, v: np.ndarray) -> np.ndarray:
    """out = ((q k^T) * lower-triangular mask incl. diagonal) v, shapes [..., N, d]."""
    scores = np.matmul(q, np.swapaxes(k, -1, -2))
    scores = scores * _tril(q.shape[-2], scores.dtype)
    return np.matmul(scores, v)


def linear_ref_grads(q, k, v, dy):
    """(dq, dk, dv) of sum(linear_ref(q,k,v) * dy): what autograd returns in test_attn.py:107-111."""
    mask = _tril(q.shape[-2], q.dtype)
    p = np.matmul(q, np.swapaxes(k, -1, -2)) * mask      # masked scores
    dp = np.matmul(dy, np.swapaxes(v, -1, -2)) * mask    # gradient w.r.t. the scores, masked
    dq = np.matmul(dp, k)
    dk = np.matmul(np.swapaxes(dp, -1, -2), q)
    dv = np.matmul(np.swapaxes(p, -1, -2), dy)
    return dq, dk, dv


def denominator(q: np.ndarray, k: np.ndarray, eps: float = 1e-5) -> np.ndarray:
    """README.md:29: (q * k.cumsum(-2)).sum(-1, keepdim=True) + eps."""
    return (q * np.cumsum(k, axis=-2)).sum(axis=-1, keepdims=True) + eps


def normalised_ref(q, k, v, eps: float = 1e-5):
    """README.md:27-30: unnormalised product divided by the denominator."""
    return linear_ref(q, k, v) / denominator(q, k, eps)


def normalised_ref_grads(q, k, v, dy, eps: float = 1e-5):
    """Gradients of sum(normalised_ref * dy) w.r.t. q, k, v (closed form of README.md:27-30)."""
    num = linear_ref(q, k, v)
    den = denominator(q, k, eps)
    dnum = dy / den
    dden = -(dy * num).sum(axis=-1, keepdims=True) / (den * den)
    dq, dk, dv = linear_ref_grads(q, k, v, dnum)
    kc = np.cumsum(k, axis=-2)
    dq = dq + dden * kc
    # d/dk of sum_i dden_i * sum_d q_id * sum_{j<=i} k_jd  ->  reverse cumulative sum over i
    w = dden * q
    dk = dk + np.flip(np.cumsum(np.flip(w, axis=-2), axis=-2), axis=-2)
    return dq, dk, dv


# ------------------------------------------------------------------------------------------------
# The Triton kernels' rounding points (inputs are bf16 values held in float32)
# ------------------------------------------------------------------------------------------------
def kernel_numerics_fwd(q, k, v):
    """fp32 scores -> mask -> bf16 -> fp32 product -> bf16 (linear_attn_kernels.py:74-82,96-100)."""
    q, k, v = (np.asarray(t, dtype=np.float32) for t in (q, k, v))
    p = np.matmul(q, np.swapaxes(k, -1, -2)) * _tril(q.shape[-2], np.float32)
    return bf16_round(np.matmul(bf16_round(p), v))


def kernel_numerics_bwd(q, k, v, dy):
    """Rounding points of flash_attn_bwd (linear_attn_kernels.py:179-197, 291-299, 220-227, 304-307)."""
    q, k, v, dy = (np.asarray(t, dtype=np.float32) for t in (q, k, v, dy))
    mask = _tril(q.shape[-2], np.float32)
    p = bf16_round(np.matmul(q, np.swapaxes(k, -1, -2)) * mask)
    dp = bf16_round(np.matmul(dy, np.swapaxes(v, -1, -2)) * mask)
    dq = bf16_round(np.matmul(dp, k))
    dk = bf16_round(np.matmul(np.swapaxes(dp, -1, -2), q))
    dv = bf16_round(np.matmul(np.swapaxes(p, -1, -2), dy))
    return dq, dk, dv


# ------------------------------------------------------------------------------------------------
# Chunked formulation with a running state (what the CUDA kernels compute)
# ------------------------------------------------------------------------------------------------
def causal_product_chunked(a, b, c, chunk=128, reverse=False, s_init=None, emulate_bf16=False):
    """out_i = sum_{j<=i} (a_i . b_j) c_j (reverse: j>=i), one chunk at a time:
        P = (A B^T) * mask ; O = P C + A S ; S += B^T C
    With emulate_bf16 the rounding points of the CUDA kernel are applied (P and S to bf16 as MMA
    operands, fp32 accumulation, bf16 output). Returns (out, final state)."""
    a, b, c = (np.asarray(t) for t in (a, b, c))
    dt = np.float32 if emulate_bf16 else np.result_type(a.dtype, np.float32)
    a, b, c = a.astype(dt), b.astype(dt), c.astype(dt)
    lead = a.shape[:-2]
    n, da = a.shape[-2:]
    dc = c.shape[-1]
    out = np.zeros(lead + (n, dc), dtype=dt)
    s = np.zeros(lead + (da, dc), dtype=dt) if s_init is None else np.array(s_init, dtype=dt).reshape(lead + (da, dc))
    nchunks = (n + chunk - 1) // chunk
    order = range(nchunks - 1, -1, -1) if reverse else range(nchunks)
    for ci in order:
        lo, hi = ci * chunk, min((ci + 1) * chunk, n)
        ac, bc, cc = a[..., lo:hi, :], b[..., lo:hi, :], c[..., lo:hi, :]
        m = hi - lo
        mask = np.triu(np.ones((m, m), dtype=dt)) if reverse else np.tril(np.ones((m, m), dtype=dt))
        p = np.matmul(ac, np.swapaxes(bc, -1, -2)) * mask
        sb = s
        if emulate_bf16:
            p = bf16_round(p)
            sb = bf16_round(s)
        o = np.matmul(p, cc) + np.matmul(ac, sb)
        out[..., lo:hi, :] = bf16_round(o) if emulate_bf16 else o
        s = s + np.matmul(np.swapaxes(bc, -1, -2), cc)
    return out, s


def causal_product_total_minus_suffix(a, b, c, total, chunk=128, first_chunk_exact=True, emulate_bf16=False):
    """The causal sum out_i = sum_{j<=i} (a_i . b_j) c_j walked from the LAST chunk to the first,
    as the CUDA kernels do for dQ when the forward's final state is known: the state starts as
    `total` = sum over all tokens of b^T c, a chunk uses it while it still contains the chunk's own
    tokens and corrects with the strictly upper part of its score tile,
        O = A S_incl - (strict_upper(A B^T)) C ;  S_incl -= B^T C,
    except for the chunk that starts the sequence (first_chunk_exact), which has no prefix and is
    computed from its lower-masked score tile alone."""
    a, b, c = (np.asarray(t) for t in (a, b, c))
    dt = np.float32 if emulate_bf16 else np.result_type(a.dtype, np.float32)
    a, b, c = a.astype(dt), b.astype(dt), c.astype(dt)
    n = a.shape[-2]
    out = np.zeros(a.shape[:-1] + (c.shape[-1],), dtype=dt)
    s = np.array(total, dtype=dt).reshape(a.shape[:-2] + (a.shape[-1], c.shape[-1]))
    rnd = bf16_round if emulate_bf16 else (lambda x: x)
    for ci in range((n + chunk - 1) // chunk - 1, -1, -1):
        lo, hi = ci * chunk, min((ci + 1) * chunk, n)
        ac, bc, cc = a[..., lo:hi, :], b[..., lo:hi, :], c[..., lo:hi, :]
        m = hi - lo
        scores = np.matmul(ac, np.swapaxes(bc, -1, -2))
        if ci == 0 and first_chunk_exact:
            o = np.matmul(rnd(scores * np.tril(np.ones((m, m), dtype=dt))), cc)
        else:
            o = np.matmul(rnd(-scores * np.triu(np.ones((m, m), dtype=dt), 1)), cc) + np.matmul(ac, rnd(s))
        out[..., lo:hi, :] = rnd(o)
        s = s - np.matmul(np.swapaxes(bc, -1, -2), cc)
    return out


def chunked_fwd(q, k, v, chunk=128, s_init=None, emulate_bf16=False):
    """Forward: (out, S_final) with S = sum k^T v."""
    return causal_product_chunked(q, k, v, chunk, False, s_init, emulate_bf16)


def chunked_bwd(q, k, v, dy, chunk=128, s_init=None, r_init=None, emulate_bf16=False):
    """Backward as three products with permuted operands:
        dQ_i = sum_{j<=i} (dO_i . v_j) k_j   (state S^T = sum v^T k)
        dV_j = sum_{i>=j} (k_j . q_i) dO_i   (state R   = sum q^T dO)
        dK_j = sum_{i>=j} (v_j . dO_i) q_i   (state R^T)
    Returns (dq, dk, dv, R_final)."""
    st = None if s_init is None else np.swapaxes(np.asarray(s_init), -1, -2)
    rt = None if r_init is None else np.swapaxes(np.asarray(r_init), -1, -2)
    dq, _ = causal_product_chunked(dy, v, k, chunk, False, st, emulate_bf16)
    dv, r_final = causal_product_chunked(k, q, dy, chunk, True, r_init, emulate_bf16)
    dk, _ = causal_product_chunked(v, dy, q, chunk, True, rt, emulate_bf16)
    return dq, dk, dv, r_final


# ------------------------------------------------------------------------------------------------
# Inputs of the benchmark configurations
# ------------------------------------------------------------------------------------------------
def elu_plus_one(x: np.ndarray) -> np.ndarray:
    return np.where(x > 0, x + 1.0, np.exp(np.minimum(x, 0.0))).astype(x.dtype)


def taylor_feature_map(x: np.ndarray) -> np.ndarray:
    """2nd-order Taylor features of raw x[..., d]: [1, x / d^(1/4), vec(x x^T) / (sqrt(2) sqrt(d))],
    so that phi(q) . phi(k) = 1 + s + s^2 / 2 with s = q . k / sqrt(d). d = 16 gives 273 features."""
    d = x.shape[-1]
    one = np.ones(x.shape[:-1] + (1,), dtype=x.dtype)
    lin = x / (d ** 0.25)
    quad = (x[..., :, None] * x[..., None, :]).reshape(x.shape[:-1] + (d * d,)) / (np.sqrt(2.0) * np.sqrt(d))
    return np.concatenate([one, lin, quad.astype(x.dtype)], axis=-1)


def taylor_feature_map_grad(x: np.ndarray, dphi: np.ndarray) -> np.ndarray:
    """Gradient of sum(taylor_feature_map(x) * dphi) with respect to x (closed form):
    dx_a = dphi_lin[a] / d^(1/4) + sum_b (dPhi[a, b] + dPhi[b, a]) x_b / (sqrt(2) sqrt(d))."""
    d = x.shape[-1]
    dlin = dphi[..., 1:1 + d]
    dquad = dphi[..., 1 + d:1 + d + d * d].reshape(x.shape[:-1] + (d, d))
    sym = dquad + np.swapaxes(dquad, -1, -2)
    return dlin / (d ** 0.25) + np.einsum("...ab,...b->...a", sym, x) / (np.sqrt(2.0) * np.sqrt(d))


def frobenius_rel_error(x: np.ndarray, y: np.ndarray) -> float:
    """|x - y|_F / |y|_F, the metric of flashlinear/test_attn.py:24-25."""
    x = np.asarray(x, dtype=np.float64)
    y = np.asarray(y, dtype=np.float64)
    return float(np.linalg.norm(x - y) / np.linalg.norm(y))


def max_rel_error(x: np.ndarray, y: np.ndarray) -> float:
    """max|x - y| / max|y| per tensor (outputs cross zero, so not elementwise)."""
    x = np.asarray(x, dtype=np.float64)
    y = np.asarray(y, dtype=np.float64)
    return float(np.abs(x - y).max() / np.abs(y).max())
