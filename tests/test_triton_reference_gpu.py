"""Same-box comparison with the reference's own Triton kernels.

baseline/install_reference.py copies the reference package to baseline/_ref/flashlinear_triton_ref
and repairs the eight one-tuple lines that Triton 3.6 refuses to compile (the kernels are
otherwise unmodified). These tests run that copy and this library on the same bf16 inputs and
compare outputs and gradients with the reference tests' own metric and bound
(flashlinear/test_attn.py:17,24-25,117-119: Frobenius relative error < 1e-2), plus the max-relative
bound of 2e-2. The copy is a comparator only; the library never imports it.

Skipped (with the reason) when the copy is absent or Triton cannot compile it on this box.
"""
import importlib
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
DEV = "cuda:0"
FROB_TOL = 1e-2      # BFLOAT16_MAX_TOL of the reference's tests
MAX_REL_TOL = 2e-2


def _reference():
    if not os.path.isdir(os.path.join(REF_DIR, "flashlinear_triton_ref")):
        pytest.skip("baseline/_ref/flashlinear_triton_ref is absent (run baseline/install_reference.py)")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    try:
        return importlib.import_module("flashlinear_triton_ref")
    except Exception as exc:  # triton missing or unusable
        pytest.skip(f"the reference package does not import here: {type(exc).__name__}: {exc}")


def _inputs(B, H, N, dk, dv, seed, reference_distribution):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    q = torch.randn(B, H, N, dk, device=DEV, generator=gen)
    k = torch.randn(B, H, N, dk, device=DEV, generator=gen)
    v = torch.randn(B, H, N, dv, device=DEV, generator=gen)
    dy = torch.randn(B, H, N, dv, device=DEV, generator=gen)
    if reference_distribution:
        # make_input_qkv of the reference's tests: softplus on q, k, q scaled by 1/sqrt(hd); dy = 0.1 randn
        q = torch.nn.functional.softplus(q) * dk ** -0.5
        k = torch.nn.functional.softplus(k)
        dy = 0.1 * dy
    else:  # the benchmark's distribution
        q = torch.nn.functional.elu(q) + 1
        k = torch.nn.functional.elu(k) + 1
    return tuple(t.to(torch.bfloat16) for t in (q, k, v, dy))


def _run(fn, q, k, v, dy):
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out = fn.apply(q, k, v)
    dq, dk_, dv = torch.autograd.grad(out, (q, k, v), dy)
    return out, dq, dk_, dv


def _compare(ours, theirs):
    for name, a, b in zip(("out", "dq", "dk", "dv"), ours, theirs):
        a, b = a.float(), b.float()
        frob = (torch.linalg.norm(a - b) / torch.linalg.norm(b)).item()
        max_rel = ((a - b).abs().max() / b.abs().max()).item()
        assert frob < FROB_TOL and max_rel <= MAX_REL_TOL, f"{name}: frobenius {frob:.3e}, max-rel {max_rel:.3e}"


def _triton_or_skip(fn, *args):
    try:
        res = _run(fn, *args)
        torch.cuda.synchronize()
        return res
    except AssertionError:
        raise
    except Exception as exc:
        pytest.skip(f"Triton did not compile or launch the reference kernel: {type(exc).__name__}: {str(exc)[:300]}")


# shapes from the ranges of the reference's own tests (test_attn.py:65-74,122-131) and benchmark
# configuration 2 at full size
SHAPES = [
    (1, 3, 256, 64, True),
    (2, 5, 1024, 128, True),
    (3, 7, 1984, 32, True),
    (2, 4, 640, 83, True),     # "masked_hd": head dim that is not a power of two
    (8, 16, 4096, 64, False),  # configuration 2
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(str(x) for x in s[:4]))
def test_linear_attention_matches_the_reference_triton_kernels(shape):
    from flashlinear import LinearAttention

    ref = _reference()
    B, H, N, D, refdist = shape
    q, k, v, dy = _inputs(B, H, N, D, D, seed=N + D, reference_distribution=refdist)
    theirs = _triton_or_skip(ref.LinearAttention, q, k, v, dy)
    ours = _run(LinearAttention, q, k, v, dy)
    torch.cuda.synchronize()
    _compare(ours, theirs)


SHAPES_SMALLV = [
    (2, 3, 512, 64, 16),
    (1, 6, 1024, 128, 32),
    (2, 2, 448, 100, 16),   # odd hd_qk inside the reference's tested range [32, 128)
    (1, 2, 512, 256, 64),   # the reference's widest legal hd_qk (linear_attn_kernels_smallv_hd.py:339)
]


@pytest.mark.parametrize("shape", SHAPES_SMALLV, ids=lambda s: "x".join(str(x) for x in s))
def test_smallv_function_matches_the_reference_triton_kernels(shape):
    from flashlinear import LinearAttentionSmallVHD

    ref = _reference()
    B, H, N, dk, dv = shape
    q, k, v, dy = _inputs(B, H, N, dk, dv, seed=N + dk + dv, reference_distribution=True)
    theirs = _triton_or_skip(ref.LinearAttentionSmallVHD, q, k, v, dy)
    ours = _run(LinearAttentionSmallVHD, q, k, v, dy)
    torch.cuda.synchronize()
    _compare(ours, theirs)
