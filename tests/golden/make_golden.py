"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE'S OWN naive PyTorch
path on the CPU: `linear_ref_torch` (flashlinear/test_attn.py:49-62) for the forward and torch
autograd through it for the gradients, exactly as the reference's tests obtain their expected
values (flashlinear/test_attn.py:107-111), plus the README denominator (README.md:27-30).

Run from the repository root where the reference checkout is available:
    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py
It is not run by the test-suite; the .npz files it writes are committed.
Inputs are generated with numpy's PCG64 so that the fixtures do not depend on torch's RNG.
"""
import os
import sys
import warnings

import numpy as np
import torch

warnings.filterwarnings("ignore")
HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("FLASHLINEAR_REFERENCE")  # or put the reference checkout on PYTHONPATH
if REF:
    sys.path.insert(0, REF)
from flashlinear.test_attn import linear_ref_torch  # noqa: E402  (the reference's oracle)


def elu1(x):
    return torch.nn.functional.elu(x) + 1.0


def make_case(name, B, H, N, dk, dv, seed, dtype, inputs="elu", denom=False, row_stride=1):
    rng = np.random.Generator(np.random.PCG64(seed))
    xq = torch.from_numpy(rng.standard_normal((B, H, N, dk)).astype(np.float32))
    xk = torch.from_numpy(rng.standard_normal((B, H, N, dk)).astype(np.float32))
    v = torch.from_numpy(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    dy = torch.from_numpy(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    if inputs == "elu":  # the benchmark configurations: q, k = elu(x) + 1
        q, k = elu1(xq), elu1(xk)
    else:  # the reference's test inputs: softplus, q scaled by 1/sqrt(hd) (test_attn.py:37-40)
        q = torch.nn.functional.softplus(xq) / (dk ** 0.5)
        k = torch.nn.functional.softplus(xk)
        dy = 0.1 * dy
    if dtype == "bf16":  # inputs are bf16 values; the reference path is evaluated on them in fp32
        q, k, v, dy = (t.to(torch.bfloat16).to(torch.float32) for t in (q, k, v, dy))
    q, k, v = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = linear_ref_torch(q, k, v)
    if denom:
        den = (q * k.cumsum(-2)).sum(dim=-1, keepdim=True) + 1e-5  # README.md:29
        res = out / den
    else:
        res = out
    res.backward(dy)
    rows = slice(None, None, row_stride)
    arrays = dict(
        q=q.detach().numpy(), k=k.detach().numpy(), v=v.detach().numpy(), dy=dy.numpy(),
        out=res.detach().numpy()[..., rows, :],
        dq=q.grad.numpy()[..., rows, :], dk=k.grad.numpy()[..., rows, :], dv=v.grad.numpy()[..., rows, :],
        row_stride=np.int64(row_stride), denom=np.int64(1 if denom else 0),
    )
    if row_stride != 1:
        # Large case: inputs are regenerated from the seed by the test; keep only their checksums.
        for nme in ("q", "k", "v", "dy"):
            a = arrays.pop(nme)
            arrays[nme + "_sum"] = np.float64(a.astype(np.float64).sum())
            arrays[nme + "_sq"] = np.float64((a.astype(np.float64) ** 2).sum())
        arrays.update(seed=np.int64(seed), shape=np.array([B, H, N, dk, dv]), inputs=np.array(inputs), dtype=np.array(dtype))
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(name, {k_: getattr(v_, "shape", None) for k_, v_ in arrays.items()}, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    # small, complete cases (inputs + outputs stored)
    make_case("ref_b1h2_n128_d32_fp32", 1, 2, 128, 32, 32, seed=1, dtype="fp32")
    make_case("ref_b1h1_n192_d64_bf16in", 1, 1, 192, 64, 64, seed=2, dtype="bf16", inputs="softplus")
    make_case("ref_b2h1_n128_dk40_dv16_bf16in", 2, 1, 128, 40, 16, seed=3, dtype="bf16", inputs="softplus")
    make_case("ref_b1h1_n256_d128_bf16in", 1, 1, 256, 128, 128, seed=4, dtype="bf16")
    make_case("ref_b1h1_n64_d16_denominator_fp32", 1, 1, 64, 16, 16, seed=5, dtype="fp32", denom=True)
    # benchmark configuration 1 at full size (B2 H4 N256 D64 fp32 with the denominator): outputs on
    # every 8th token, inputs by seed
    make_case("ref_cfg1_b2h4_n256_d64_fp32_denominator", 2, 4, 256, 64, 64, seed=6, dtype="fp32", denom=True, row_stride=8)
    make_case("ref_cfg1_b2h4_n256_d64_fp32_unnormalised", 2, 4, 256, 64, 64, seed=6, dtype="fp32", denom=False, row_stride=8)
