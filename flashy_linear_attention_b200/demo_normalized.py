"""Times the normalised attention (`LinearAttentionNormalized`) and its three normalisation kernels
against the reference's recipe (product kernels + the README's PyTorch denominator, README.md:27-30)
on seeded synthetic inputs:

    python -m flashy_linear_attention_b200.demo_normalized [--shape B H N D] [--iters K] [--no-recipe]

Needs an sm_100 GPU and the built library; prints one line per measurement (CUDA events).
"""
from __future__ import annotations

import argparse

import torch

from . import LinearAttention, LinearAttentionNormalized, ops


def _time(fn, iters: int) -> float:
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", type=int, nargs=4, default=[4, 32, 8192, 128], metavar=("B", "H", "N", "D"))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-recipe", action="store_true", help="skip the PyTorch-denominator comparison")
    args = ap.parse_args()
    B, H, N, D = args.shape
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(0)
    mk = lambda: torch.randn(B, H, N, D, generator=g)
    q = (torch.nn.functional.elu(mk()) + 1).to(torch.bfloat16).to(dev)
    k = (torch.nn.functional.elu(mk()) + 1).to(torch.bfloat16).to(dev)
    v = mk().to(torch.bfloat16).to(dev)
    dy = mk().to(torch.bfloat16).to(dev)

    num = ops.causal_dot_product_fwd(q, k, v)
    print(f"normalize_fwd          {_time(lambda: ops.normalize_fwd(q, k, num), args.iters):8.3f} ms")
    den = ops.normalize_fwd(q, k, num)
    print(f"normalize_bwd_prepare  {_time(lambda: ops.normalize_bwd_prepare(dy, num, den), args.iters):8.3f} ms")
    _, dden = ops.normalize_bwd_prepare(dy, num, den)
    dq, dk = torch.zeros_like(q), torch.zeros_like(k)
    print(f"normalize_bwd_sweep    {_time(lambda: ops.normalize_bwd_sweep(q, k, dq, dk, dden), args.iters):8.3f} ms")

    def fused():
        q_, k_, v_ = (t.detach().requires_grad_(True) for t in (q, k, v))
        return torch.autograd.grad(LinearAttentionNormalized.apply(q_, k_, v_, 1e-5), (q_, k_, v_), dy)

    def recipe():
        q_, k_, v_ = (t.detach().requires_grad_(True) for t in (q, k, v))
        out = LinearAttention.apply(q_, k_, v_)
        denom = (q_ * k_.cumsum(-2)).sum(dim=-1, keepdim=True) + 1e-5
        return torch.autograd.grad(out / denom, (q_, k_, v_), dy)

    print(f"LinearAttentionNormalized fwd+bwd            {_time(fused, args.iters):8.3f} ms")
    if not args.no_recipe:
        print(f"LinearAttention + PyTorch denominator fwd+bwd {_time(recipe, max(2, args.iters // 2)):8.3f} ms")
    ops.check_status(dev)


if __name__ == "__main__":
    main()
