"""Times `TaylorLinearAttention` (raw q, k -> second-order Taylor features -> causal product, all in
the library's kernels) against the same computation with the feature map written in PyTorch and
`LinearAttentionSmallVHD` on the materialised features, on seeded synthetic inputs:

    python -m flashy_linear_attention_b200.demo_taylor [--shape B H N DV] [--iters K] [--no-torch-map]

Raw head dim 16 (273 features). Needs an sm_100 GPU and the built library.
"""
from __future__ import annotations

import argparse

import torch

from . import LinearAttentionSmallVHD, TaylorLinearAttention, ops


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


def torch_feature_map(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1]
    x2 = (x.unsqueeze(-1) * x.unsqueeze(-2)).flatten(-2) / (2 ** 0.5 * d ** 0.5)
    return torch.cat([torch.ones_like(x[..., :1]), x / d ** 0.25, x2], dim=-1)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", type=int, nargs=4, default=[8, 16, 2048, 64], metavar=("B", "H", "N", "DV"))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-torch-map", action="store_true", help="skip the PyTorch feature-map comparison")
    args = ap.parse_args()
    B, H, N, dv = args.shape
    d = 16
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(0)
    xq = torch.randn(B, H, N, d, generator=g).to(torch.bfloat16).to(dev)
    xk = torch.randn(B, H, N, d, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(B, H, N, dv, generator=g).to(torch.bfloat16).to(dev)
    dy = torch.randn(B, H, N, dv, generator=g).to(torch.bfloat16).to(dev)

    print(f"taylor_features         {_time(lambda: ops.taylor_features(xq), args.iters):8.3f} ms")
    phi = ops.taylor_features(xq)
    dphi = torch.randn(phi.shape[:-1] + (phi.stride(2),), device=dev).to(torch.bfloat16)[..., : phi.shape[-1]]
    print(f"taylor_features_bwd     {_time(lambda: ops.taylor_features_bwd(dphi, xq), args.iters):8.3f} ms")

    def fused():
        a, b, c = (t.detach().requires_grad_(True) for t in (xq, xk, v))
        return torch.autograd.grad(TaylorLinearAttention.apply(a, b, c), (a, b, c), dy)

    def unfused():
        a, b, c = (t.detach().requires_grad_(True) for t in (xq, xk, v))
        out = LinearAttentionSmallVHD.apply(torch_feature_map(a), torch_feature_map(b), c)
        return torch.autograd.grad(out, (a, b, c), dy)

    print(f"TaylorLinearAttention fwd+bwd                        {_time(fused, args.iters):8.3f} ms")
    if not args.no_torch_map:
        print(f"PyTorch feature map + LinearAttentionSmallVHD fwd+bwd {_time(unfused, max(2, args.iters // 2)):8.3f} ms")
    ops.check_status(dev)


if __name__ == "__main__":
    main()
