"""Two-GPU tests (skipped on a single-GPU box): sequence sharding with the NCCL state scan and
batch*head sharding, each against the unsharded result on one GPU."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make(B, H, N, D, device):
    gen = torch.Generator(device="cpu").manual_seed(7)  # identical on every rank
    q = (torch.nn.functional.elu(torch.randn(B, H, N, D, generator=gen)) + 1).to(torch.bfloat16)
    k = (torch.nn.functional.elu(torch.randn(B, H, N, D, generator=gen)) + 1).to(torch.bfloat16)
    v = torch.randn(B, H, N, D, generator=gen).to(torch.bfloat16)
    dy = torch.randn(B, H, N, D, generator=gen).to(torch.bfloat16)
    return [t.to(device) for t in (q, k, v, dy)]


def _rel(a, b):
    return (torch.linalg.norm(a.float() - b.float()) / torch.linalg.norm(b.float())).item()


def _worker(rank, world, port, mode):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    from flashlinear import LinearAttention
    from flashy_linear_attention_b200 import ops
    from flashy_linear_attention_b200.sharding import (
        PeerShardedLinearAttention,
        PeerStateExchange,
        SequenceShardedLinearAttention,
        shard_batch_heads,
    )

    B, H, N, D = 2, 4, 2048, 128
    q, k, v, dy = _make(B, H, N, D, device)
    # unsharded result on this GPU
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    full = LinearAttention.apply(qf, kf, vf)
    full.backward(dy)
    if mode in ("sequence", "sequence_peer"):
        lo, hi = rank * N // world, (rank + 1) * N // world
        ql, kl, vl = (t[:, :, lo:hi].contiguous().requires_grad_(True) for t in (q, k, v))
        if mode == "sequence":
            out = SequenceShardedLinearAttention.apply(ql, kl, vl, None)
            out.backward(dy[:, :, lo:hi].contiguous())
        else:
            # exchange fused into the state kernels over peer-mapped memory; two steps, so that both
            # parity buffers and the epoch counters are exercised
            ex = PeerStateExchange(B, H, D, D, device)
            for step in range(2):
                ql.grad = kl.grad = vl.grad = None
                out = PeerShardedLinearAttention.apply(ql, kl, vl, ex)
                out.backward(dy[:, :, lo:hi].contiguous())
            torch.cuda.synchronize()
            # the same exchange replayed from a CUDA graph (its exchange count lives on the device)
            from flashy_linear_attention_b200.graphs import capture_step

            def fwd_only():
                ws, _, _ = ex.state_and_exchange(kl.detach(), vl.detach(), reverse=False)
                return ops.causal_dot_product_fwd(ql.detach(), kl.detach(), vl.detach(), segment_workspace=ws)

            replay = capture_step(fwd_only)
            for _ in range(3):
                graphed = replay()
            torch.cuda.synchronize()
            assert torch.equal(graphed, out.detach()), (rank, "graph replay differs from the eager call")
            ex.close()
        want = (full[:, :, lo:hi], qf.grad[:, :, lo:hi], kf.grad[:, :, lo:hi], vf.grad[:, :, lo:hi])
    else:
        ql, kl, vl = (shard_batch_heads(t, rank, world).contiguous().requires_grad_(True) for t in (q, k, v))
        out = LinearAttention.apply(ql, kl, vl)
        out.backward(shard_batch_heads(dy, rank, world).contiguous())
        want = tuple(shard_batch_heads(t, rank, world) for t in (full, qf.grad, kf.grad, vf.grad))
    torch.cuda.synchronize()
    ops.check_status(device)
    for name, got, ref in zip(("out", "dq", "dk", "dv"), (out, ql.grad, kl.grad, vl.grad), want):
        err = _rel(got, ref)
        # the sharded run sums the same products in another order: well inside the bf16 tolerance
        assert err < 5e-3, (mode, rank, name, err)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["sequence", "sequence_peer", "batch_head"])
def test_two_gpu_sharding(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port(), mode), nprocs=2, join=True)
