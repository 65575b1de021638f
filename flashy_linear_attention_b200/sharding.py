"""Multi-GPU use of the causal linear attention kernels: one process per GPU, torch.distributed.

Two partitionings (the reference has neither; its launch grid is a single GPU's
(seq blocks, batch*heads), flashlinear/kernels/linear_attn_kernels.py:329-330):

* batch*head sharding -- heads are independent, so every rank runs the ordinary Functions on its
  slice of [batch, heads]; there is no data-path collective (`shard_batch_heads`).
* sequence sharding -- rank r holds tokens [r*N/W, (r+1)*N/W) of every head. The only exchange is
  the per-rank dk x dv fp32 state: an exclusive scan over ranks of S_r = sum k^T v for the forward
  and dQ, and a reverse exclusive scan of R_r = sum q^T dO for dK, dV
  (`exclusive_state_scan`, `SequenceShardedLinearAttention`). The states land in local memory
  through one all-gather; kernels read them from there.
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
import torch.distributed as dist

from . import ops


def shard_batch_heads(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rank `rank`'s slice of a [batch, heads, ...] tensor when the batch*heads independent heads are
    split evenly over `world` ranks (batch first, then heads). Returns a view."""
    B, H = t.shape[0], t.shape[1]
    if (B * H) % world != 0:
        raise ValueError(f"batch*heads = {B * H} is not divisible by world size {world}")
    if B % world == 0:
        per = B // world
        return t[rank * per:(rank + 1) * per]
    if world % B != 0 or H % (world // B) != 0:
        raise ValueError(f"cannot split batch={B}, heads={H} evenly over {world} ranks")
    ranks_per_batch = world // B
    hper = H // ranks_per_batch
    b = rank // ranks_per_batch
    h0 = (rank % ranks_per_batch) * hper
    return t[b:b + 1, h0:h0 + hper]


def exclusive_state_scan(
    local: torch.Tensor, group: Optional[dist.ProcessGroup] = None, reverse: bool = False
) -> torch.Tensor:
    """Sum of the `local` tensors of all ranks before this one (after it when reverse=True), fp32.

    One all-gather into local memory followed by a local sum: with at most 8 ranks and states of a
    few MB the exchange is latency-bound, so a single collective beats a send/recv chain.
    Works with NCCL (CUDA tensors) and gloo (CPU tensors)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if world == 1:
        return torch.zeros_like(local)
    local = local.contiguous()
    flat = torch.empty(world * local.numel(), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, local.reshape(-1), group=group)
    gathered = flat.view((world,) + tuple(local.shape))
    sel = gathered[rank + 1:] if reverse else gathered[:rank]
    if sel.shape[0] == 0:
        return torch.zeros_like(local)
    return sel.sum(dim=0)


class SequenceShardedLinearAttention(torch.autograd.Function):
    """``apply(q, k, v, group)`` on the local token shard of every head; returns the local shard of
    the unnormalised causal product over the whole (sharded) sequence."""

    @staticmethod
    def forward(ctx: Any, q, k, v, group=None):
        rank = dist.get_rank(group)
        # State pass first (its per-segment states stay in `ws` for the forward below), then the
        # exchange of the per-GPU totals, then the forward on top of the received prefix.
        s_local, ws = ops.chunk_state(k, v, keep_workspace=True)
        s_prefix = exclusive_state_scan(s_local, group, reverse=False)
        out = ops.causal_dot_product_fwd(q, k, v, s_init=s_prefix if rank > 0 else None,
                                         segment_workspace=ws if ws.numel() > 0 else None)
        # The state after this shard's tokens lets the backward sweep its inputs once.
        s_after = s_prefix + s_local
        ctx.save_for_backward(q, k, v, s_prefix, s_after)
        ctx.group = group
        return out

    @staticmethod
    def backward(ctx: Any, grad_output) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, None]:
        q, k, v, s_prefix, s_after = ctx.saved_tensors
        rank, world = dist.get_rank(ctx.group), dist.get_world_size(ctx.group)
        grad_output = grad_output.contiguous()
        r_local = ops.chunk_state(q, grad_output)
        r_suffix = exclusive_state_scan(r_local, ctx.group, reverse=True)
        dq, dk, dv = ops.causal_dot_product_bwd(
            grad_output, q, k, v,
            s_init=s_prefix if rank > 0 else None,        # rank 0 starts the sequence: no prefix
            r_init=r_suffix if rank < world - 1 else None,  # the last rank ends it: no suffix
            s_last=s_after,
        )
        return dq, dk, dv, None
