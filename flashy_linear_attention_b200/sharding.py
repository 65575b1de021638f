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

import ctypes
from typing import Any, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib, ops
from ._lib import FlaArgs, FlaExchange


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


class PeerStateExchange:
    """State exchange of sequence sharding over peer-mapped memory instead of NCCL.

    Every rank owns an inbox and a flag array in its own HBM; the other ranks of the node map them
    through CUDA IPC. `state_and_exchange()` then runs the state pass and ONE kernel that scans the
    segment states, stores this rank's total into every peer's inbox over NVLink, waits (bounded)
    for the peers' totals and folds the ones that precede (follow) this rank into the segment
    prefixes -- see fla_sm100_state_exchange in include/flashlinear_sm100.h.
    All ranks must call it the same number of times in the same order.

    A wait that runs out does not stop the step: the kernel sets bit 1 of the device's status word
    and turns everything it produces into NaN, so the outputs of that step are NaN. Call
    `ops.check_status(device)` at the next point where the host synchronises anyway (end of a step,
    before an optimizer update); `close()` does so as well."""

    def __init__(self, batch: int, heads: int, dk: int, dv: int, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None, wait_limit_us: int = 0):
        # wait_limit_us: how long a block waits for a peer's flag before it gives up (0 = the
        # library's default of 0.4 s). Ranks that may reach an exchange further apart than that
        # (first-step compilation, a slow data loader) should raise it.
        self.wait_limit_us = int(wait_limit_us)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > _lib.FLA_MAX_RANKS:
            raise ValueError(f"PeerStateExchange supports up to {_lib.FLA_MAX_RANKS} ranks")
        self.device = device
        self.shape = (batch, heads, dk, dv)
        self._lib = lib = _lib.load()
        a = FlaArgs()
        a.batch, a.heads, a.seqlen, a.dk, a.dv = batch, heads, 128, dk, dv
        inbox_b, flag_b = ctypes.c_size_t(0), ctypes.c_size_t(0)
        rc = lib.fla_sm100_exchange_bytes(ctypes.byref(a), self.world, ctypes.byref(inbox_b), ctypes.byref(flag_b))
        if rc != 0:
            raise RuntimeError(_lib.strerror(rc))
        self._owned, self._opened = [], []
        # one buffer set per direction (forward states / backward states), each with its own epoch
        self._sets = []
        with torch.cuda.device(device):
            for _ in range(2):
                mine = []
                for nbytes in (inbox_b.value, flag_b.value):
                    ptr = ctypes.c_void_p()
                    handle = ctypes.create_string_buffer(64)
                    rc = lib.fla_sm100_exchange_alloc(nbytes, ctypes.byref(ptr), handle)
                    if rc != 0:
                        raise RuntimeError(f"flashlinear: exchange buffer allocation: {_lib.strerror(rc)}")
                    self._owned.append(ptr.value)
                    mine.append((ptr.value, handle.raw))
                gathered = [None] * self.world
                dist.all_gather_object(gathered, (self.rank, mine[0][1], mine[1][1]), group=group)
                inbox_ptrs, flag_ptrs = [0] * self.world, [0] * self.world
                for r, h_inbox, h_flags in gathered:
                    if r == self.rank:
                        inbox_ptrs[r], flag_ptrs[r] = mine[0][0], mine[1][0]
                        continue
                    for dst, h in ((inbox_ptrs, h_inbox), (flag_ptrs, h_flags)):
                        ptr = ctypes.c_void_p()
                        # opened with THIS rank's device current: its kernels store into the peer
                        rc = lib.fla_sm100_exchange_open(h, ctypes.byref(ptr))
                        if rc != 0:
                            raise RuntimeError(f"flashlinear: mapping rank {r}'s exchange buffer: {_lib.strerror(rc)}")
                        self._opened.append(ptr.value)
                        dst[r] = ptr.value
                # the exchange count lives on the device (one word per buffer set), so that calls
                # carry no argument that changes between launches and can be replayed from a CUDA graph
                counter = torch.zeros(1, dtype=torch.int32, device=device)
                self._sets.append({"inbox": inbox_ptrs, "flags": flag_ptrs, "counter": counter})
        dist.barrier(group=group)

    def close(self) -> None:
        """Unmaps the peers' buffers and frees this rank's (call on every rank, after a barrier)."""
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            failure = None
            try:
                ops.check_status(self.device)
            except RuntimeError as exc:  # report it after the buffers are released
                failure = exc
            for p in self._opened:
                self._lib.fla_sm100_exchange_close(p)
            self._opened = []
            if dist.is_initialized():
                dist.barrier(group=self.group)  # nobody frees memory a peer still has mapped
            for p in self._owned:
                self._lib.fla_sm100_exchange_free(p)
            self._owned = []
        if failure is not None:
            raise failure

    def state_and_exchange(self, b: torch.Tensor, c: torch.Tensor, reverse: bool, segments: int = 0):
        """States of this rank's tokens (sum b^T c), exchanged. Returns (workspace, remote, inclusive):
        the scratch with the per-segment prefixes (for segment_workspace=...), the fp32
        [batch*heads, db, dc] sum over the ranks before (after, if reverse) this one, and that sum
        plus this rank's own total."""
        ops._check_inputs(b, c)
        B, H, N, db = b.shape
        dc = c.shape[-1]
        if (B, H, db, dc) != self.shape:
            raise ValueError("PeerStateExchange was created for another shape")
        lib = _lib.load()
        bset = self._sets[1 if reverse else 0]
        bv, cv = ops._kernel_view(b), ops._kernel_view(c)
        remote = torch.empty(B * H, db, dc, dtype=torch.float32, device=b.device)
        inclusive = torch.empty_like(remote)
        a = FlaArgs()
        a.batch, a.heads, a.seqlen, a.dk, a.dv = B, H, N, db, dc
        # operands go where fla_sm100_state_exchange(which) reads them: which=0 reads k, v
        a.k, a.v = ops._desc(bv), ops._desc(cv)
        a.segments = segments
        x = FlaExchange()
        x.rank, x.world, x.reverse, x.epoch = self.rank, self.world, 1 if reverse else 0, 0
        x.epoch_counter = bset["counter"].data_ptr()
        x.wait_limit_us = self.wait_limit_us
        for r in range(self.world):
            x.inbox[r] = bset["inbox"][r]
            x.flags[r] = bset["flags"][r]
        x.remote_out = remote.data_ptr()
        x.inclusive_out = inclusive.data_ptr()
        with torch.cuda.device(b.device):
            need = lib.fla_sm100_exchange_workspace_bytes(ctypes.byref(a))
            ws = torch.empty(need, dtype=torch.uint8, device=b.device)
            a.workspace, a.workspace_bytes = ws.data_ptr(), need
            a.stream = torch.cuda.current_stream(b.device).cuda_stream
            a.status = ops._status_word(b.device).data_ptr()
            rc = lib.fla_sm100_state_exchange(ctypes.byref(a), 0, ctypes.byref(x))
        if rc != 0:
            raise RuntimeError(f"flashlinear: fla_sm100_state_exchange returned {rc}: {_lib.strerror(rc)}")
        return ws, remote, inclusive


class PeerShardedLinearAttention(torch.autograd.Function):
    """SequenceShardedLinearAttention with the exchange fused into the state kernels
    (`apply(q, k, v, exchange)` with a PeerStateExchange made for these shapes)."""

    @staticmethod
    def forward(ctx: Any, q, k, v, exchange: PeerStateExchange):
        ws, s_prefix, s_after = exchange.state_and_exchange(k, v, reverse=False)
        # the scratch already holds prefix-of-other-ranks + local segment prefixes
        out = ops.causal_dot_product_fwd(q, k, v, segment_workspace=ws)
        ctx.save_for_backward(q, k, v, s_prefix, s_after)
        ctx.exchange = exchange
        return out

    @staticmethod
    def backward(ctx: Any, grad_output):
        q, k, v, s_prefix, s_after = ctx.saved_tensors
        ex = ctx.exchange
        grad_output = grad_output.contiguous()
        _, r_suffix, _ = ex.state_and_exchange(q, grad_output, reverse=True)
        dq, dk, dv = ops.causal_dot_product_bwd(
            grad_output, q, k, v,
            s_init=s_prefix if ex.rank > 0 else None,
            r_init=r_suffix if ex.rank < ex.world - 1 else None,
            s_last=s_after,
        )
        return dq, dk, dv, None
