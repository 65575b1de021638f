"""Forward + backward for tensors that live in pinned host memory.

The causal product is independent per (batch, head), so host-resident q, k, v, dO are cut into
slabs of heads and streamed: while slab i is computed, slab i+1 crosses PCIe host->device and
the results of slab i-1 cross device->host (three CUDA streams, events between them). One step
then costs about max(host->device, device->host) instead of their sum plus the kernels.

This has no counterpart in the reference (its wrappers, flashlinear/kernels/
linear_attn_kernels.py:310-384, take device tensors only); it exists for callers whose
activations are offloaded to host memory.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import ops


def _flat_heads(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 4 or not t.is_contiguous():
        raise ValueError("host pipeline: tensors must be contiguous [batch, heads, tokens, dim]")
    return t.view(t.shape[0] * t.shape[1], t.shape[2], t.shape[3])


class HostPipeline:
    """Streams slabs of heads through the sm_100a kernels.

    depth staging sets of device buffers are allocated on first use (torch's caching allocator)
    and reused by every later call with the same slab shape. Not thread-safe: one pipeline per
    calling thread and device.
    """

    def __init__(self, device, heads_per_slab: int = 16, depth: int = 3):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("host pipeline: needs a CUDA device (no CPU fallback exists)")
        if heads_per_slab < 1 or depth < 2:
            raise ValueError("host pipeline: heads_per_slab >= 1 and depth >= 2 required")
        self.heads_per_slab = heads_per_slab
        self.depth = depth
        self._h2d = torch.cuda.Stream(self.device)
        self._d2h = torch.cuda.Stream(self.device)
        self._staging: List[Optional[Tuple[torch.Tensor, ...]]] = [None] * depth
        self._staging_key = None

    def _stage(self, slot: int, shapes: Sequence[Tuple[int, ...]], dtype) -> Tuple[torch.Tensor, ...]:
        key = (tuple(shapes), dtype)
        if self._staging_key != key:
            self._staging = [None] * self.depth
            self._staging_key = key
        if self._staging[slot] is None:
            self._staging[slot] = tuple(torch.empty(s, dtype=dtype, device=self.device) for s in shapes)
        return self._staging[slot]

    def fwd_bwd(
        self,
        q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, grad_output: torch.Tensor,
        out: torch.Tensor, d_q: torch.Tensor, d_k: torch.Tensor, d_v: torch.Tensor,
    ) -> None:
        """out = causal product of (q, k, v); (d_q, d_k, d_v) = its gradients for `grad_output`.

        All eight tensors are pinned host tensors, bf16, contiguous [batch, heads, tokens, dim]
        (q, k, d_q, d_k with dim dk; v, grad_output, out, d_v with dim dv). The call is
        asynchronous: the results are complete once the current stream of the device has been
        synchronised.
        """
        ins = (q, k, v, grad_output)
        outs = (out, d_q, d_k, d_v)
        for t in ins + outs:
            if t.is_cuda or not t.is_pinned():
                raise ValueError("host pipeline: all tensors must be pinned host tensors")
            if t.dtype != torch.bfloat16:
                raise ValueError("host pipeline: tensors must be bfloat16")
        for a, b in ((out, v), (d_q, q), (d_k, k), (d_v, v), (k, q), (grad_output, v)):
            if a.shape != b.shape:
                raise ValueError("host pipeline: shape mismatch between inputs and outputs")
        fin = [_flat_heads(t) for t in ins]
        fout = [_flat_heads(t) for t in outs]
        BH, N = fin[0].shape[0], fin[0].shape[1]
        hs = min(self.heads_per_slab, BH)
        nslab = (BH + hs - 1) // hs

        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        self._h2d.wait_event(start)
        self._d2h.wait_event(start)
        computed: List[Optional[torch.cuda.Event]] = [None] * self.depth
        last_out = None
        for s in range(nslab):
            h0, h1 = s * hs, min(BH, (s + 1) * hs)
            n = h1 - h0
            slot = s % self.depth
            stage = self._stage(slot, [(hs,) + tuple(t.shape[1:]) for t in fin], torch.bfloat16)
            with torch.cuda.stream(self._h2d):
                if computed[slot] is not None:      # the kernels that read this staging set are done
                    self._h2d.wait_event(computed[slot])
                for dst, src in zip(stage, fin):
                    dst[:n].copy_(src[h0:h1], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(self._h2d)
            cur.wait_event(arrived)
            qs, ks, vs, gs = (t[:n].unsqueeze(0) for t in stage)
            state = seg_states = None
            if ops.backward_uses_final_state(qs, vs):
                state = torch.empty(n, qs.shape[-1], vs.shape[-1], dtype=torch.float32, device=self.device)
                seg_states = ops.segment_states_buffer(qs, vs)
            o = ops.causal_dot_product_fwd(qs, ks, vs, s_final=state, seg_states=seg_states)
            grads = ops.causal_dot_product_bwd(gs, qs, ks, vs, s_last=state, seg_states=seg_states)
            done = torch.cuda.Event()
            done.record(cur)
            computed[slot] = done
            with torch.cuda.stream(self._d2h):
                self._d2h.wait_event(done)
                for dst, src in zip(fout, (o,) + tuple(grads)):
                    dst[h0:h1].copy_(src[0], non_blocking=True)
                    src.record_stream(self._d2h)
                last_out = torch.cuda.Event()
                last_out.record(self._d2h)
        cur.wait_event(last_out)
