"""Launch wrappers with the names, arguments and error behaviour of the reference's
``flashlinear.kernels`` module (flashlinear/kernels/linear_attn_kernels.py:310-384 and
flashlinear/kernels/linear_attn_kernels_smallv_hd.py:320-405), calling the sm_100a kernels of
libflashlinear_sm100.so through its C ABI instead of Triton.

All four wrappers return the *unnormalised* causal product ``(Q K^T (.) M) V`` (or its gradients);
the denominator stays in PyTorch, as in the reference (README.md:22-30).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import FlaArgs, FlaTensor

KERNEL_HEAD_DIM = 128  # widest head-dim tile of the main kernel
WIDE_HEAD_DIM = 384    # widest head dim (either side) that one library call covers
WIDE_NARROW_DIM = 64   # c/out width of one launch of the wide (SmallVHD) kernel
MAX_HEAD_DIM = 256     # cap of LinearAttention, as in the reference (linear_attn_kernels.py:322)
MAX_HEAD_DIM_QK_SMALLV = 512  # cap of q/k for LinearAttentionSmallVHD (273-dim Taylor features fit)

_status_words = {}
# FLA_DEBUG_* bits passed with every call; FLA_DEBUG_FLAGS in the environment sets the initial value
_debug_flags = int(os.environ.get("FLA_DEBUG_FLAGS", "0") or 0)


def set_debug_flags(flags: int) -> int:
    """Sets the FLA_DEBUG_* bits passed with every later call (0 in production) and returns the
    previous value. Used by tests, e.g. to keep the three-launch segmented form for comparison."""
    global _debug_flags
    old, _debug_flags = _debug_flags, int(flags)
    return old


def _next_pow2(x: int) -> int:
    return 1 << (max(int(x), 1) - 1).bit_length()


_first_use_status: dict = {}  # device index -> status word after the first-use launches (0 = clean)


def _status_word(device: torch.device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _status_words[key] = w
        _first_use(torch.device("cuda", key), w)
    return w


def _first_use(device: torch.device, status: torch.Tensor) -> None:
    """One throw-away forward + backward per kernel instantiation (head dims 64 and 128) the first
    time a device is used, then the status word is cleared.

    Why: on some B200 hosts the very first launch of the 64-wide kernel in a process that started
    right after another one had exited ran into its wait limit (then 0.4 s of the SM's cycle counter;
    about one fresh process in ten on two hosts, never on three others, never in any later launch).
    The likely cause is preemption: the kernel shares the GPU with the previous process's context
    while that is being torn down, and a CTA that is switched out keeps "waiting" by the clock, or
    resumes on another SM whose cycle counter is unrelated. The waits are timed with the global
    timer and allowed 2 s since; this launch on 160 heads of 128 tokens, whose results nobody reads,
    additionally keeps the module load, the SMs' switch to the kernel's shared-memory configuration
    and the cold instruction caches off a caller's first real call. Skipped while a stream is being
    captured (nothing may synchronise then)."""
    if torch.cuda.is_current_stream_capturing():
        return
    lib = _lib.load()
    stream = torch.cuda.current_stream(device).cuda_stream
    with torch.cuda.device(device):
        for d in (64, 128):
            x = torch.ones(1, 160, 128, d, dtype=torch.bfloat16, device=device)  # a CTA on every SM
            outs = [torch.empty_like(x) for _ in range(4)]
            a = FlaArgs()
            a.batch, a.heads, a.seqlen, a.dk, a.dv = 1, 160, 128, d, d
            a.q, a.k, a.v, a.d_o = _desc(x), _desc(x), _desc(x), _desc(x)
            a.o, a.d_q, a.d_k, a.d_v = (_desc(t) for t in outs)
            a.segments = 1
            a.status = status.data_ptr()
            a.stream = stream
            lib.fla_sm100_fwd(ctypes.byref(a))
            lib.fla_sm100_bwd(ctypes.byref(a))
        torch.cuda.synchronize(device)
        _first_use_status[device.index] = int(status.item())  # kept for diagnosis; not an error
        status.zero_()
        scratch = (ctypes.c_uint * 8)()
        lib.fla_sm100_timeout_records(scratch, 1)  # drop whatever the warm-up may have recorded


def check_status(device=None) -> None:
    """Synchronises and raises RuntimeError if a kernel on `device` gave up on a bounded wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _status_word(dev)
    val = int(w.item())
    if val != 0:
        w.zero_()
        raise RuntimeError(
            f"flashlinear sm_100a kernel reported status {val}: a device-side wait timed out; "
            "results of the affected call are invalid"
        )


def _check_inputs(*tensors: torch.Tensor, allow_half: bool = False) -> None:
    """Device, rank and dtype checks shared by the wrappers. bfloat16 everywhere; the product
    kernels also take float16 (allow_half) when every tensor of the call is float16 and no head dim
    exceeds 128."""
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError(
                "flashlinear: tensors must be CUDA tensors on an sm_100 GPU (no CPU fallback exists)"
            )
        if t.device != dev:
            raise RuntimeError("flashlinear: all tensors must be on the same device")
    if allow_half and all(t.dtype == torch.float16 for t in tensors):
        if max(t.shape[-1] for t in tensors) > KERNEL_HEAD_DIM:
            raise TypeError("flashlinear: float16 tensors need head dims <= 128 (wider heads are bfloat16 only)")
    else:
        for t in tensors:
            if t.dtype != torch.bfloat16:
                raise TypeError(
                    "flashlinear: expected torch.bfloat16 tensors"
                    + (" (or torch.float16 throughout)" if allow_half else "")
                    + f", got {t.dtype} (use torch.autocast or cast the inputs)"
                )
    for t in tensors:
        if t.dim() != 4:
            raise ValueError("flashlinear: expected [batch, heads, seq, head_dim] tensors")


def _addressable(t: torch.Tensor) -> bool:
    """True if the kernels can read or write `t` in place: unit innermost stride, 16-byte aligned
    base and row/head/batch strides (what a TMA tensor map needs)."""
    d = t.shape[-1]
    ok = t.stride(3) == 1 and t.data_ptr() % 16 == 0 and t.stride(2) >= d
    for dim in (0, 1, 2):
        if t.shape[dim] > 1 and t.stride(dim) % 8 != 0:
            ok = False
    return ok


def _padded_empty(shape, dtype, device) -> torch.Tensor:
    """View [..., :d] of a fresh tensor whose rows are padded to a multiple of 8 elements."""
    d = shape[-1]
    dpad = (d + 7) // 8 * 8
    buf = torch.empty(tuple(shape[:-1]) + (dpad,), dtype=dtype, device=device)
    return buf[..., :d]


def _rows_call(name: str, src: torch.Tensor, dst: torch.Tensor, rows: int, d: int, dpad: int) -> None:
    lib = _lib.load()
    with torch.cuda.device(src.device):
        rc = getattr(lib, name)(src.data_ptr(), dst.data_ptr(), rows, d, dpad,
                                torch.cuda.current_stream(src.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"flashlinear: {name} returned {rc}: {_lib.strerror(rc)}")


def _kernel_view(t: torch.Tensor) -> torch.Tensor:
    """Returns `t` if the kernels can read it in place, else a repacked copy whose rows are padded
    to 8 elements (the library's pad kernel for contiguous tensors, a strided torch copy otherwise)."""
    if _addressable(t):
        return t
    view = _padded_empty(t.shape, t.dtype, t.device)
    d = t.shape[-1]
    if t.is_contiguous() and t.data_ptr() % 4 == 0:
        _rows_call("fla_sm100_pad_rows", t, view, t.numel() // d, d, view.stride(2))
    else:
        view.copy_(t)
    return view


def kernel_view(t: torch.Tensor) -> torch.Tensor:
    """Public form of the repack: callers that run several passes over the same tensor (forward then
    backward) repack it once and hand the view to every pass."""
    return _kernel_view(t)


def _out_like(t: torch.Tensor, keep_padded: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Output with the layout of ``torch.empty_like(t)`` plus the view the kernel writes to
    (a padded scratch tensor when empty_like's layout is not addressable by the kernels).
    keep_padded=True returns the padded view as the output itself (no copy back)."""
    if keep_padded and t.shape[-1] % 8 != 0:
        view = _padded_empty(t.shape, t.dtype, t.device)
        return view, view
    out = torch.empty_like(t)
    kv = _kernel_view_for_output(out)
    return out, kv


def _kernel_view_for_output(out: torch.Tensor) -> torch.Tensor:
    if _addressable(out):
        return out
    return _padded_empty(out.shape, out.dtype, out.device)


def _copy_back(full: torch.Tensor, view: torch.Tensor) -> None:
    """Result from the padded scratch rows into the caller-layout output."""
    if view is full:
        return
    d = full.shape[-1]
    if full.is_contiguous() and full.data_ptr() % 4 == 0:
        _rows_call("fla_sm100_unpad_rows", view, full, full.numel() // d, d, view.stride(2))
    else:
        full.copy_(view)


def _dtype_code(t: torch.Tensor) -> int:
    return _lib.FLA_DTYPE_F16 if t.dtype == torch.float16 else _lib.FLA_DTYPE_BF16


def _desc(t: Optional[torch.Tensor]) -> FlaTensor:
    if t is None:
        return FlaTensor(None, 0, 0, 0)
    return FlaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _fptr(t: Optional[torch.Tensor], name: str, shape) -> Optional[int]:
    if t is None:
        return None
    if t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != tuple(shape):
        raise ValueError(f"flashlinear: {name} must be a contiguous float32 tensor of shape {tuple(shape)}")
    return t.data_ptr()


def _call(pass_id: int, args: FlaArgs, device: torch.device, which: int = 0,
          workspace: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """One C-ABI call on the current stream. Scratch comes from torch's allocator unless the
    caller hands in `workspace`; the scratch tensor (or None) is returned."""
    lib = _lib.load()
    with torch.cuda.device(device):
        args.stream = torch.cuda.current_stream(device).cuda_stream
        args.status = _status_word(device).data_ptr()
        args.debug_flags = _debug_flags
        need = lib.fla_sm100_workspace_bytes(ctypes.byref(args), 0 if pass_id == 3 else pass_id)
        ws = workspace
        if ws is not None:
            if ws.numel() * ws.element_size() < need:
                raise ValueError("flashlinear: the workspace handed in is too small for this call")
            args.workspace = ws.data_ptr()
            args.workspace_bytes = ws.numel() * ws.element_size()
        elif need > 0:
            ws = torch.empty(need, dtype=torch.uint8, device=device)
            args.workspace = ws.data_ptr()
            args.workspace_bytes = need
        if pass_id == 0:
            rc = lib.fla_sm100_fwd(ctypes.byref(args))
        elif pass_id == 1:
            rc = lib.fla_sm100_bwd(ctypes.byref(args))
        elif pass_id == 2:
            rc = lib.fla_sm100_state(ctypes.byref(args), which)
        else:
            rc = lib.fla_sm100_product(ctypes.byref(args), which)
    if rc != 0:
        raise RuntimeError(f"flashlinear: libflashlinear_sm100 returned {rc}: {_lib.strerror(rc)}")
    if os.environ.get("FLA_DEBUG", "0") == "1":
        check_status(device)
    return ws


def _product_call(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, out: torch.Tensor, anticausal: bool) -> None:
    """out = causal (or anti-causal) product of kernel-addressable views, head dims <= 128."""
    B, H, N, da = a.shape
    args = FlaArgs()
    args.batch, args.heads, args.seqlen, args.dk, args.dv = B, H, N, da, c.shape[-1]
    args.q, args.k, args.v, args.o = _desc(a), _desc(b), _desc(c), _desc(out)
    args.dtype = _dtype_code(a)
    _call(3, args, a.device, which=1 if anticausal else 0)


def _native_dims(da: int, dc: int) -> bool:
    """Head-dim pairs (a/b side, c/out side) that one library call covers."""
    return da <= WIDE_HEAD_DIM and dc <= WIDE_HEAD_DIM


def _product_sliced(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, like: torch.Tensor, anticausal: bool) -> torch.Tensor:
    """Causal product for any head dims. Up to 384 on either side the library takes the call as it
    is (128-wide tiles; a/b wider: the wide kernel, which accumulates the whole a/b width on chip;
    c/out wider: independent column slices). Beyond that the product is assembled here by
    linearity: output columns are independent (slices of c), and (a_i . b_j) is the sum over
    slices of the a/b head dim, so the partial products of those slices are added. Each partial
    product leaves its kernel rounded to bf16; their sum is formed in fp32 and rounded once more."""
    av, bv, cv = _kernel_view(a), _kernel_view(b), _kernel_view(c)
    da, dc = a.shape[-1], c.shape[-1]
    W = KERNEL_HEAD_DIM
    out, ov = _out_like(like)
    if _native_dims(da, dc):
        _product_call(av, bv, cv, ov, anticausal)
        _copy_back(out, ov)
        return out
    for c0 in range(0, dc, W):
        c1 = min(dc, c0 + W)
        if da <= W:
            _product_call(av, bv, cv[..., c0:c1], ov[..., c0:c1], anticausal)
            continue
        acc = None
        part = torch.empty(c.shape[:-1] + (c1 - c0,), dtype=c.dtype, device=c.device)
        for a0 in range(0, da, W):
            a1 = min(da, a0 + W)
            _product_call(av[..., a0:a1], bv[..., a0:a1], cv[..., c0:c1], part, anticausal)
            acc = part.float() if acc is None else acc + part.float()
        ov[..., c0:c1] = acc.to(c.dtype)
    _copy_back(out, ov)
    return out


def causal_dot_product_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    s_init: Optional[torch.Tensor] = None,
    s_final: Optional[torch.Tensor] = None,
    segments: int = 0,
    segment_workspace: Optional[torch.Tensor] = None,
    seg_states: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """out[b,h,i] = sum_{j<=i} (q_i . k_j) v_j, bf16 in / bf16 out (or fp16 in / fp16 out for head
    dims up to 128), fp32 accumulation.

    s_init / s_final are optional fp32 [batch*heads, dk, dv] running states (sum of k_j^T v_j
    before / after this call's tokens) for sequence-sharded or resumed calls.
    segment_workspace: the scratch tensor returned by chunk_state(k, v, keep_workspace=True) for the
    same k, v and `segments`; the call then reuses the segment states found there instead of
    reading k, v once more to recompute them (s_final is not available in that case).
    seg_states: buffer from segment_states_buffer(q, v); a segmented forward stores the state at its
    segment boundaries there, and causal_dot_product_bwd(..., s_last=..., seg_states=...) then runs
    the backward as one launch split at those boundaries (few heads per GPU).
    """
    _check_inputs(q, k, v, allow_half=True)
    B, H, N, dk = q.shape
    dv = v.shape[-1]
    if dk > KERNEL_HEAD_DIM or dv > KERNEL_HEAD_DIM:
        if s_init is not None or s_final is not None:
            raise NotImplementedError("running-state arguments need head dims <= 128")
        return _product_sliced(q, k, v, v, anticausal=False)  # one library call for SmallVHD shapes
    qv, kv_, vv = _kernel_view(q), _kernel_view(k), _kernel_view(v)
    out, ov = _out_like(v)
    a = FlaArgs()
    a.batch, a.heads, a.seqlen, a.dk, a.dv = B, H, N, dk, dv
    a.q, a.k, a.v, a.o = _desc(qv), _desc(kv_), _desc(vv), _desc(ov)
    a.dtype = _dtype_code(q)
    a.s_init = _fptr(s_init, "s_init", (B * H, dk, dv))
    a.s_final = _fptr(s_final, "s_final", (B * H, dk, dv))
    a.segments = segments
    if segment_workspace is not None:
        if s_final is not None:
            raise ValueError("flashlinear: s_final cannot be combined with segment_workspace")
        a.segment_states_ready = 1
    if seg_states is not None:
        a.seg_states, a.seg_states_bytes = seg_states.data_ptr(), seg_states.numel() * seg_states.element_size()
    _call(0, a, q.device, workspace=segment_workspace)
    _copy_back(out, ov)
    return out


def causal_dot_product_bwd(
    grad_output: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    s_init: Optional[torch.Tensor] = None,
    r_init: Optional[torch.Tensor] = None,
    r_final: Optional[torch.Tensor] = None,
    segments: int = 0,
    s_last: Optional[torch.Tensor] = None,
    keep_padded: bool = False,
    seg_states: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients (dQ, dK, dV) of causal_dot_product_fwd for upstream gradient `grad_output`.

    s_last (optional) is the forward state after these tokens, i.e. what the forward call wrote to
    `s_final`; with it the backward reads q, k, v, dO from HBM only once.
    keep_padded=True: gradients whose head dim is not a multiple of 8 are returned as views of the
    row-padded tensors the kernels wrote, instead of being copied to the contiguous layout."""
    _check_inputs(grad_output, q, k, v, allow_half=True)
    B, H, N, dk = q.shape
    dv = v.shape[-1]
    wide = max(dk, dv) > KERNEL_HEAD_DIM and max(dk, dv) <= WIDE_HEAD_DIM  # one library call covers it
    if wide and any(t is not None for t in (s_init, r_init, r_final, s_last)):
        raise NotImplementedError("running-state arguments need head dims <= 128")
    if (dk > KERNEL_HEAD_DIM or dv > KERNEL_HEAD_DIM) and not wide:
        if any(t is not None for t in (s_init, r_init, r_final, s_last)):
            raise NotImplementedError("running-state arguments need head dims <= 128")
        # the three gradients as products with permuted operands (see fla_sm100_product)
        dQ = _product_sliced(grad_output, v, k, q, anticausal=False)
        dV = _product_sliced(k, q, grad_output, v, anticausal=True)
        dK = _product_sliced(v, grad_output, q, k, anticausal=True)
        return dQ, dK, dV
    gv, qv, kv_, vv = (_kernel_view(t) for t in (grad_output, q, k, v))
    dQ, dQv = _out_like(q, keep_padded)
    dK, dKv = _out_like(k, keep_padded)
    dV, dVv = _out_like(v, keep_padded)
    a = FlaArgs()
    a.batch, a.heads, a.seqlen, a.dk, a.dv = B, H, N, dk, dv
    a.q, a.k, a.v, a.d_o = _desc(qv), _desc(kv_), _desc(vv), _desc(gv)
    a.d_q, a.d_k, a.d_v = _desc(dQv), _desc(dKv), _desc(dVv)
    a.dtype = _dtype_code(q)
    a.s_init = _fptr(s_init, "s_init", (B * H, dk, dv))
    a.r_init = _fptr(r_init, "r_init", (B * H, dk, dv))
    a.r_final = _fptr(r_final, "r_final", (B * H, dk, dv))
    a.s_last = _fptr(s_last, "s_last", (B * H, dk, dv))
    a.segments = segments
    if seg_states is not None:
        a.seg_states, a.seg_states_bytes = seg_states.data_ptr(), seg_states.numel() * seg_states.element_size()
    _call(1, a, q.device)
    for full, view in ((dQ, dQv), (dK, dKv), (dV, dVv)):
        _copy_back(full, view)
    return dQ, dK, dV


def _norm_args(ref: torch.Tensor, dk: int, dv: int) -> FlaArgs:
    a = FlaArgs()
    a.batch, a.heads, a.seqlen, a.dk, a.dv = ref.shape[0], ref.shape[1], ref.shape[2], dk, dv
    a.stream = torch.cuda.current_stream(ref.device).cuda_stream
    a.status = _status_word(ref.device).data_ptr()
    return a


def _norm_workspace(a: FlaArgs, device: torch.device) -> Optional[torch.Tensor]:
    need = _lib.load().fla_sm100_normalize_workspace_bytes(ctypes.byref(a))
    if need == 0:
        return None
    ws = torch.empty(need, dtype=torch.uint8, device=device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), need
    return ws


def _norm_check(rc: int, name: str) -> None:
    if rc != 0:
        raise RuntimeError(f"flashlinear: {name} returned {rc}: {_lib.strerror(rc)}")


def normalize_fwd(q: torch.Tensor, k: torch.Tensor, num: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """Divides `num` (the unnormalised product, [B,H,N,dv] bf16) IN PLACE by the denominator of
    README.md:27-30, den_i = q_i . sum_{j<=i} k_j + eps, and returns den as fp32 [B*H, N].
    q, k, num must be addressable by the kernels (see kernel_view)."""
    _check_inputs(q, k, num)
    if not (_addressable(q) and _addressable(k) and _addressable(num)):
        raise ValueError("flashlinear: normalize_fwd needs 16-byte aligned rows (use ops.kernel_view)")
    B, H, N, dk = q.shape
    den = torch.empty(B * H, N, dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        a = _norm_args(q, dk, num.shape[-1])
        a.q, a.k, a.o = _desc(q), _desc(k), _desc(num)
        ws = _norm_workspace(a, q.device)  # noqa: F841 (kept alive until the launches are queued)
        _norm_check(_lib.load().fla_sm100_normalize_fwd(ctypes.byref(a), float(eps), den.data_ptr()),
                    "fla_sm100_normalize_fwd")
    return den


def normalize_bwd_prepare(g: torch.Tensor, out: torch.Tensor, den: torch.Tensor):
    """(dnum, dden) for upstream gradient g of the normalised output `out`: dnum = g / den (bf16,
    the upstream gradient of the unnormalised product), dden = -(g . out) / den (fp32 [B*H, N])."""
    _check_inputs(g, out)
    g = _kernel_view(g)
    B, H, N, dv = out.shape
    dnum = _padded_empty(out.shape, out.dtype, out.device) if dv % 8 else torch.empty(
        out.shape, dtype=out.dtype, device=out.device)
    dden = torch.empty(B * H, N, dtype=torch.float32, device=out.device)
    with torch.cuda.device(out.device):
        a = _norm_args(out, dv, dv)
        a.d_o, a.o, a.d_v = _desc(g), _desc(out), _desc(dnum)
        _norm_check(_lib.load().fla_sm100_normalize_bwd_prepare(ctypes.byref(a), den.data_ptr(), dden.data_ptr()),
                    "fla_sm100_normalize_bwd_prepare")
    return dnum, dden


def normalize_bwd_sweep(q: torch.Tensor, k: torch.Tensor, dq: torch.Tensor, dk: torch.Tensor,
                        dden: torch.Tensor) -> None:
    """Adds the denominator's gradient to dq and dk in place:
    dq_i += dden_i * sum_{j<=i} k_j,  dk_j += sum_{i>=j} dden_i q_i."""
    _check_inputs(q, k, dq, dk)
    if not all(_addressable(t) for t in (q, k, dq, dk)):
        raise ValueError("flashlinear: normalize_bwd_sweep needs 16-byte aligned rows (use ops.kernel_view)")
    with torch.cuda.device(q.device):
        a = _norm_args(q, q.shape[-1], q.shape[-1])
        a.q, a.k, a.d_q, a.d_k = _desc(q), _desc(k), _desc(dq), _desc(dk)
        ws = _norm_workspace(a, q.device)  # noqa: F841
        _norm_check(_lib.load().fla_sm100_normalize_bwd_sweep(ctypes.byref(a), dden.data_ptr()),
                    "fla_sm100_normalize_bwd_sweep")


def taylor_features(x: torch.Tensor) -> torch.Tensor:
    """Second-order Taylor features phi(x) = [1, x / d^(1/4), vec(x x^T) / (sqrt(2) sqrt(d))] of raw
    x [B, H, N, d] (bf16, d = 8 or 16): a [B, H, N, 1 + d + d^2] view of rows padded to a multiple
    of 8 elements, which the attention kernels read in place (no repack)."""
    _check_inputs(x)
    lib = _lib.load()
    d = x.shape[-1]
    f, fp = ctypes.c_int(0), ctypes.c_int(0)
    if lib.fla_sm100_taylor_dims(d, ctypes.byref(f), ctypes.byref(fp)) != 0:
        raise NotImplementedError("flashlinear: Taylor features are built for raw head dims 8 and 16")
    xc = x.contiguous()
    buf = torch.empty(x.shape[:-1] + (fp.value,), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.fla_sm100_taylor_features(xc.data_ptr(), buf.data_ptr(), xc.numel() // d, d,
                                           torch.cuda.current_stream(x.device).cuda_stream)
    _norm_check(rc, "fla_sm100_taylor_features")
    return buf[..., :f.value]


def taylor_features_bwd(dphi: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Gradient with respect to raw x of taylor_features(x) for feature gradients dphi
    ([B, H, N, 1 + d + d^2], rows padded to a multiple of 8 elements as taylor_features returns
    and as causal_dot_product_bwd(..., keep_padded=True) produces)."""
    _check_inputs(dphi, x)
    lib = _lib.load()
    d = x.shape[-1]
    f, fp = ctypes.c_int(0), ctypes.c_int(0)
    if lib.fla_sm100_taylor_dims(d, ctypes.byref(f), ctypes.byref(fp)) != 0:
        raise NotImplementedError("flashlinear: Taylor features are built for raw head dims 8 and 16")
    rows = x.numel() // d
    dense = (dphi.shape[-1] == f.value and dphi.stride(3) == 1 and dphi.stride(2) == fp.value
             and dphi.stride(1) == fp.value * dphi.shape[2] and dphi.stride(0) == dphi.stride(1) * dphi.shape[1])
    if not dense:  # bring the gradient into padded rows
        buf = torch.zeros(dphi.shape[:-1] + (fp.value,), dtype=dphi.dtype, device=dphi.device)
        buf[..., :f.value] = dphi
        dphi = buf[..., :f.value]
    xc = x.contiguous()
    dx = torch.empty_like(xc)
    with torch.cuda.device(x.device):
        rc = lib.fla_sm100_taylor_features_bwd(dphi.data_ptr(), xc.data_ptr(), dx.data_ptr(), rows, d,
                                               torch.cuda.current_stream(x.device).cuda_stream)
    _norm_check(rc, "fla_sm100_taylor_features_bwd")
    return dx


def backward_uses_final_state(q: torch.Tensor, v: torch.Tensor) -> bool:
    """True when the backward of this shape can take the forward's final state (`s_last`) and sweep
    q, k, v, dO once for all three gradients: it runs unsegmented, or as one launch split at the
    forward's segment boundaries (then segment_states_buffer() is not None as well), and the
    sequence is longer than 2048 tokens (shorter ones keep the two-direction form, which is a
    little more accurate there)."""
    B, H, N, dk = q.shape
    if dk > KERNEL_HEAD_DIM or v.shape[-1] > KERNEL_HEAD_DIM:
        return False
    a = FlaArgs()
    a.batch, a.heads, a.seqlen, a.dk, a.dv = B, H, N, dk, v.shape[-1]
    a.debug_flags = _debug_flags
    with torch.cuda.device(q.device):
        return _lib.load().fla_sm100_bwd_uses_final_state(ctypes.byref(a)) != 0


def segment_states_buffer(q: torch.Tensor, v: torch.Tensor, segments: int = 0) -> Optional[torch.Tensor]:
    """Scratch for the states a segmented forward hands to its backward (few heads per GPU), or None
    when forward + backward of this shape do not use it. Pass it as `seg_states` to
    causal_dot_product_fwd and causal_dot_product_bwd, together with s_final / s_last."""
    B, H, N, dk = q.shape
    if dk > KERNEL_HEAD_DIM or v.shape[-1] > KERNEL_HEAD_DIM:
        return None
    a = FlaArgs()
    a.batch, a.heads, a.seqlen, a.dk, a.dv = B, H, N, dk, v.shape[-1]
    a.segments = segments
    a.debug_flags = _debug_flags
    with torch.cuda.device(q.device):
        need = _lib.load().fla_sm100_seg_states_bytes(ctypes.byref(a))
    if need == 0:
        return None
    return torch.empty(need, dtype=torch.uint8, device=q.device)


def chunk_state(b: torch.Tensor, c: torch.Tensor, segments: int = 0, keep_workspace: bool = False):
    """fp32 [batch*heads, db, dc] sum over tokens of b_j^T c_j: with (k, v) the forward state S of
    these tokens, with (q, dO) the backward state R. Used by sequence-sharded callers.
    keep_workspace=True returns (state, workspace): the scratch then holds the per-segment prefix
    states, which causal_dot_product_fwd(..., segment_workspace=workspace) can reuse."""
    _check_inputs(b, c, allow_half=True)
    B, H, N, db = b.shape
    dc = c.shape[-1]
    bv, cv = _kernel_view(b), _kernel_view(c)
    out = torch.empty(B * H, db, dc, dtype=torch.float32, device=b.device)
    a = FlaArgs()
    a.batch, a.heads, a.seqlen, a.dk, a.dv = B, H, N, db, dc
    a.dtype = _dtype_code(b)
    a.k, a.v = _desc(bv), _desc(cv)
    a.s_final = out.data_ptr()
    a.segments = segments
    ws = _call(2, a, b.device, which=0)
    if keep_workspace:
        if ws is None:  # unsegmented call: nothing to reuse, but keep the calling convention
            ws = torch.empty(0, dtype=torch.uint8, device=b.device)
        return out, ws
    return out


# ------------------------------------------------------------------------------------------------
# The reference's four wrapper names.
# ------------------------------------------------------------------------------------------------


def _assert_shapes(hd_qk: int, sq: int, cap: int = MAX_HEAD_DIM) -> None:
    # Same preconditions (and AssertionError) as the reference wrappers
    # (linear_attn_kernels.py:316-325: hd <= 256, sq a multiple of BLOCK_SQ = 64, or 32 above 128).
    block_sq = 64 if _next_pow2(hd_qk) <= 128 else 32
    assert hd_qk <= cap, f"Only head_dims <= {cap} are supported."
    assert (
        sq % block_sq == 0
    ), f"Number of elements in sequence must be a multiple of {block_sq}, {sq, block_sq}"


def check_forward_preconditions(q: torch.Tensor, v: torch.Tensor, smallv: bool) -> None:
    """The AssertionErrors of linear_flash_wrapper_fwd / linear_flash_wrapper_fwd_smallv_hd."""
    hd_qk, sq, hd_v = q.shape[-1], q.shape[-2], v.shape[-1]
    if smallv:
        assert _next_pow2(hd_v) == hd_v, "Expected value head dimension to be a power of 2."
        assert _next_pow2(hd_v) <= _next_pow2(
            hd_qk
        ), "Value head dimension must be less than Query/Key head dimension."
    # The reference caps hd_qk at 256 (linear_attn_kernels_smallv_hd.py:339); the cap is raised
    # here so that 273-dimensional second-order Taylor features are accepted.
    _assert_shapes(hd_qk, sq, MAX_HEAD_DIM_QK_SMALLV if smallv else MAX_HEAD_DIM)


def linear_flash_wrapper_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Causal linear attention forward, dk == dv (linear_attn_kernels.py:310-341)."""
    check_forward_preconditions(q, v, smallv=False)
    return causal_dot_product_fwd(q, k, v)


def linear_flash_wrapper_bwd(
    grad_output: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Causal linear attention backward, dk == dv (linear_attn_kernels.py:345-384)."""
    batch, nh, sq, hd = q.shape
    _assert_shapes(hd, sq)
    return causal_dot_product_bwd(grad_output, q, k, v)


def linear_flash_wrapper_fwd_smallv_hd(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor
) -> torch.Tensor:
    """Forward with separate q/k and v head dims (linear_attn_kernels_smallv_hd.py:320-359)."""
    check_forward_preconditions(q, v, smallv=True)
    return causal_dot_product_fwd(q, k, v)


def linear_flash_wrapper_bwd_smallv_hd(
    grad_output: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Backward with separate q/k and v head dims (linear_attn_kernels_smallv_hd.py:363-405)."""
    batch, nh, sq, hd_qk = q.shape
    assert hd_qk <= MAX_HEAD_DIM_QK_SMALLV, f"Only head_dims <= {MAX_HEAD_DIM_QK_SMALLV} are supported."
    assert sq % 64 == 0, "Number of elements in sequence must be a multiple of 64"
    return causal_dot_product_bwd(grad_output, q, k, v)
