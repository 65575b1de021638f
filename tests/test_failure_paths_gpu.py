"""The paths that only run when something goes wrong, and the edges of what the kernels write.

* Bounded device-side waits: a wait that nothing ends must give up after its limit, set the
  status word and leave the context usable. Both kinds are made to run out in forms that return
  normally -- a peer flag that never arrives (state exchange), and a tile that is never loaded
  (mbarrier waits of the chunk kernel, through the library's test hook). Nothing here faults,
  traps or hangs the GPU; the limits are set to 20 ms.
* Guard bands: outputs are placed inside larger buffers filled with a sentinel; every byte outside
  the output's own rows and columns must be untouched (TMA stores clipped at ragged sequence ends
  and odd head dims, the wide-head kernels, the row pad / unpad kernels).
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")
SENTINEL = -7.0  # exactly representable in bf16


def _lib():
    from flashy_linear_attention_b200 import _lib

    return _lib


def _desc(t):
    return _lib().FlaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _inputs(B, H, N, dk, dv, seed=0):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    q = (torch.nn.functional.elu(torch.randn(B, H, N, dk, device=DEV, generator=gen)) + 1) / dk ** 0.5
    k = torch.nn.functional.elu(torch.randn(B, H, N, dk, device=DEV, generator=gen)) + 1
    v = torch.randn(B, H, N, dv, device=DEV, generator=gen)
    dy = torch.randn(B, H, N, dv, device=DEV, generator=gen)
    return tuple(t.to(torch.bfloat16) for t in (q, k, v, dy))


def _fresh_status():
    from flashy_linear_attention_b200 import ops

    w = ops._status_word(DEV)
    w.zero_()
    return w


# ------------------------------------------------------------------------------------------------
# bounded waits
# ------------------------------------------------------------------------------------------------
def test_exchange_wait_for_a_peer_that_never_arrives_times_out_cleanly():
    """World of two emulated in one process: rank 0 runs fla_sm100_state_exchange with the 'peer'
    inbox and flags being ordinary local buffers that nobody ever flags."""
    from flashy_linear_attention_b200 import ops

    L = _lib()
    lib = L.load()
    B, H, N, D = 1, 2, 512, 64
    q, k, v, _ = _inputs(B, H, N, D, D)
    a = L.FlaArgs()
    a.batch, a.heads, a.seqlen, a.dk, a.dv = B, H, N, D, D
    a.k, a.v = _desc(k), _desc(v)
    a.segments = 2
    inbox_b, flag_b = ctypes.c_size_t(0), ctypes.c_size_t(0)
    assert lib.fla_sm100_exchange_bytes(ctypes.byref(a), 2, ctypes.byref(inbox_b), ctypes.byref(flag_b)) == 0
    inboxes = [torch.zeros(inbox_b.value, dtype=torch.uint8, device=DEV) for _ in range(2)]
    flags = [torch.zeros(flag_b.value, dtype=torch.uint8, device=DEV) for _ in range(2)]
    remote = torch.zeros(B * H, D, D, dtype=torch.float32, device=DEV)
    inclusive = torch.zeros_like(remote)
    need = lib.fla_sm100_exchange_workspace_bytes(ctypes.byref(a))
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    a.workspace, a.workspace_bytes = ws.data_ptr(), need
    status = _fresh_status()
    a.status = status.data_ptr()
    a.stream = torch.cuda.current_stream(DEV).cuda_stream
    x = L.FlaExchange()
    x.rank, x.world, x.reverse, x.epoch = 0, 2, 0, 1
    for r in range(2):
        x.inbox[r], x.flags[r] = inboxes[r].data_ptr(), flags[r].data_ptr()
    x.remote_out, x.inclusive_out = remote.data_ptr(), inclusive.data_ptr()
    x.wait_limit_us = 20000
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lib.fla_sm100_state_exchange(ctypes.byref(a), 0, ctypes.byref(x)) == 0
    t1.record()
    torch.cuda.synchronize()
    assert 15.0 < t0.elapsed_time(t1) < 2000.0   # waited for the limit, not for the default 0.4 s x blocks
    assert int(status.item()) & 2
    # nothing plausible is left behind
    assert torch.isnan(remote).all() and torch.isnan(inclusive).all()
    assert torch.isnan(ws[: B * H * 2 * D * D * 4].view(torch.float32)).all()
    # rank 0 did publish its total into the 'peer' inbox and raise its flag there
    assert inboxes[1].view(torch.float32).abs().sum().item() > 0
    assert flags[1].view(torch.int32).max().item() == 1
    with pytest.raises(RuntimeError, match="timed out"):
        ops.check_status(DEV)
    # the context is intact and the status word is clear again: an ordinary call works
    out = ops.causal_dot_product_fwd(q, k, v)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert torch.isfinite(out.float()).all()


@pytest.mark.parametrize("dims", [(128, 128), (64, 64), (273, 64)], ids=lambda d: f"dk{d[0]}_dv{d[1]}")
def test_mbarrier_wait_that_runs_out_sets_the_status_bit(dims):
    """The library's test hook withholds the first tile load; every wait that depends on it gives
    up after 20 ms, bit 0 of the status word is set and the kernel returns normally."""
    from flashy_linear_attention_b200 import ops

    L = _lib()
    lib = L.load()
    dk, dv = dims
    B, H, N = 1, 2, 512
    q, k, v, _ = _inputs(B, H, N, dk, dv)
    q, k = ops.kernel_view(q), ops.kernel_view(k)
    out = torch.empty_like(v)
    a = L.FlaArgs()
    a.batch, a.heads, a.seqlen, a.dk, a.dv = B, H, N, dk, dv
    a.q, a.k, a.v, a.o = _desc(q), _desc(k), _desc(v), _desc(out)
    a.segments = 1
    status = _fresh_status()
    a.status = status.data_ptr()
    a.stream = torch.cuda.current_stream(DEV).cuda_stream
    a.wait_limit_us = 20000
    a.debug_flags = L.FLA_DEBUG_WITHHOLD_FIRST_TILE
    assert lib.fla_sm100_fwd(ctypes.byref(a)) == 0
    torch.cuda.synchronize()
    assert int(status.item()) & 1
    # the library recorded which waits gave up first: block indices inside the launch's grid, a
    # thread of the CTA, a barrier inside the CTA's barrier area (just below its abort flag)
    recs = (ctypes.c_uint * (8 * 32))()
    n = lib.fla_sm100_timeout_records(recs, 32)
    assert 1 <= n <= 32
    for r in range(n):
        bar, parity, tid, bx, by, bz, flag_addr, _clk = recs[8 * r: 8 * r + 8]
        assert parity in (0, 1) and tid < 512 and bz < B * H and by == 0
        if dk <= 128:  # the chunk kernel keeps its abort flag right behind its barriers
            assert 0 < flag_addr - bar <= 512 and (flag_addr - bar) % 4 == 0
    assert lib.fla_sm100_timeout_records(recs, 32) == 0  # reading clears them
    with pytest.raises(RuntimeError, match="timed out"):
        ops.check_status(DEV)
    # same arguments without the hook: the call completes and matches the ordinary wrapper
    a.debug_flags = 0
    assert lib.fla_sm100_fwd(ctypes.byref(a)) == 0
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert torch.equal(out, ops.causal_dot_product_fwd(q, k, v, segments=1))


# ------------------------------------------------------------------------------------------------
# guard bands
# ------------------------------------------------------------------------------------------------
def _framed(B, H, N, d, rows_margin=5, cols_margin=8):
    """A [B, H, N, d] view in the middle of a larger sentinel-filled buffer whose row pitch is a
    multiple of 8 elements (16 bytes): `rows_margin` extra rows on both sides of every head and
    `cols_margin` extra columns left and at least that many right of every row."""
    pitch = (d + 7) // 8 * 8 + 2 * cols_margin
    full = torch.full((B, H, N + 2 * rows_margin, pitch), SENTINEL, dtype=torch.bfloat16, device=DEV)
    view = full[:, :, rows_margin:rows_margin + N, cols_margin:cols_margin + d]
    return full, view


def _assert_frame_untouched(full, view, name):
    """Everything outside the view still holds the sentinel. One documented exception: rows are
    stored in 16-byte units, so when the head dim is not a multiple of 8 the (at most 7) elements
    between a row's last column and the next 16-byte boundary are overwritten -- with zeros (the
    header states this and requires the row pitch to cover them)."""
    inside = torch.zeros(full.shape, dtype=torch.bool, device=full.device)
    off = (view.data_ptr() - full.data_ptr()) // 2
    r0, c0 = (off % (full.stride(1))) // full.stride(2), off % full.stride(2)
    d = view.shape[3]
    d8 = (d + 7) // 8 * 8
    inside[:, :, r0:r0 + view.shape[2], c0:c0 + d8] = True
    outside = full[~inside]
    assert (outside == SENTINEL).all(), f"{name}: {(outside != SENTINEL).sum().item()} elements outside the output were written"
    tail = full[:, :, r0:r0 + view.shape[2], c0 + d:c0 + d8]
    assert ((tail == 0) | (tail == SENTINEL)).all(), f"{name}: the 16-byte tail of a row holds something other than zeros"
    assert (view.float() != SENTINEL).any(), f"{name}: output looks unwritten"


@pytest.mark.parametrize("shape", [(1, 2, 200, 128, 128), (2, 1, 333, 64, 64), (1, 2, 192, 83, 83),
                                   (1, 2, 77, 96, 32), (1, 2, 320, 273, 64), (1, 1, 130, 200, 16)],
                         ids=lambda s: "x".join(map(str, s)))
def test_outputs_stay_inside_their_rows_and_columns(shape):
    """Forward and backward through the C ABI with every output framed by sentinel values:
    ragged last chunks, head dims that are not multiples of 8 or 64, and the wide-head kernels."""
    from flashy_linear_attention_b200 import ops

    L = _lib()
    lib = L.load()
    B, H, N, dk, dv = shape
    q, k, v, dy = _inputs(B, H, N, dk, dv, seed=N)
    q, k, v, dy = (ops.kernel_view(t) for t in (q, k, v, dy))
    o_full, o = _framed(B, H, N, dv)
    dq_full, dq = _framed(B, H, N, dk)
    dk_full, dk_ = _framed(B, H, N, dk)
    dv_full, dv_ = _framed(B, H, N, dv)
    a = L.FlaArgs()
    a.batch, a.heads, a.seqlen, a.dk, a.dv = B, H, N, dk, dv
    a.q, a.k, a.v, a.o, a.d_o = _desc(q), _desc(k), _desc(v), _desc(o), _desc(dy)
    a.d_q, a.d_k, a.d_v = _desc(dq), _desc(dk_), _desc(dv_)
    a.segments = 1
    a.status = _fresh_status().data_ptr()
    a.stream = torch.cuda.current_stream(DEV).cuda_stream
    assert lib.fla_sm100_fwd(ctypes.byref(a)) == 0
    assert lib.fla_sm100_bwd(ctypes.byref(a)) == 0
    torch.cuda.synchronize()
    ops.check_status(DEV)
    for name, full, view in (("out", o_full, o), ("dq", dq_full, dq), ("dk", dk_full, dk_), ("dv", dv_full, dv_)):
        _assert_frame_untouched(full, view, name)
    # and the framed results are the ones the ordinary wrappers return
    want_o = ops.causal_dot_product_fwd(q, k, v, segments=1)
    want = ops.causal_dot_product_bwd(dy, q, k, v, segments=1)
    assert torch.equal(o, want_o)
    for got, w in zip((dq, dk_, dv_), want):
        assert torch.equal(got, w)


@pytest.mark.parametrize("rows,d", [(1000, 273), (77, 17), (33, 9), (4096, 83)], ids=lambda x: str(x))
def test_row_pad_and_unpad_kernels_stay_inside_their_destination(rows, d):
    lib = _lib().load()
    dpad = (d + 7) // 8 * 8
    gen = torch.Generator(device=DEV).manual_seed(rows + d)
    src = torch.randn(rows, d, device=DEV, generator=gen).to(torch.bfloat16)
    margin = 64  # elements; keeps the destination 16-byte aligned
    stream = torch.cuda.current_stream(DEV).cuda_stream
    padded = torch.full((rows * dpad + 2 * margin,), SENTINEL, dtype=torch.bfloat16, device=DEV)
    assert lib.fla_sm100_pad_rows(src.data_ptr(), padded[margin:].data_ptr(), rows, d, dpad, stream) == 0
    body = padded[margin:margin + rows * dpad].view(rows, dpad)
    assert torch.equal(body[:, :d], src) and (body[:, d:] == 0).all()
    assert (padded[:margin] == SENTINEL).all() and (padded[margin + rows * dpad:] == SENTINEL).all()
    back = torch.full((rows * d + 2 * margin,), SENTINEL, dtype=torch.bfloat16, device=DEV)
    assert lib.fla_sm100_unpad_rows(body.data_ptr(), back[margin:].data_ptr(), rows, d, dpad, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(back[margin:margin + rows * d].view(rows, d), src)
    assert (back[:margin] == SENTINEL).all() and (back[margin + rows * d:] == SENTINEL).all()
