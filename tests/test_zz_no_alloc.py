"""fla_sm100_fwd_static_scratch: the forward pass for callers that cannot allocate device memory
(a plugin running inside another runtime's fixed memory plan, a serving loop that forbids
allocation once it is warm, host code that is only handed raw pointers). The segmented forward
normally needs caller-provided scratch; this entry point keeps that scratch in an array built into
the library. The test calls it through the C ABI exactly as such a caller would -- inputs and the
output are the caller's, no workspace is passed -- and checks the result against the ordinary
entry point (which gets its scratch from the test), twice in a row because the array is reused
from call to call.

Collected last on purpose (file name), so that a run that stops at the first failure has already
executed every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _args(q, k, v, out, segments, stream, status):
    from flashy_linear_attention_b200._lib import FlaArgs, FlaTensor

    def d(t):
        return FlaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))

    a = FlaArgs()
    a.batch, a.heads, a.seqlen, a.dk = q.shape
    a.dv = v.shape[-1]
    a.q, a.k, a.v, a.o = d(q), d(k), d(v), d(out)
    a.segments = segments
    a.stream = stream
    a.status = status.data_ptr()
    return a


@pytest.mark.parametrize("shape,segments", [((1, 2, 2048, 128, 128), 4), ((2, 3, 1536, 64, 64), 3), ((1, 4, 4096, 128, 128), 0)],
                         ids=["d128_seg4", "d64_seg3", "d128_auto"])
def test_static_scratch_forward_matches_ordinary_forward(shape, segments):
    from flashy_linear_attention_b200 import _lib

    lib = _lib.load()
    B, H, N, dk, dv = shape
    gen = torch.Generator(device=DEV).manual_seed(1234 + N)
    q = (torch.nn.functional.elu(torch.randn(B, H, N, dk, device=DEV, generator=gen)) + 1).to(torch.bfloat16)
    k = (torch.nn.functional.elu(torch.randn(B, H, N, dk, device=DEV, generator=gen)) + 1).to(torch.bfloat16)
    v = torch.randn(B, H, N, dv, device=DEV, generator=gen).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream(torch.device(DEV)).cuda_stream

    with torch.cuda.device(torch.device(DEV)):
        # ordinary entry point: scratch supplied by the caller
        want = torch.empty_like(v)
        a = _args(q, k, v, want, segments, stream, status)
        need = lib.fla_sm100_workspace_bytes(ctypes.byref(a), 0)
        assert need > 0, "the case must be one that uses scratch"
        ws = torch.empty(need, dtype=torch.uint8, device=DEV)
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
        assert lib.fla_sm100_fwd(ctypes.byref(a)) == 0

        # the entry point under test: no workspace, two calls in a row on fresh (poisoned) outputs
        for call in range(2):
            got = torch.full_like(v, float("nan"))
            b = _args(q, k, v, got, segments, stream, status)
            rc = lib.fla_sm100_fwd_static_scratch(ctypes.byref(b))
            assert rc == 0, _lib.strerror(rc)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            assert not torch.isnan(got.float()).any()
            # same kernels in the same order on the same inputs: the tolerance of the parity tests
            # (Frobenius relative error < 1e-2) is met with room to spare, normally exactly
            err = (torch.linalg.norm(got.float() - want.float()) / torch.linalg.norm(want.float())).item()
            assert err < 1e-2, (call, err)
            assert torch.equal(got, want), f"call {call}: differs from fla_sm100_fwd (rel. error {err:.2e})"


def _run_both(lib, q, k, v, segments, s_init=None, want_final=False):
    """(fla_sm100_fwd result, [two fla_sm100_fwd_static_scratch results]) with optional running state;
    each result is (out, s_final or None)."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream(torch.device(DEV)).cuda_stream
    B, H, _, dk = q.shape
    dv = v.shape[-1]

    def one(fn, with_ws):
        out = torch.full_like(v, float("nan"))
        fin = torch.full((B * H, dk, dv), float("nan"), dtype=torch.float32, device=DEV) if want_final else None
        a = _args(q, k, v, out, segments, stream, status)
        if s_init is not None:
            a.s_init = s_init.data_ptr()
        if fin is not None:
            a.s_final = fin.data_ptr()
        ws = None
        if with_ws:
            need = lib.fla_sm100_workspace_bytes(ctypes.byref(a), 0)
            if need:
                ws = torch.empty(need, dtype=torch.uint8, device=DEV)
                a.workspace, a.workspace_bytes = ws.data_ptr(), need
        rc = fn(ctypes.byref(a))
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        return out, fin

    with torch.cuda.device(torch.device(DEV)):
        want = one(lib.fla_sm100_fwd, True)
        got = [one(lib.fla_sm100_fwd_static_scratch, False) for _ in range(2)]
    return want, got


@pytest.mark.parametrize("case", ["unsegmented", "running_state", "wide_qk", "exact_limit"])
def test_static_scratch_forward_covers_what_the_ordinary_forward_covers(case):
    """Shapes that need no scratch are dispatched like fla_sm100_fwd (one segment; q/k wider than
    128 with a narrow v), running-state arguments work with segments, and a shape whose segment
    states fill the built-in array to the last byte is accepted."""
    from flashy_linear_attention_b200 import _lib

    lib = _lib.load()
    shape, segments, state = {
        "unsegmented": ((2, 80, 512, 64, 64), 0, False),     # 160 heads: one segment, no scratch
        "running_state": ((1, 3, 2048, 128, 128), 4, True),
        "wide_qk": ((1, 2, 512, 272, 64), 0, False),
        "exact_limit": ((1, 32, 4096, 128, 128), 16, False),  # 32 x 16 x 128 x 128 x 4 B = 32 MiB
    }[case]
    B, H, N, dk, dv = shape
    gen = torch.Generator(device=DEV).manual_seed(99 + N + dk)
    q = ((torch.nn.functional.elu(torch.randn(B, H, N, dk, device=DEV, generator=gen)) + 1) / dk ** 0.5).to(torch.bfloat16)
    k = (torch.nn.functional.elu(torch.randn(B, H, N, dk, device=DEV, generator=gen)) + 1).to(torch.bfloat16)
    v = torch.randn(B, H, N, dv, device=DEV, generator=gen).to(torch.bfloat16)
    s_init = torch.randn(B * H, dk, dv, device=DEV, generator=gen) if state else None
    if case == "exact_limit":
        assert B * H * segments * dk * dv * 4 == 32 * 1024 * 1024
    want, got = _run_both(lib, q, k, v, segments, s_init=s_init, want_final=state)
    for out, fin in got:
        assert torch.equal(out, want[0])
        if state:
            assert torch.equal(fin, want[1])


def test_static_scratch_rejects_shapes_beyond_its_limit():
    from flashy_linear_attention_b200 import _lib

    lib = _lib.load()
    # 64 heads x 16 segments x 128 x 128 x 4 B = 64 MiB of segment states > 32 MiB built in
    B, H, N, d = 1, 64, 4096, 128
    q = torch.zeros(B, H, N, d, dtype=torch.bfloat16, device=DEV)
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream(torch.device(DEV)).cuda_stream
    with torch.cuda.device(torch.device(DEV)):
        a = _args(q, q, q, out, 16, stream, status)
        rc = lib.fla_sm100_fwd_static_scratch(ctypes.byref(a))
    assert rc == -7
    assert "scratch" in _lib.strerror(rc)
