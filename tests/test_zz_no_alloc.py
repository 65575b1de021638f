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
