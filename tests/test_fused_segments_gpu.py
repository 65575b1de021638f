"""Few heads per GPU: the segmented forward and backward as ONE cooperative launch each.

When batch*heads is far below the SM count (the headline job split over 8 GPUs leaves 16 heads per
GPU) every head is cut into sequence segments. The fused form sums each segment's state, meets at a
grid-wide barrier and starts every segment's attention loop from the partial sums of the segments
before it, all inside one launch; the forward also hands the state at its segment boundaries to the
backward. These tests compare it with the CPU oracle, with the unsegmented kernels and with the
older three-launch form (kept behind a debug flag), which computes the same sums in another order.
"""
import numpy as np
import pytest
import torch

from oracle import linear_attention_oracle as orc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
MAX_REL_TOL = 2e-2
FROB_TOL = 1e-2


def _inputs(B, H, N, D, seed):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    q = (torch.nn.functional.elu(torch.randn(B, H, N, D, device=DEV, generator=gen)) + 1).to(torch.bfloat16)
    k = (torch.nn.functional.elu(torch.randn(B, H, N, D, device=DEV, generator=gen)) + 1).to(torch.bfloat16)
    v = torch.randn(B, H, N, D, device=DEV, generator=gen).to(torch.bfloat16)
    dy = torch.randn(B, H, N, D, device=DEV, generator=gen).to(torch.bfloat16)
    return q, k, v, dy


def _frob(a, b):
    return (torch.linalg.norm(a.float() - b.float()) / torch.linalg.norm(b.float())).item()


def _step(q, k, v, dy, segments=0, use_seg_states=True, sync=True):
    """Forward + backward the way LinearAttention.apply runs them; returns (out, dq, dk, dv, used_seg_states)."""
    from flashy_linear_attention_b200 import ops

    B, H, _, D = q.shape
    s_final = torch.empty(B * H, D, D, dtype=torch.float32, device=DEV)
    seg_states = ops.segment_states_buffer(q, v, segments) if use_seg_states else None
    out = ops.causal_dot_product_fwd(q, k, v, s_final=s_final, segments=segments, seg_states=seg_states)
    grads = ops.causal_dot_product_bwd(dy, q, k, v, s_last=s_final, segments=segments, seg_states=seg_states)
    if sync:
        torch.cuda.synchronize()
        ops.check_status(DEV)
    return (out,) + tuple(grads) + (seg_states is not None,)


@pytest.mark.parametrize("shape", [(1, 16, 8192, 128), (1, 4, 4096, 128), (2, 4, 4096, 64), (1, 1, 2048, 128),
                                   (1, 7, 3072, 128), (1, 3, 1920, 64)],
                         ids=lambda s: "x".join(map(str, s)))
def test_fused_forward_and_backward_match_the_other_forms(shape):
    from flashy_linear_attention_b200 import _lib, ops

    B, H, N, D = shape
    q, k, v, dy = _inputs(B, H, N, D, seed=N + H)
    fused = _step(q, k, v, dy)
    # the same call without the boundary states: fused forward, the backward falls back
    plain = _step(q, k, v, dy, use_seg_states=False)
    # the older three-launch segmented form
    old = ops.set_debug_flags(_lib.FLA_DEBUG_NO_FUSED_SEGMENTS)
    try:
        three = _step(q, k, v, dy)
        assert not three[4]
    finally:
        ops.set_debug_flags(old)
    # unsegmented kernels
    whole = _step(q, k, v, dy, segments=1)
    for name, a, b, c, d in zip(("out", "dq", "dk", "dv"), fused, plain, three, whole):
        # the forms sum the same terms in different orders (and dQ either as a growing prefix or as
        # total minus suffix), so they differ by bf16 roundings of a few outputs
        for other, label in ((b, "fused fwd only"), (c, "three launches"), (d, "unsegmented")):
            assert _frob(a, other) < 5e-3, (name, label, _frob(a, other))
        assert torch.isfinite(a.float()).all()
    # one head against the oracle
    h = H - 1
    q64, k64, v64, dy64 = (t[B - 1, h].float().cpu().numpy().astype(np.float64) for t in (q, k, v, dy))
    want = (orc.linear_ref(q64, k64, v64),) + tuple(orc.linear_ref_grads(q64, k64, v64, dy64))
    for name, got, w in zip(("out", "dq", "dk", "dv"), fused, want):
        g = got[B - 1, h].float().cpu().numpy()
        mr, fr = orc.max_rel_error(g, w), orc.frobenius_rel_error(g, w)
        assert mr <= MAX_REL_TOL and fr < FROB_TOL, f"{name}: max-rel {mr:.3e}, frobenius {fr:.3e}"


def test_sixteen_heads_use_the_boundary_states():
    """The shape the headline job leaves on each of 8 GPUs must actually take the fused backward."""
    from flashy_linear_attention_b200 import ops

    q, k, v, dy = _inputs(1, 16, 8192, 128, seed=1)
    assert ops.segment_states_buffer(q, v) is not None
    assert ops.backward_uses_final_state(q, v)
    from flashy_linear_attention_b200 import _lib
    lib = _lib.load()
    s_final = torch.empty(16, 128, 128, dtype=torch.float32, device=DEV)
    seg_states = ops.segment_states_buffer(q, v)
    ops.causal_dot_product_fwd(q, k, v, s_final=s_final, seg_states=seg_states)
    assert lib.fla_sm100_last_launch_count() == 1
    ops.causal_dot_product_bwd(dy, q, k, v, s_last=s_final, seg_states=seg_states)
    assert lib.fla_sm100_last_launch_count() == 1
    torch.cuda.synchronize()
    ops.check_status(DEV)


@pytest.mark.parametrize("shape", [(1, 16, 8192, 128), (1, 2, 2048, 64)], ids=lambda s: "x".join(map(str, s)))
def test_function_with_few_heads_against_the_oracle_and_repeated(shape):
    """LinearAttention.apply + backward on a few-heads shape, twice in a row (the barrier words and
    the scratch are reused from call to call), and replayed from a CUDA graph."""
    from flashlinear import LinearAttention
    from flashy_linear_attention_b200 import ops
    from flashy_linear_attention_b200.graphs import capture_step

    B, H, N, D = shape
    q, k, v, dy = _inputs(B, H, N, D, seed=7)
    results = []
    for _ in range(2):
        tq, tk, tv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
        out = LinearAttention.apply(tq, tk, tv)
        grads = torch.autograd.grad(out, (tq, tk, tv), dy)
        results.append((out.detach(),) + grads)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    for a, b in zip(*results):
        assert torch.equal(a, b)
    h = H // 2
    q64, k64, v64, dy64 = (t[0, h].float().cpu().numpy().astype(np.float64) for t in (q, k, v, dy))
    want = (orc.linear_ref(q64, k64, v64),) + tuple(orc.linear_ref_grads(q64, k64, v64, dy64))
    for name, got, w in zip(("out", "dq", "dk", "dv"), results[0], want):
        g = got[0, h].float().cpu().numpy()
        mr, fr = orc.max_rel_error(g, w), orc.frobenius_rel_error(g, w)
        assert mr <= MAX_REL_TOL and fr < FROB_TOL, f"{name}: max-rel {mr:.3e}, frobenius {fr:.3e}"

    def step():  # nothing in a captured step may synchronise
        return _step(q, k, v, dy, sync=False)[:4]

    eager = step()
    graph = capture_step(step)
    for _ in range(3):
        replayed = graph()
    torch.cuda.synchronize()
    ops.check_status(DEV)
    for a, b in zip(eager, replayed):
        assert torch.equal(a, b)


def test_fused_forward_with_running_state_arguments():
    """s_init / s_final with the fused segmented forward, and r_init / r_final with the fused
    backward, against the same call cut into two halves that hand their states over."""
    from flashy_linear_attention_b200 import ops

    B, H, N, D = 1, 3, 4096, 128
    q, k, v, dy = _inputs(B, H, N, D, seed=11)
    half = N // 2
    first = [t[:, :, :half].contiguous() for t in (q, k, v, dy)]
    second = [t[:, :, half:].contiguous() for t in (q, k, v, dy)]
    s_mid = torch.empty(B * H, D, D, dtype=torch.float32, device=DEV)
    s_end = torch.empty_like(s_mid)
    o1 = ops.causal_dot_product_fwd(first[0], first[1], first[2], s_final=s_mid)
    o2 = ops.causal_dot_product_fwd(second[0], second[1], second[2], s_init=s_mid, s_final=s_end)
    s_whole = torch.empty_like(s_mid)
    whole = ops.causal_dot_product_fwd(q, k, v, s_final=s_whole, segments=1)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert _frob(torch.cat([o1, o2], dim=2), whole) < 2e-3
    assert _frob(s_end, s_whole) < 1e-5
    # backward of the second half: needs the prefix state and hands back nothing; of the first half:
    # needs the suffix state R of the second half
    r_mid = torch.empty_like(s_mid)
    g2 = ops.causal_dot_product_bwd(second[3], second[0], second[1], second[2], s_init=s_mid, r_final=r_mid)
    g1 = ops.causal_dot_product_bwd(first[3], first[0], first[1], first[2], r_init=r_mid)
    gw = ops.causal_dot_product_bwd(dy, q, k, v, segments=1)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    for a, b, w in zip(g1, g2, gw):
        assert _frob(torch.cat([a, b], dim=2), w) < 2e-3


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_shapes_segment_counts_and_dtypes_match_the_unsegmented_kernels(seed):
    """Seeded random sweep over heads (1 .. 74), chunk counts, ragged lengths, head dims 32 .. 128,
    automatic and explicit segment counts, bf16 / fp16 and an initial state: whatever form the
    library picks (fused with or without boundary states, three launches, unsegmented) must agree
    with the unsegmented kernels on out, dQ, dK, dV and the final state."""
    import random

    from flashy_linear_attention_b200 import ops

    rng = random.Random(seed)
    ran = 0
    for case in range(60):
        D = rng.choice([64, 128, 128, 96, 32])
        H = rng.choice([1, 2, 3, 5, 7, 8, 12, 16, 20, 24, 31, 40, 49, 64, 74])
        N = rng.choice([2, 3, 5, 8, 17, 18, 24, 33, 40, 64, 65]) * 128 - rng.choice([0, 0, 0, 64])
        if H * N * D > 40e6:
            continue
        segments = rng.choice([0, 0, 0, 2, 3, 4, 7, 9])
        dt = rng.choice([torch.bfloat16, torch.bfloat16, torch.float16])
        with_init = rng.random() < 0.3
        gen = torch.Generator(device=DEV).manual_seed(N * 7 + H)
        q = ((torch.nn.functional.elu(torch.randn(1, H, N, D, device=DEV, generator=gen)) + 1) / D ** 0.5).to(dt)
        k = (torch.nn.functional.elu(torch.randn(1, H, N, D, device=DEV, generator=gen)) + 1).to(dt)
        v = torch.randn(1, H, N, D, device=DEV, generator=gen).to(dt)
        dy = torch.randn(1, H, N, D, device=DEV, generator=gen).to(dt)
        s_init = torch.randn(H, D, D, device=DEV, generator=gen) * 0.1 if with_init else None

        def run(segs, use_states):
            s_final = torch.empty(H, D, D, dtype=torch.float32, device=DEV)
            seg_states = ops.segment_states_buffer(q, v, segs) if use_states else None
            out = ops.causal_dot_product_fwd(q, k, v, s_init=s_init, s_final=s_final, segments=segs,
                                             seg_states=seg_states)
            grads = ops.causal_dot_product_bwd(dy, q, k, v, s_init=s_init, s_last=s_final, segments=segs,
                                               seg_states=seg_states)
            return (out,) + tuple(grads) + (s_final,)

        got, want = run(segments, True), run(1, False)
        torch.cuda.synchronize()
        ops.check_status(DEV)
        label = (case, H, N, D, segments, str(dt), with_init)
        for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
            assert torch.isfinite(a.float()).all(), (label, name)
            assert _frob(a, b) < 1.2e-2, (label, name, _frob(a, b))
        assert _frob(got[4], want[4]) < 1e-4, (label, "s_final", _frob(got[4], want[4]))
        ran += 1
    assert ran >= 40
