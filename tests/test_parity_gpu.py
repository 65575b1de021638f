"""GPU parity tests: the sm_100a kernels, called through the C ABI (via the ctypes wrappers), against
the CPU oracle on the same inputs -- the committed fixtures that came from the reference's own
naive path, seeded inputs at sizes the oracle finishes in seconds, and size-independent
properties at the benchmark's full sizes.

Tolerances (bf16 in / bf16 out, fp32 accumulation):
    max relative error  max|a-b| / max|b|  <= 2e-2     (north-star bound for bf16)
    Frobenius relative error               <  1e-2     (the reference tests' bound, test_attn.py:17)
"""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import linear_attention_oracle as orc

pytestmark = pytest.mark.gpu

MAX_REL_TOL = 2e-2
FROB_TOL = 1e-2
DEV = "cuda:0"


def _ops():
    from flashy_linear_attention_b200 import ops

    return ops


def _to_dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).to(DEV)


def _np(t):
    return t.detach().float().cpu().numpy()


def _check(name, got, want):
    mr = orc.max_rel_error(got, want)
    fr = orc.frobenius_rel_error(got, want)
    assert mr <= MAX_REL_TOL and fr < FROB_TOL, f"{name}: max-rel {mr:.3e}, frobenius {fr:.3e}"


def _run_and_check(q, k, v, dy, segments=0):
    """q, k, v, dy: float32 numpy arrays holding bf16-representable values."""
    ops = _ops()
    tq, tk, tv, tdy = (_to_dev(t) for t in (q, k, v, dy))
    out = ops.causal_dot_product_fwd(tq, tk, tv, segments=segments)
    dq, dk, dv = ops.causal_dot_product_bwd(tdy, tq, tk, tv, segments=segments)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    q64, k64, v64, dy64 = (t.astype(np.float64) for t in (q, k, v, dy))
    _check("out", _np(out), orc.linear_ref(q64, k64, v64))
    rq, rk, rv = orc.linear_ref_grads(q64, k64, v64, dy64)
    _check("dq", _np(dq), rq)
    _check("dk", _np(dk), rk)
    _check("dv", _np(dv), rv)


def _golden_paths():
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    return [p for p in sorted(glob.glob(os.path.join(here, "*.npz"))) if "cfg1" not in p and "denominator" not in p]


@pytest.mark.parametrize("path", _golden_paths(), ids=lambda p: os.path.basename(p)[:-4])
def test_against_reference_fixture(path):
    """Kernel results vs outputs of the reference's naive path stored in the fixture."""
    ops = _ops()
    g = np.load(path)
    q, k, v, dy = (orc.bf16_round(g[n]) for n in ("q", "k", "v", "dy"))
    exact_inputs = all(np.array_equal(orc.bf16_round(g[n]), g[n]) for n in ("q", "k", "v", "dy"))
    tq, tk, tv, tdy = (_to_dev(t) for t in (q, k, v, dy))
    out = ops.causal_dot_product_fwd(tq, tk, tv)
    dq, dk, dv = ops.causal_dot_product_bwd(tdy, tq, tk, tv)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    # fixtures made from fp32 inputs were rounded to bf16 here, which alone costs ~4e-3
    tol_scale = 1.0 if exact_inputs else 1.5
    for name, got in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        mr = orc.max_rel_error(_np(got), g[name])
        assert mr <= MAX_REL_TOL * tol_scale, (name, mr)


def test_cfg1_with_pytorch_denominator():
    """Benchmark configuration 1 (B2 H4 N256 D64, elu+1 inputs): kernel + the README's PyTorch
    denominator, forward and backward through autograd, against the reference fixture."""
    from flashlinear import LinearAttention

    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    g = np.load(os.path.join(here, "ref_cfg1_b2h4_n256_d64_fp32_denominator.npz"))
    B, H, N, dk, dv = (int(x) for x in g["shape"])
    rng = np.random.Generator(np.random.PCG64(int(g["seed"])))
    xq = rng.standard_normal((B, H, N, dk)).astype(np.float32)
    xk = rng.standard_normal((B, H, N, dk)).astype(np.float32)
    v = rng.standard_normal((B, H, N, dv)).astype(np.float32)
    dy = rng.standard_normal((B, H, N, dv)).astype(np.float32)
    q = torch.from_numpy(orc.elu_plus_one(xq)).to(DEV).requires_grad_(True)
    k = torch.from_numpy(orc.elu_plus_one(xk)).to(DEV).requires_grad_(True)
    vv = torch.from_numpy(v).to(DEV).requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        num = LinearAttention.apply(q, k, vv)
    assert num.dtype == torch.bfloat16
    den = (q * k.cumsum(-2)).sum(dim=-1, keepdim=True) + 1e-5  # README.md:29, fp32
    res = num.float() / den
    res.backward(torch.from_numpy(dy).to(DEV))
    torch.cuda.synchronize()
    rows = slice(None, None, int(g["row_stride"]))
    for name, got in (("out", res), ("dq", q.grad), ("dk", k.grad), ("dv", vv.grad)):
        mr = orc.max_rel_error(_np(got)[..., rows, :], g[name])
        assert mr <= MAX_REL_TOL * 1.5, (name, mr)  # fp32 fixture inputs are rounded to bf16 here


SHAPES = [
    # B, H, N, dk, dv
    (1, 1, 64, 64, 64),      # shorter than one chunk
    (1, 1, 128, 128, 128),   # exactly one chunk
    (2, 3, 256, 64, 64),
    (1, 2, 320, 128, 128),   # chunk boundary inside: 128 + 128 + 64
    (1, 2, 192, 32, 32),
    (1, 1, 448, 83, 83),     # odd head dim: padded rows
    (2, 2, 256, 96, 32),     # dk != dv
    (1, 2, 384, 127, 16),
    (1, 1, 1984, 128, 128),  # longest sequence of the reference's tests
    (3, 31, 64, 16, 16),
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_seeded_inputs_against_oracle(shape):
    B, H, N, dk, dv = shape
    rng = np.random.default_rng(hash(shape) % (2 ** 31))
    q = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk)).astype(np.float32)))
    k = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk)).astype(np.float32)))
    v = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    dy = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    _run_and_check(q, k, v, dy)


@pytest.mark.parametrize("shape", [(1, 2, 256, 256, 256), (1, 2, 192, 200, 136), (2, 2, 256, 273, 64),
                                   (1, 1, 128, 384, 64), (1, 2, 640, 273, 32), (2, 1, 320, 144, 16),
                                   (1, 2, 1152, 256, 64), (1, 1, 448, 330, 64), (1, 2, 384, 256, 128),
                                   (2, 2, 512, 160, 192), (1, 1, 320, 96, 256), (1, 1, 256, 384, 384)],
                         ids=lambda s: "x".join(map(str, s)))
def test_head_dims_above_the_kernel_tile(shape):
    """Head dims above 128 (the reference allows up to 256, flashlinear/kernels/
    linear_attn_kernels.py:322; benchmark configuration 4 uses 273 Taylor features), every
    combination up to 384 inside ONE library call per pass: a/b wider than 128 run in the wide
    kernel, whose c/out side is cut into 64-column launches when it is wider than that; c/out
    wider than 128 with a/b at most 128 run as 128-column slices of one grid. Same tolerance."""
    B, H, N, dk, dv = shape
    rng = np.random.default_rng(dk * 1000 + dv)
    # scaled so that the scores stay O(1) at these widths
    q = orc.bf16_round((orc.elu_plus_one(rng.standard_normal((B, H, N, dk))) / np.sqrt(dk)).astype(np.float32))
    k = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk))).astype(np.float32))
    v = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    dy = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    _run_and_check(q, k, v, dy)


def test_taylor_feature_configuration_through_the_function():
    """Benchmark configuration 4 in miniature: raw 16-dim q, k -> 273 second-order Taylor features
    -> LinearAttentionSmallVHD with dv = 64, forward and backward, against the oracle."""
    from flashlinear import LinearAttentionSmallVHD

    rng = np.random.default_rng(4)
    B, H, N = 1, 2, 384
    q = orc.bf16_round(orc.taylor_feature_map(rng.standard_normal((B, H, N, 16))).astype(np.float32))
    k = orc.bf16_round(orc.taylor_feature_map(rng.standard_normal((B, H, N, 16))).astype(np.float32))
    v = orc.bf16_round(rng.standard_normal((B, H, N, 64)).astype(np.float32))
    dy = orc.bf16_round(rng.standard_normal((B, H, N, 64)).astype(np.float32))
    tq, tk, tv = (_to_dev(t).requires_grad_(True) for t in (q, k, v))
    out = LinearAttentionSmallVHD.apply(tq, tk, tv)
    out.backward(_to_dev(dy))
    torch.cuda.synchronize()
    q64, k64, v64, dy64 = (t.astype(np.float64) for t in (q, k, v, dy))
    _check("out", _np(out), orc.linear_ref(q64, k64, v64))
    rq, rk, rv = orc.linear_ref_grads(q64, k64, v64, dy64)
    _check("dq", _np(tq.grad), rq)
    _check("dk", _np(tk.grad), rk)
    _check("dv", _np(tv.grad), rv)


@pytest.mark.parametrize("rows,d", [(1000, 273), (77, 17), (5, 1), (4096, 83), (33, 9), (64, 271)],
                         ids=lambda x: str(x))
def test_row_padding_kernels_are_bit_exact(rows, d):
    """fla_sm100_pad_rows / fla_sm100_unpad_rows: byte-for-byte copies, zero padding, round trip."""
    ops = _ops()
    t = torch.randn(rows, d, device=DEV).to(torch.bfloat16).reshape(1, 1, rows, d)
    v = ops.kernel_view(t)
    dpad = v.stride(2)
    assert dpad % 8 == 0 and dpad >= d and v.data_ptr() % 16 == 0
    whole = v.as_strided((rows, dpad), (dpad, 1))
    back = torch.full_like(t, float("nan"))
    ops._copy_back(back, v)
    torch.cuda.synchronize()
    assert torch.equal(whole[:, :d].view(torch.int16), t.view(rows, d).view(torch.int16))
    assert bool((whole[:, d:].view(torch.int16) == 0).all())
    assert torch.equal(back.view(torch.int16), t.view(torch.int16))


def test_smallv_function_returns_reference_values_for_unaligned_head_dim():
    """dk = 273: the Function repacks q and k once and returns dQ, dK as views of padded rows; the
    wrappers return contiguous gradients like the reference's. Both carry the same values."""
    from flashlinear import LinearAttentionSmallVHD
    from flashlinear.kernels import linear_flash_wrapper_bwd_smallv_hd, linear_flash_wrapper_fwd_smallv_hd

    ops = _ops()
    torch.manual_seed(3)
    B, H, N, dk, dv = 2, 2, 256, 273, 64
    q = (torch.nn.functional.softplus(torch.randn(B, H, N, dk, device=DEV)) / dk ** 0.5).to(torch.bfloat16)
    k = torch.nn.functional.softplus(torch.randn(B, H, N, dk, device=DEV)).to(torch.bfloat16)
    v = torch.randn(B, H, N, dv, device=DEV).to(torch.bfloat16)
    dy = torch.randn(B, H, N, dv, device=DEV).to(torch.bfloat16)
    out_w = linear_flash_wrapper_fwd_smallv_hd(q, k, v)
    gq_w, gk_w, gv_w = linear_flash_wrapper_bwd_smallv_hd(dy, q, k, v)
    assert gq_w.is_contiguous() and gk_w.is_contiguous() and out_w.is_contiguous()
    q_, k_, v_ = (t.clone().requires_grad_(True) for t in (q, k, v))
    out_f = LinearAttentionSmallVHD.apply(q_, k_, v_)
    gq_f, gk_f, gv_f = torch.autograd.grad(out_f, (q_, k_, v_), dy)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert gq_f.shape == q.shape and gk_f.shape == k.shape
    for a, b in ((out_w, out_f), (gq_w, gq_f), (gk_w, gk_f), (gv_w, gv_f)):
        assert torch.equal(a, b)
    q_.grad = None
    out_f2 = LinearAttentionSmallVHD.apply(q_, k_, v_)
    out_f2.backward(dy)  # accumulation into .grad accepts the padded-row views
    assert torch.equal(q_.grad, gq_w) and torch.equal(k_.grad, gk_w)


@pytest.mark.parametrize("segments", [2, 3, 8])
def test_segmented_equals_oracle(segments):
    rng = np.random.default_rng(segments)
    B, H, N, d = 1, 2, 1536, 64
    q = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, d)).astype(np.float32)))
    k = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, d)).astype(np.float32)))
    v = orc.bf16_round(rng.standard_normal((B, H, N, d)).astype(np.float32))
    dy = orc.bf16_round(rng.standard_normal((B, H, N, d)).astype(np.float32))
    _run_and_check(q, k, v, dy, segments=segments)


@pytest.mark.parametrize("shape", [(1, 1, 128, 128, 128), (2, 2, 576, 64, 64), (1, 3, 1024, 128, 128), (1, 2, 320, 96, 32),
                                   (1, 2, 2304, 128, 128)],
                         ids=lambda s: "x".join(map(str, s)))
def test_single_sweep_backward_with_forward_state(shape):
    """Backward given the forward's final state (s_last): dQ is computed in the same descending
    sweep as dK, dV from "total minus suffix" states. Same tolerance as the ordinary backward.
    The library keeps that form for sequences above 2048 tokens; the debug flag lifts the rule so
    that short sequences exercise it too."""
    from flashy_linear_attention_b200 import _lib
    ops = _ops()
    old_flags = ops.set_debug_flags(_lib.FLA_DEBUG_FORCE_SINGLE_SWEEP)
    try:
        _single_sweep_case(ops, shape)
    finally:
        ops.set_debug_flags(old_flags)


def _single_sweep_case(ops, shape):
    B, H, N, dk, dv = shape
    rng = np.random.default_rng(N + dk)
    q = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk)).astype(np.float32)))
    k = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk)).astype(np.float32)))
    v = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    dy = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    tq, tk, tv, tdy = (_to_dev(t) for t in (q, k, v, dy))
    s_state = torch.empty(B * H, dk, dv, dtype=torch.float32, device=DEV)
    ops.causal_dot_product_fwd(tq, tk, tv, s_final=s_state, segments=1)
    dq, dk_, dv_ = ops.causal_dot_product_bwd(tdy, tq, tk, tv, s_last=s_state, segments=1)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    rq, rk, rv = orc.linear_ref_grads(*(t.astype(np.float64) for t in (q, k, v, dy)))
    _check("dq", _np(dq), rq)
    _check("dk", _np(dk_), rk)
    _check("dv", _np(dv_), rv)


def test_kernel_rounding_matches_emulated_rounding_tightly():
    """Against the oracle's emulation of the kernel's own rounding points the difference is only
    summation order inside the MMAs: far below the bf16 tolerance."""
    ops = _ops()
    rng = np.random.default_rng(99)
    B, H, N, d = 1, 2, 512, 64
    q = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, d)).astype(np.float32)))
    k = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, d)).astype(np.float32)))
    v = orc.bf16_round(rng.standard_normal((B, H, N, d)).astype(np.float32))
    out = ops.causal_dot_product_fwd(_to_dev(q), _to_dev(k), _to_dev(v))
    emu, _ = orc.chunked_fwd(q, k, v, chunk=128, emulate_bf16=True)
    # elements may differ by one bf16 ulp where the fp32 sums straddle a rounding boundary
    assert orc.frobenius_rel_error(_np(out), emu) < 2e-3
    assert orc.max_rel_error(_np(out), emu) < 8e-3


def test_running_state_arguments():
    """fwd(N) == fwd(first half) then fwd(second half, s_init); same for the backward with R."""
    ops = _ops()
    rng = np.random.default_rng(5)
    B, H, N, d = 2, 2, 512, 128
    h = 256
    mk = lambda a: _to_dev(orc.bf16_round(a.astype(np.float32)))
    q = mk(orc.elu_plus_one(rng.standard_normal((B, H, N, d))))
    k = mk(orc.elu_plus_one(rng.standard_normal((B, H, N, d))))
    v = mk(rng.standard_normal((B, H, N, d)))
    dy = mk(rng.standard_normal((B, H, N, d)))
    full = ops.causal_dot_product_fwd(q, k, v)
    fq, fk, fv = ops.causal_dot_product_bwd(dy, q, k, v)
    s_mid = torch.empty(B * H, d, d, dtype=torch.float32, device=DEV)
    q1, k1, v1, dy1 = (t[:, :, :h].contiguous() for t in (q, k, v, dy))
    q2, k2, v2, dy2 = (t[:, :, h:].contiguous() for t in (q, k, v, dy))
    o1 = ops.causal_dot_product_fwd(q1, k1, v1, s_final=s_mid)
    o2 = ops.causal_dot_product_fwd(q2, k2, v2, s_init=s_mid)
    # state read-out equals the state-only entry point and the oracle
    s_only = ops.chunk_state(k1, v1)
    want_s = np.matmul(np.swapaxes(_np(k1).astype(np.float64), -1, -2), _np(v1).astype(np.float64)).reshape(B * H, d, d)
    assert orc.max_rel_error(_np(s_mid), want_s) < 1e-4
    assert orc.max_rel_error(_np(s_only), want_s) < 1e-4
    r_mid = torch.empty(B * H, d, d, dtype=torch.float32, device=DEV)
    dq2, dk2, dv2 = ops.causal_dot_product_bwd(dy2, q2, k2, v2, s_init=s_mid, r_final=r_mid)
    dq1, dk1, dv1 = ops.causal_dot_product_bwd(dy1, q1, k1, v1, r_init=r_mid)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    # the split run equals the unsplit one (the state is carried in fp32)
    for a, b, full_t in ((o1, o2, full), (dq1, dq2, fq), (dk1, dk2, fk), (dv1, dv2, fv)):
        got = torch.cat([a, b], dim=2)
        assert orc.frobenius_rel_error(_np(got), _np(full_t)) < 2e-3


@pytest.mark.parametrize("segments", [1, 4])
def test_forward_reuses_segment_states_of_the_state_pass(segments):
    """chunk_state(keep_workspace) -> forward(segment_workspace, s_init): the sequence-sharded
    forward's way of not reading k, v a third time. Must equal the plain forward with s_init."""
    ops = _ops()
    torch.manual_seed(3)
    B, H, N, d = 1, 3, 2048, 128
    q = torch.nn.functional.softplus(torch.randn(B, H, N, d, device=DEV)).to(torch.bfloat16)
    k = torch.nn.functional.softplus(torch.randn(B, H, N, d, device=DEV)).to(torch.bfloat16)
    v = torch.randn(B, H, N, d, device=DEV).to(torch.bfloat16)
    prefix = torch.randn(B * H, d, d, device=DEV)
    want = ops.causal_dot_product_fwd(q, k, v, s_init=prefix, segments=segments)
    state, ws = ops.chunk_state(k, v, segments=segments, keep_workspace=True)
    got = ops.causal_dot_product_fwd(q, k, v, s_init=prefix, segments=segments,
                                     segment_workspace=ws if ws.numel() else None)
    got0 = ops.causal_dot_product_fwd(q, k, v, segments=segments, segment_workspace=ws if ws.numel() else None)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    want_state = torch.matmul(k.float().transpose(-1, -2), v.float()).reshape(B * H, d, d)
    assert (torch.linalg.norm(state - want_state) / torch.linalg.norm(want_state)).item() < 1e-4
    assert (torch.linalg.norm(got.float() - want.float()) / torch.linalg.norm(want.float())).item() < 2e-3
    plain = ops.causal_dot_product_fwd(q, k, v, segments=segments)
    assert (torch.linalg.norm(got0.float() - plain.float()) / torch.linalg.norm(plain.float())).item() < 2e-3


def test_strided_and_offset_inputs():
    """Per-tensor strides: q from a fused [B,N,3,H,D] projection, transposed v, expanded grad."""
    ops = _ops()
    torch.manual_seed(0)
    B, H, N, d = 2, 3, 256, 64
    qkv = torch.randn(B, N, 3, H, d, device=DEV).to(torch.bfloat16)
    q = torch.nn.functional.softplus(qkv[:, :, 0]).transpose(1, 2)
    k = torch.nn.functional.softplus(qkv[:, :, 1]).transpose(1, 2)
    v = qkv[:, :, 2].transpose(1, 2)          # non-contiguous view, stride_n = 3*H*d
    assert not v.is_contiguous()
    out = ops.causal_dot_product_fwd(q, k, v)
    ref = ops.causal_dot_product_fwd(q.contiguous(), k.contiguous(), v.contiguous())
    assert torch.equal(out, ref)
    dy = torch.randn(1, 1, N, d, device=DEV).to(torch.bfloat16).expand(B, H, N, d)  # zero strides
    g1 = ops.causal_dot_product_bwd(dy, q, k, v)
    g2 = ops.causal_dot_product_bwd(dy.contiguous(), q.contiguous(), k.contiguous(), v.contiguous())
    for a, b in zip(g1, g2):
        assert torch.equal(a, b)
    qn = _np(q).astype(np.float64); kn = _np(k).astype(np.float64); vn = _np(v).astype(np.float64)
    _check("out", _np(out), orc.linear_ref(qn, kn, vn))


def test_autocast_and_dtype_behaviour():
    """custom_fwd(cast_inputs=bf16): fp32 inputs are cast under autocast (linear_attn.py:13);
    outside autocast a non-bf16 input is an error rather than a silent wrong result."""
    from flashlinear import LinearAttention

    q = torch.rand(1, 2, 128, 64, device=DEV, requires_grad=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = LinearAttention.apply(q, q, q)
    assert out.dtype == torch.bfloat16
    out.float().sum().backward()
    assert q.grad is not None and q.grad.dtype == torch.float32
    with pytest.raises(TypeError):
        LinearAttention.apply(q, q, q)


def test_outputs_are_fully_written():
    """NaN-poisoned allocator blocks must be completely overwritten by the kernels."""
    ops = _ops()
    B, H, N, d = 1, 3, 320, 64
    poison = torch.full((B, H, N, d), float("nan"), device=DEV, dtype=torch.bfloat16)
    del poison  # returns the block to the caching allocator; empty_like below reuses it
    q = torch.rand(B, H, N, d, device=DEV).to(torch.bfloat16)
    out = ops.causal_dot_product_fwd(q, q, q)
    dq, dk, dv = ops.causal_dot_product_bwd(q, q, q, q)
    for t in (out, dq, dk, dv):
        assert not torch.isnan(t.float()).any()


@pytest.mark.parametrize("cfg", [(8, 16, 4096, 64), (4, 32, 8192, 128)], ids=["cfg2", "cfg3"])
def test_full_size_properties(cfg):
    """Benchmark sizes, checked through properties that need no O(N^2) oracle:
    (1) with q = all-ones the product collapses to a cumulative sum, out_i = cumsum_j (sum_d k_jd) v_j;
    (2) linearity in v; (3) segmented == unsegmented; (4) one head against the naive oracle path."""
    ops = _ops()
    B, H, N, d = cfg
    gen = torch.Generator(device=DEV).manual_seed(1)
    k = (torch.nn.functional.elu(torch.randn(B, H, N, d, device=DEV, generator=gen)) + 1).to(torch.bfloat16)
    q = (torch.nn.functional.elu(torch.randn(B, H, N, d, device=DEV, generator=gen)) + 1).to(torch.bfloat16)
    v = torch.randn(B, H, N, d, device=DEV, generator=gen).to(torch.bfloat16)
    ones = torch.ones_like(q)
    out1 = ops.causal_dot_product_fwd(ones, k, v)
    want1 = torch.cumsum(k.float().sum(-1, keepdim=True).double() * v.double(), dim=2)
    rel = ((out1.double() - want1).abs().max() / want1.abs().max()).item()
    assert rel <= MAX_REL_TOL, rel
    out = ops.causal_dot_product_fwd(q, k, v)
    out_neg = ops.causal_dot_product_fwd(q, k, -v)
    assert torch.equal(out, -out_neg)
    v2 = torch.randn(B, H, N, d, device=DEV, generator=gen).to(torch.bfloat16)
    lhs = ops.causal_dot_product_fwd(q, k, (v.float() + v2.float()).to(torch.bfloat16)).float()
    rhs = out.float() + ops.causal_dot_product_fwd(q, k, v2).float()
    assert (torch.linalg.norm(lhs - rhs) / torch.linalg.norm(rhs)).item() < FROB_TOL
    seg = ops.causal_dot_product_fwd(q, k, v, segments=4)
    assert (torch.linalg.norm(seg.float() - out.float()) / torch.linalg.norm(out.float())).item() < 2e-3
    dy = torch.randn(B, H, N, d, device=DEV, generator=gen).to(torch.bfloat16)
    s_state = torch.empty(B * H, d, d, dtype=torch.float32, device=DEV)
    ops.causal_dot_product_fwd(q, k, v, s_final=s_state)
    dq, dk, dv = ops.causal_dot_product_bwd(dy, q, k, v, s_last=s_state)   # single-sweep form
    dq2, dk2, dv2 = ops.causal_dot_product_bwd(dy, q, k, v)                # two-direction form
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert (torch.linalg.norm(dq.float() - dq2.float()) / torch.linalg.norm(dq2.float())).item() < FROB_TOL
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2)
    # one head, full length, against the oracle (naive O(N^2) path on the CPU)
    b, h = B - 1, H - 1
    qs, ks, vs, dys = (_np(t[b, h]).astype(np.float64) for t in (q, k, v, dy))
    _check("out[head]", _np(out[b, h]), orc.linear_ref(qs, ks, vs))
    rq, rk, rv = orc.linear_ref_grads(qs, ks, vs, dys)
    _check("dq[head]", _np(dq[b, h]), rq)
    _check("dk[head]", _np(dk[b, h]), rk)
    _check("dv[head]", _np(dv[b, h]), rv)


@pytest.mark.parametrize("shape,heads_per_slab", [((2, 5, 512, 64, 64), 3), ((1, 4, 1024, 128, 128), 16),
                                                  ((2, 3, 256, 96, 32), 2)],
                         ids=["ragged-slabs", "one-slab", "smallv"])
def test_host_pipeline_equals_oracle_and_device_path(shape, heads_per_slab):
    """Pinned host tensors streamed in slabs of heads give what the device-resident call gives."""
    from flashy_linear_attention_b200.host import HostPipeline

    ops = _ops()
    B, H, N, dk, dv = shape
    rng = np.random.default_rng(7)
    q = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk))).astype(np.float32))
    k = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk))).astype(np.float32))
    v = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    dy = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    host_in = [torch.from_numpy(a).to(torch.bfloat16).pin_memory() for a in (q, k, v, dy)]
    host_out = [torch.full(s, float("nan"), dtype=torch.bfloat16).pin_memory()
                for s in ((B, H, N, dv), (B, H, N, dk), (B, H, N, dk), (B, H, N, dv))]
    pipe = HostPipeline(DEV, heads_per_slab=heads_per_slab, depth=2)
    for _ in range(2):  # the second call reuses the staging buffers
        pipe.fwd_bwd(*host_in, *host_out)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    q64, k64, v64, dy64 = (t.astype(np.float64) for t in (q, k, v, dy))
    want = (orc.linear_ref(q64, k64, v64),) + tuple(orc.linear_ref_grads(q64, k64, v64, dy64))
    for name, got, ref in zip(("out", "dq", "dk", "dv"), host_out, want):
        assert not torch.isnan(got.float()).any(), f"{name}: rows left unwritten"
        _check(name, got.float().numpy(), ref)
    tq, tk, tv, tdy = (t.to(DEV) for t in host_in)
    dev_out = ops.causal_dot_product_fwd(tq, tk, tv)
    _check("out vs device-resident call", host_out[0].float().numpy(), _np(dev_out))
    with pytest.raises(ValueError):
        pipe.fwd_bwd(host_in[0].clone(), *host_in[1:], *host_out)  # not pinned


@pytest.mark.parametrize("shape", [(2, 2, 512, 128, 128), (1, 3, 384, 64, 64), (1, 2, 256, 96, 32)],
                         ids=lambda s: "x".join(map(str, s)))
def test_resumable_function_carries_state_and_gradients(shape):
    """Two calls chained through the state (and autograd through it) equal one call on all tokens."""
    from flashy_linear_attention_b200 import LinearAttentionResumable

    ops = _ops()
    B, H, N, dk, dv = shape
    h = N // 2 if (N // 2) % 64 == 0 else 64
    rng = np.random.default_rng(11)
    q = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk))).astype(np.float32))
    k = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk))).astype(np.float32))
    v = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    dy = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    tq, tk, tv, tdy = (_to_dev(t).requires_grad_(True) for t in (q, k, v, dy))
    o1, s1 = LinearAttentionResumable.apply(tq[:, :, :h], tk[:, :, :h], tv[:, :, :h], None)
    o2, s2 = LinearAttentionResumable.apply(tq[:, :, h:], tk[:, :, h:], tv[:, :, h:], s1)
    out = torch.cat([o1, o2], dim=2)
    assert s2.dtype == torch.float32 and tuple(s2.shape) == (B, H, dk, dv)
    gq, gk, gv = torch.autograd.grad(out, (tq, tk, tv), tdy.detach())
    torch.cuda.synchronize()
    ops.check_status(DEV)
    q64, k64, v64, dy64 = (t.astype(np.float64) for t in (q, k, v, dy))
    _check("out", _np(out), orc.linear_ref(q64, k64, v64))
    rq, rk, rv = orc.linear_ref_grads(q64, k64, v64, dy64)
    _check("dq", _np(gq), rq)
    _check("dk", _np(gk), rk)
    _check("dv", _np(gv), rv)
    want_s = np.matmul(np.swapaxes(k64, -1, -2), v64)
    assert orc.max_rel_error(_np(s2), want_s) < 1e-4
    # a loss on the state alone: d/dk sum(s_final * W) = v W^T, d/dv = k W
    w = torch.from_numpy(rng.standard_normal((B, H, dk, dv)).astype(np.float32)).to(DEV)
    _, s = LinearAttentionResumable.apply(tq, tk, tv, None)
    gk2, gv2 = torch.autograd.grad((s * w).sum(), (tk, tv))
    _check("dk from the state", _np(gk2), np.matmul(v64, np.swapaxes(w.double().cpu().numpy(), -1, -2)))
    _check("dv from the state", _np(gv2), np.matmul(k64, w.double().cpu().numpy()))


def test_normalized_function_against_the_reference_denominator_fixture():
    """LinearAttentionNormalized (product + denominator kernels) against the fixture that holds the
    reference's naive path followed by the README's denominator (README.md:27-30), cfg1."""
    from flashy_linear_attention_b200 import LinearAttentionNormalized

    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    g = np.load(os.path.join(here, "ref_cfg1_b2h4_n256_d64_fp32_denominator.npz"))
    B, H, N, dk, dv = (int(x) for x in g["shape"])
    rng = np.random.Generator(np.random.PCG64(int(g["seed"])))
    xq = rng.standard_normal((B, H, N, dk)).astype(np.float32)
    xk = rng.standard_normal((B, H, N, dk)).astype(np.float32)
    v = rng.standard_normal((B, H, N, dv)).astype(np.float32)
    dy = rng.standard_normal((B, H, N, dv)).astype(np.float32)
    q = torch.from_numpy(orc.elu_plus_one(xq)).to(DEV).requires_grad_(True)
    k = torch.from_numpy(orc.elu_plus_one(xk)).to(DEV).requires_grad_(True)
    vv = torch.from_numpy(v).to(DEV).requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        res = LinearAttentionNormalized.apply(q, k, vv, 1e-5)
    assert res.dtype == torch.bfloat16
    res.backward(torch.from_numpy(dy).to(DEV).to(torch.bfloat16))
    torch.cuda.synchronize()
    _ops().check_status(DEV)
    rows = slice(None, None, int(g["row_stride"]))
    for name, got in (("out", res), ("dq", q.grad), ("dk", k.grad), ("dv", vv.grad)):
        mr = orc.max_rel_error(_np(got)[..., rows, :], g[name])
        assert mr <= MAX_REL_TOL * 1.5, (name, mr)  # fp32 fixture inputs are rounded to bf16 here


@pytest.mark.parametrize("shape", [(1, 2, 512, 128, 128), (2, 3, 320, 64, 64), (1, 2, 256, 96, 32),
                                   (1, 2, 256, 273, 64), (1, 1, 192, 83, 16), (1, 1, 2048, 128, 128)],
                         ids=lambda s: "x".join(map(str, s)))
def test_normalized_function_against_oracle(shape):
    """Forward and all three gradients of the normalised attention vs the closed-form oracle."""
    from flashy_linear_attention_b200 import LinearAttentionNormalized

    B, H, N, dk, dv = shape
    rng = np.random.default_rng(dk + 7 * dv)
    q = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk))).astype(np.float32))
    k = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk))).astype(np.float32))
    v = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    dy = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    tq, tk, tv = (_to_dev(t).requires_grad_(True) for t in (q, k, v))
    out = LinearAttentionNormalized.apply(tq, tk, tv, 1e-5)
    gq, gk, gv = torch.autograd.grad(out, (tq, tk, tv), _to_dev(dy))
    torch.cuda.synchronize()
    _ops().check_status(DEV)
    q64, k64, v64, dy64 = (t.astype(np.float64) for t in (q, k, v, dy))
    _check("out", _np(out), orc.normalised_ref(q64, k64, v64))
    rq, rk, rv = orc.normalised_ref_grads(q64, k64, v64, dy64)
    _check("dv", _np(gv), rv)
    # dQ and dK of the normalised attention are the SUM of the product's gradient (rounded to bf16
    # by the product kernels, as in the reference's recipe) and the denominator's part, which
    # largely cancel: |product part| is 2-6 x |sum| at these shapes, and so is the amplification of
    # the product's 2e-3 rounding error. Tolerance for these two: twice the usual.
    for name, got, want in (("dq", gq, rq), ("dk", gk, rk)):
        mr = orc.max_rel_error(_np(got), want)
        fr = orc.frobenius_rel_error(_np(got), want)
        assert mr <= 2 * MAX_REL_TOL and fr < 2 * FROB_TOL, f"{name}: max-rel {mr:.3e}, frobenius {fr:.3e}"
    # the denominator itself, fp32: q . cumsum(k) + eps
    ops = _ops()
    qv, kv = ops.kernel_view(_to_dev(q)), ops.kernel_view(_to_dev(k))
    num = torch.ones(B, H, N, 8, dtype=torch.bfloat16, device=DEV)
    den = ops.normalize_fwd(qv, kv, num, 1e-5)
    torch.cuda.synchronize()
    assert orc.max_rel_error(_np(den).reshape(B, H, N, 1), orc.denominator(q64, k64)) < 1e-5


@pytest.mark.parametrize("d", [8, 16])
def test_taylor_feature_kernels_against_oracle(d):
    """Feature map and its gradient kernel vs the numpy restatement (bf16 outputs, fp32 math)."""
    ops = _ops()
    rng = np.random.default_rng(d)
    B, H, N = 2, 3, 200  # 1200 rows: not a multiple of the backward kernel's 128-row tiles
    x = orc.bf16_round(rng.standard_normal((B, H, N, d)).astype(np.float32))
    tx = _to_dev(x)
    phi = ops.taylor_features(tx)
    F = 1 + d + d * d
    assert tuple(phi.shape) == (B, H, N, F) and phi.stride(2) % 8 == 0 and phi.stride(2) >= F
    want = orc.taylor_feature_map(x.astype(np.float64))
    assert orc.max_rel_error(_np(phi), want) <= 2.0 ** -8
    whole = phi.as_strided((B * H * N, phi.stride(2)), (phi.stride(2), 1))
    assert bool((whole[:, F:] == 0).all())
    dphi = orc.bf16_round(rng.standard_normal((B, H, N, F)).astype(np.float32))
    tdphi = torch.zeros_like(whole).view(B, H, N, -1)
    tdphi[..., :F] = _to_dev(dphi)
    dx = ops.taylor_features_bwd(tdphi[..., :F], tx)
    dx2 = ops.taylor_features_bwd(_to_dev(dphi), tx)  # contiguous gradient: brought into padded rows first
    torch.cuda.synchronize()
    want_dx = orc.taylor_feature_map_grad(x.astype(np.float64), dphi.astype(np.float64))
    assert orc.max_rel_error(_np(dx), want_dx) <= 2.0 ** -7
    assert torch.equal(dx, dx2)


@pytest.mark.parametrize("shape", [(1, 2, 384, 16, 64), (2, 2, 256, 16, 32), (1, 2, 320, 8, 64)],
                         ids=lambda s: "x".join(map(str, s)))
def test_taylor_attention_function_against_oracle(shape):
    """Raw q, k -> Taylor features -> causal product, forward and gradients w.r.t. the RAW inputs."""
    from flashy_linear_attention_b200 import TaylorLinearAttention

    B, H, N, d, dv = shape
    rng = np.random.default_rng(31 * d + dv)
    xq = orc.bf16_round(rng.standard_normal((B, H, N, d)).astype(np.float32))
    xk = orc.bf16_round(rng.standard_normal((B, H, N, d)).astype(np.float32))
    v = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    dy = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    tq, tk, tv = (_to_dev(t).requires_grad_(True) for t in (xq, xk, v))
    out = TaylorLinearAttention.apply(tq, tk, tv)
    gq, gk, gv = torch.autograd.grad(out, (tq, tk, tv), _to_dev(dy))
    torch.cuda.synchronize()
    _ops().check_status(DEV)
    q64, k64, v64, dy64 = (t.astype(np.float64) for t in (xq, xk, v, dy))
    pq, pk = orc.taylor_feature_map(q64), orc.taylor_feature_map(k64)
    _check("out", _np(out), orc.linear_ref(pq, pk, v64))
    dpq, dpk, rv = orc.linear_ref_grads(pq, pk, v64, dy64)
    _check("dv", _np(gv), rv)
    _check("dxq", _np(gq), orc.taylor_feature_map_grad(q64, dpq))
    _check("dxk", _np(gk), orc.taylor_feature_map_grad(k64, dpk))


@pytest.mark.parametrize("shape", [(1, 4, 1024, 128, 128), (2, 16, 512, 64, 64)], ids=["segmented", "one-wave"])
def test_cuda_graph_capture_replays_the_same_results(shape):
    """The entry points only enqueue work, so a forward + backward over fixed buffers can be captured
    in a CUDA graph; a replay after the inputs changed in place gives what an eager call gives."""
    from flashy_linear_attention_b200.graphs import capture_step

    ops = _ops()
    B, H, N, dk, dv = shape
    torch.manual_seed(5)
    q = (torch.nn.functional.elu(torch.randn(B, H, N, dk, device=DEV)) + 1).to(torch.bfloat16)
    k = (torch.nn.functional.elu(torch.randn(B, H, N, dk, device=DEV)) + 1).to(torch.bfloat16)
    v = torch.randn(B, H, N, dv, device=DEV).to(torch.bfloat16)
    dy = torch.randn(B, H, N, dv, device=DEV).to(torch.bfloat16)

    def step():
        return (ops.causal_dot_product_fwd(q, k, v),) + tuple(ops.causal_dot_product_bwd(dy, q, k, v))

    captured = capture_step(step)
    v.copy_(torch.randn_like(v))  # new data in the same buffers
    dy.copy_(torch.randn_like(dy))
    got = [t.clone() for t in captured()]
    want = step()
    torch.cuda.synchronize()
    ops.check_status(DEV)
    for a, b in zip(got, want):
        assert torch.equal(a, b)


@pytest.mark.parametrize("shape", [(1, 2, 100, 64, 64), (2, 1, 1, 128, 128), (1, 1, 129, 128, 128), (1, 2, 250, 96, 32),
                                   (1, 1, 200, 273, 64)], ids=lambda s: "x".join(map(str, s)))
def test_ragged_sequence_lengths_below_the_wrappers_granularity(shape):
    """The reference wrappers insist on multiples of 64 tokens (linear_attn_kernels.py:323-325); the
    kernels themselves take any length: out-of-range tokens of the last chunk read as zero and are
    not written."""
    B, H, N, dk, dv = shape
    rng = np.random.default_rng(N)
    q = orc.bf16_round((orc.elu_plus_one(rng.standard_normal((B, H, N, dk))) / np.sqrt(dk / 64)).astype(np.float32))
    k = orc.bf16_round(orc.elu_plus_one(rng.standard_normal((B, H, N, dk))).astype(np.float32))
    v = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    dy = orc.bf16_round(rng.standard_normal((B, H, N, dv)).astype(np.float32))
    _run_and_check(q, k, v, dy)
