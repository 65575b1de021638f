"""CPU tests of the host side: the C-ABI library loads and exports every symbol the header
declares, argument errors are reported before any launch, and the Python wrappers keep the
reference's preconditions and refuse to run without a GPU (there is no CPU fallback)."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from flashy_linear_attention_b200 import _lib

    header = open(os.path.join(ROOT, "include", "flashlinear_sm100.h")).read()
    declared = sorted(set(re.findall(r"\b(fla_sm100_\w+)\s*\(", header)))
    assert declared, "no declarations found in the header"
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/flashlinear_sm100.h but not exported"
    assert set(declared) == set(_lib.EXPORTED_SYMBOLS)
    assert lib.fla_sm100_abi_version() == _lib.FLA_ABI_VERSION
    assert b"16" in lib.fla_sm100_strerror(-3)


def test_struct_layout_matches_header():
    # field order and count of FlaArgs in the header vs the ctypes mirror
    from flashy_linear_attention_b200._lib import FlaArgs, FlaTensor

    assert ctypes.sizeof(FlaTensor) == 32
    names = [f[0] for f in FlaArgs._fields_]
    header = open(os.path.join(ROOT, "include", "flashlinear_sm100.h")).read()
    body = header[header.index("typedef struct FlaArgs {"):header.index("} FlaArgs;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    decl = []
    for stmt in body.split(";"):
        stmt = stmt.replace("typedef struct FlaArgs {", "").strip()
        if not stmt:
            continue
        parts = stmt.replace("*", " ").split(",")
        first = parts[0].split()
        decl.append(first[-1])
        decl.extend(p.strip() for p in parts[1:])
    assert decl == names


def test_invalid_arguments_are_rejected_without_a_gpu():
    from flashy_linear_attention_b200 import _lib
    from flashy_linear_attention_b200._lib import FlaArgs

    lib = _lib.load()
    assert lib.fla_sm100_fwd(None) == -1
    a = FlaArgs()
    assert lib.fla_sm100_fwd(ctypes.byref(a)) == -1  # zero sizes
    assert lib.fla_sm100_bwd(ctypes.byref(a)) == -1
    a.batch, a.heads, a.seqlen, a.dk, a.dv = 1, 1, 128, 64, 64
    if not torch.cuda.is_available():
        # valid sizes but no usable device: a CUDA / device error, never a crash
        assert lib.fla_sm100_fwd(ctypes.byref(a)) in (-4, -6)
    # workspace query is pure host arithmetic
    a.batch, a.heads, a.seqlen, a.dk, a.dv, a.segments = 1, 2, 4096, 128, 128, 4
    need = lib.fla_sm100_workspace_bytes(ctypes.byref(a), 0)
    assert need >= 2 * 4 * 128 * 128 * 4
    a.segments = 1
    assert lib.fla_sm100_workspace_bytes(ctypes.byref(a), 0) == 0
    # more (batch, head) pairs than a grid dimension holds: refused before any device work
    big = FlaArgs()
    big.batch, big.heads, big.seqlen, big.dk, big.dv = 1024, 64, 128, 64, 64
    assert lib.fla_sm100_fwd(ctypes.byref(big)) == -2
    assert lib.fla_sm100_bwd(ctypes.byref(big)) == -2
    # the wide (SmallVHD) shapes never split the sequence: no scratch, one segment
    a.dk, a.dv, a.segments = 273, 64, 0
    assert lib.fla_sm100_workspace_bytes(ctypes.byref(a), 0) == 0
    assert lib.fla_sm100_workspace_bytes(ctypes.byref(a), 1) == 0
    assert lib.fla_sm100_auto_segments(ctypes.byref(a), 1) == 1
    # entry points added beside the reference's interface reject null / empty arguments as well
    z = FlaArgs()
    assert lib.fla_sm100_normalize_fwd(None, 1e-5, None) == -1
    assert lib.fla_sm100_normalize_fwd(ctypes.byref(z), 1e-5, None) == -1
    assert lib.fla_sm100_normalize_bwd_prepare(ctypes.byref(z), None, None) == -1
    assert lib.fla_sm100_normalize_bwd_sweep(ctypes.byref(z), None) == -1
    assert lib.fla_sm100_normalize_workspace_bytes(None) == 0
    assert lib.fla_sm100_pad_rows(None, None, 1, 8, 8, None) == -1
    assert lib.fla_sm100_unpad_rows(None, None, 1, 8, 8, None) == -1
    assert lib.fla_sm100_pad_rows(ctypes.c_void_p(16), ctypes.c_void_p(32), 4, 9, 12, None) == -3  # dpad % 8
    assert lib.fla_sm100_pad_rows(ctypes.c_void_p(16), ctypes.c_void_p(32), 4, 9, 8, None) == -1   # dpad < d


def test_wrappers_keep_reference_preconditions():
    from flashlinear.kernels import (
        linear_flash_wrapper_bwd,
        linear_flash_wrapper_fwd,
        linear_flash_wrapper_fwd_smallv_hd,
    )

    q = torch.zeros(1, 1, 96, 64, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):  # sq % 64 != 0 (linear_attn_kernels.py:323-325)
        linear_flash_wrapper_fwd(q, q, q)
    with pytest.raises(AssertionError):
        linear_flash_wrapper_bwd(q, q, q, q)
    big = torch.zeros(1, 1, 64, 512, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):  # head dim cap (linear_attn_kernels.py:322)
        linear_flash_wrapper_fwd(big, big, big)
    q = torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16)
    v = torch.zeros(1, 1, 64, 24, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):  # hd_v must be a power of two (smallv_hd.py:336)
        linear_flash_wrapper_fwd_smallv_hd(q, q, v)
    v = torch.zeros(1, 1, 64, 128, dtype=torch.bfloat16)
    qs = torch.zeros(1, 1, 64, 32, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):  # hd_v <= hd_qk (smallv_hd.py:337)
        linear_flash_wrapper_fwd_smallv_hd(qs, qs, v)


def test_no_cpu_fallback():
    from flashlinear import LinearAttention, LinearAttentionSmallVHD

    q = torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        LinearAttention.apply(q, q, q)
    v = torch.zeros(1, 1, 64, 16, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        LinearAttentionSmallVHD.apply(q, q, v)


def test_public_names_match_reference():
    import flashlinear
    import flashlinear.kernels as fk

    assert issubclass(flashlinear.LinearAttention, torch.autograd.Function)
    assert issubclass(flashlinear.LinearAttentionSmallVHD, torch.autograd.Function)
    for name in (
        "linear_flash_wrapper_fwd",
        "linear_flash_wrapper_bwd",
        "linear_flash_wrapper_fwd_smallv_hd",
        "linear_flash_wrapper_bwd_smallv_hd",
    ):
        assert callable(getattr(fk, name))


def test_shard_batch_heads_partitions_every_head_once():
    from flashy_linear_attention_b200.sharding import shard_batch_heads

    t = torch.arange(4 * 32).reshape(4, 32, 1, 1)
    for world in (1, 2, 4, 8, 16):
        seen = torch.cat([shard_batch_heads(t, r, world).reshape(-1) for r in range(world)])
        assert torch.equal(seen.sort().values, t.reshape(-1))
    with pytest.raises(ValueError):
        shard_batch_heads(t, 0, 3)


def test_host_pipeline_has_no_cpu_fallback():
    from flashy_linear_attention_b200.host import HostPipeline

    with pytest.raises(RuntimeError, match="CUDA"):
        HostPipeline("cpu")


def test_segment_planning_queries_without_a_gpu():
    """How a call will be split is host arithmetic (148 SMs assumed when no device answers): the
    queries that size the caller's scratch must agree with each other for the shapes of the
    benchmark and its per-GPU shares."""
    from flashy_linear_attention_b200 import _lib
    from flashy_linear_attention_b200._lib import FlaArgs

    lib = _lib.load()

    def query(B, H, N, dk, dv, segments=0):
        a = FlaArgs()
        a.batch, a.heads, a.seqlen, a.dk, a.dv, a.segments = B, H, N, dk, dv, segments
        return {
            "seg_fwd": lib.fla_sm100_auto_segments(ctypes.byref(a), 0),
            "seg_bwd": lib.fla_sm100_auto_segments(ctypes.byref(a), 1),
            "ws_fwd": lib.fla_sm100_workspace_bytes(ctypes.byref(a), 0),
            "ws_bwd": lib.fla_sm100_workspace_bytes(ctypes.byref(a), 1),
            "states": lib.fla_sm100_seg_states_bytes(ctypes.byref(a)),
            "uses_final": lib.fla_sm100_bwd_uses_final_state(ctypes.byref(a)),
        }

    # the whole benchmark job: 128 heads fill the GPU, nothing is split, the backward sweeps once
    full = query(4, 32, 8192, 128, 128)
    assert full["seg_fwd"] == 1 and full["seg_bwd"] == 1
    assert full["ws_fwd"] == 0 and full["ws_bwd"] == 0 and full["states"] == 0
    assert full["uses_final"] == 1
    # its share on one of 8 GPUs: 16 heads, forward in 8 segments, backward in 3, both from one launch
    share = query(1, 16, 8192, 128, 128)
    assert share["seg_fwd"] == 8 and share["seg_bwd"] == 3
    assert share["states"] == 16 * 7 * 128 * 128 * 4      # one boundary state per segment but the first
    assert share["ws_fwd"] >= 16 * 8 * 128 * 128 * 4 and share["ws_bwd"] >= 3 * 16 * 3 * 128 * 128 * 4
    assert share["uses_final"] == 1
    # scratch states are padded to the kernel's tile: head dim 96 is sized like 128
    assert query(1, 16, 8192, 96, 96)["states"] == share["states"]
    assert query(1, 16, 8192, 64, 64)["states"] == 16 * 7 * 64 * 64 * 4
    # a long sequence whose even split (57 chunks) would not divide it gets equal segments (64)
    long = query(1, 16, 65536, 128, 128)
    assert long["states"] == 16 * 7 * 128 * 128 * 4
    # short sequences keep the two-direction backward; dk != dv and wide heads have no boundary states
    assert query(1, 16, 2048, 128, 128)["uses_final"] == 0
    assert query(1, 16, 8192, 128, 64)["states"] == 0
    assert query(1, 16, 8192, 256, 64)["states"] == 0
    # an explicit segment count is honoured
    assert query(1, 4, 8192, 128, 128, segments=4)["seg_fwd"] == 4
