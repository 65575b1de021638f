"""Benchmark of the causal linear attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference|reference_triton]
                    [--workload cfg3 | --shape B,H,N,dk,dv] [--scaling strong|weak] [--function linear]

One "step" = one forward + one backward of `LinearAttention` over the whole workload.
Headline workload (cfg3): bf16, B=4, H=32, N=8192, dk=dv=128; q, k = elu(N(0,1)) + 1,
v, dO ~ N(0,1), seeded synthetic data. Metric: Mtokens/s = B*N / step time, whole job.

At N > 1 (launched by torch.distributed.run, one rank per GPU) the B*H heads of the ONE workload are
split over the GPUs (strong scaling; heads are independent, so there is no data-path collective).
Before timing, every rank also runs the unsharded job and compares its shard of outputs and
gradients with it (`parity_check`; the run fails when the headline's is above 2e-2). The same line
carries two secondary measurements: the weak-scaling number (every GPU runs the whole workload) and a sequence-sharded
run of the long-context configuration (cfg5: every GPU holds N/W tokens of every head and the
per-GPU dk x dv states are exclusive-scanned between the GPUs), each with its own parity check.
Timing is barrier + CUDA events + max over ranks; one JSON line on rank 0.

`--impl reference` times the reference's naive PyTorch path (restated in oracle/torch_naive.py) on
the host cores, on a bounded sample of the same workload. `--impl reference_triton` times the
reference's own Triton kernels (the copy made by baseline/install_reference.py) on GPU 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: (B, H, N, dk, dv)
    "cfg2": (8, 16, 4096, 64, 64),
    "cfg3": (4, 32, 8192, 128, 128),
    "cfg4": (8, 16, 2048, 273, 64),  # LinearAttentionSmallVHD, 2nd-order Taylor features of 16 dims
    "cfg5": (1, 32, 65536, 128, 128),
}
METRIC = "fwd+bwd Mtokens/s, N=8K D=128 bf16, 1/2/4/8 B200; % tensor/HBM roofline"
UNIT = "Mtokens/s"
PARITY_TOL = 2e-2

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of the forward and the backward launch
# of one cfg3 step: a constant, not a measurement of the run that prints it. It comes from an ncu
# capture of the same grids at half the sequence length (518.1 + 952.6 MB), doubled: the traffic of
# these launches grows in proportion to N. Other workloads report null.
NCU_TRAFFIC_BYTES_PER_STEP = {"cfg3": 2.941e9}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s of a cuBLAS GEMM on this pool: the sustained figure (the bench's timed
    region is a long loop under the power cap), else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops_sustained"]), "measured sustained (MEASURED_PEAKS.json)"
    except Exception:
        return 1400.0, "fallback (1.4 PFLOP/s sustained, earlier measurement on this pool)"


def algorithmic_flops(B, H, N, dk, dv, chunk=128):
    """Tensor-core flops per step of the chunked algorithm with dense 128-token tiles: forward
    2C*dk + 2C*dv + 4*dk*dv per token-head (score tile, tile x values, state read and update),
    backward 6C*dk + 4C*dv + 10*dk*dv (three products, two of them with dk-wide outputs)."""
    th = B * H * N
    fwd = th * (2 * chunk * dk + 2 * chunk * dv + 4 * dk * dv)
    bwd = th * (6 * chunk * dk + 4 * chunk * dv + 10 * dk * dv)
    return fwd, bwd


def algorithmic_bytes(B, H, N, dk, dv):
    """Compulsory HBM bytes per step, bf16: fwd reads q,k,v and writes o; bwd reads q,k,v,dO and
    writes dQ,dK,dV."""
    th = B * H * N
    fwd = th * (2 * dk + 2 * dv) * 2
    bwd = th * ((2 * dk + 2 * dv) + (2 * dk + dv)) * 2
    return fwd, bwd


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi. It is started before the warm-up
    (nvidia-smi needs ~100 ms to deliver its first sample) and only the samples that fall inside
    the timed region, by wall clock, are reported."""

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "10", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t_start: float, t_end: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.thread.join(timeout=2)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

        def parse(window):
            sm, smax, reasons = [], [], set()
            for stamp, line in self.lines:
                if window and not (t_start <= stamp <= t_end + 0.02):
                    continue
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    sm.append(float(parts[1]))
                    smax.append(float(parts[2]))
                except ValueError:
                    continue
                for nme, val in zip(names, parts[4:8]):
                    if val.lower().startswith("active"):
                        reasons.add(nme)
            return sm, smax, reasons

        sm, smax, reasons = parse(True)
        scope = "timed region"
        if not sm:  # region shorter than the sampling period: fall back to the whole run
            sm, smax, reasons = parse(False)
            scope = "whole run (timed region shorter than one sample)"
        out = {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_min_mhz": min(sm) if sm else None,
            "sm_max_mhz": max(smax) if smax else None,
            "samples": len(sm),
            "scope": scope,
            "reasons": sorted(reasons),
        }
        # SM clock well below its maximum with no throttle reason active: somebody else's clock
        # lock on a shared host. The number is still reported, with this flag, for a re-measurement.
        if sm and smax and not reasons and statistics.median(sm) < 0.9 * max(smax):
            out["suspect"] = "sm clock below 90 % of max with no throttle reason active (clock lock?)"
        return out


def taylor_features(x):
    """[1, x / d^(1/4), vec(x x^T) / (sqrt(2) sqrt(d))] of raw x[..., d] (configuration 4)."""
    d = x.shape[-1]
    quad = (x.unsqueeze(-1) * x.unsqueeze(-2)).flatten(-2) / (2.0 ** 0.5 * d ** 0.5)
    return torch.cat([torch.ones_like(x[..., :1]), x / d ** 0.25, quad], dim=-1)


def make_inputs(B, H, N, dk, dv, device, seed=0):
    gen = torch.Generator(device=device).manual_seed(seed)
    if dk == 273:  # second-order Taylor features of 16-dimensional raw q, k
        q = taylor_features(torch.randn(B, H, N, 16, device=device, generator=gen)).to(torch.bfloat16)
        k = taylor_features(torch.randn(B, H, N, 16, device=device, generator=gen)).to(torch.bfloat16)
        v = torch.randn(B, H, N, dv, device=device, generator=gen).to(torch.bfloat16)
        dy = torch.randn(B, H, N, dv, device=device, generator=gen).to(torch.bfloat16)
        return q, k, v, dy
    q = (torch.nn.functional.elu(torch.randn(B, H, N, dk, device=device, generator=gen)) + 1).to(torch.bfloat16)
    k = (torch.nn.functional.elu(torch.randn(B, H, N, dk, device=device, generator=gen)) + 1).to(torch.bfloat16)
    v = torch.randn(B, H, N, dv, device=device, generator=gen).to(torch.bfloat16)
    dy = torch.randn(B, H, N, dv, device=device, generator=gen).to(torch.bfloat16)
    return q, k, v, dy


def cpu_baseline_sample(B, H, N, dk, dv, budget_s=12.0, heads=8):
    """Times the naive PyTorch path (oracle port) on the host on a bounded sample: `heads` whole
    heads of one batch entry at the full sequence length per pass, repeated for about `budget_s`
    seconds of CPU work. Returns the cpu_baseline dict."""
    from oracle import torch_naive

    threads = os.cpu_count() or 1
    heads = min(heads, H)
    t1, used = torch_naive.time_fwd_bwd_cpu(1, heads, N, dk, dv, steps=1, warmup=0, threads=threads)
    reps = int(max(1, min(30, budget_s // max(t1, 1e-3))))
    t, used = torch_naive.time_fwd_bwd_cpu(1, heads, N, dk, dv, steps=reps, warmup=0, threads=threads)
    tokens_equiv = N * heads / H  # a token counts once all H heads of it are done
    return {
        "value": tokens_equiv / t / 1e6,
        "unit": UNIT,
        "cores": used,
        "kind": "port",
        "sample": f"{heads} of {B * H} heads at full N={N}, fp32 fwd+autograd bwd, mean of {reps} passes "
                  f"of {t:.2f} s; scaled to tokens by heads/{H}",
        "seconds": t * reps,
    }


def run_reference(args, rank, shape, name, emit):
    if rank != 0:
        return
    B, H, N, dk, dv = shape
    from oracle import torch_naive

    threads = os.cpu_count() or 1
    heads = min(8, H)
    total = args.warmup + args.steps
    t_probe, used = torch_naive.time_fwd_bwd_cpu(1, heads, N, dk, dv, steps=1, threads=threads)
    # keep the whole run near a minute of CPU work
    if t_probe * total > 60:
        steps, warmup = max(1, int(60 // t_probe) - 1), 1
    else:
        steps, warmup = args.steps, args.warmup
    t, used = torch_naive.time_fwd_bwd_cpu(1, heads, N, dk, dv, steps=steps, warmup=warmup, threads=threads)
    value = (N * heads / H) / t / 1e6
    sample = f"{heads} of {B * H} heads at full N={N} per step, fp32 fwd+autograd bwd on {used} host threads"
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{name}: B={B} H={H} N={N} dk={dk} dv={dv}",
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": used, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def run_triton_reference(args, rank, shape, name, emit):
    """The reference's own Triton kernels (tuple-fixed copy under baseline/_ref) through its public
    Functions on GPU 0: the same-box comparator. Quadratic in N, so a few steps only."""
    if rank != 0:
        return
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    line = {"impl": "reference_triton"}
    try:
        if ref_dir not in sys.path:
            sys.path.insert(0, ref_dir)
        import flashlinear_triton_ref as ref
    except Exception as exc:
        line["unavailable"] = f"reference copy not importable: {type(exc).__name__}: {exc}"
        emit(line)
        return
    B, H, N, dk, dv = shape
    device = torch.device("cuda", 0)
    q, k, v, dy = make_inputs(B, H, N, dk, dv, device)
    fn = ref.LinearAttentionSmallVHD if dk != dv else ref.LinearAttention
    q, k, v = (t.requires_grad_(True) for t in (q, k, v))
    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 2))
    try:
        for _ in range(warmup):
            out = fn.apply(q, k, v)
            torch.autograd.grad(out, (q, k, v), dy)
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        fwd_ms = bwd_ms = 0.0
        for _ in range(steps):
            ev[0].record()
            out = fn.apply(q, k, v)
            ev[1].record()
            torch.autograd.grad(out, (q, k, v), dy)
            ev[2].record()
            torch.cuda.synchronize()
            fwd_ms += ev[0].elapsed_time(ev[1]) / steps
            bwd_ms += ev[1].elapsed_time(ev[2]) / steps
    except Exception as exc:
        line["unavailable"] = f"Triton did not compile or launch the reference kernels: {type(exc).__name__}: {str(exc)[:200]}"
        emit(line)
        return
    ms = fwd_ms + bwd_ms
    import triton
    line.update({
        "metric": METRIC, "value": B * N / (ms * 1e-3) / 1e6, "unit": UNIT, "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": ms, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{name}: B={B} H={H} N={N} dk={dk} dv={dv}",
                   "label": f"reference (Triton {triton.__version__}, tuple fix), {fn.__name__}.apply + torch.autograd.grad"},
    })
    emit(line)


def parse_shape(args):
    if args.shape:
        dims = tuple(int(x) for x in args.shape.split(","))
        if len(dims) != 5:
            raise SystemExit("--shape wants B,H,N,dk,dv")
        return dims, "custom"
    return WORKLOADS[args.workload], args.workload


def main():
    # Libraries (NCCL's version banner, for one) print to stdout; the contract is ONE JSON line
    # there, so everything else is sent to stderr and the line goes to the saved descriptor.
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(line: dict) -> None:
        os.write(json_fd, (json.dumps(line) + "\n").encode())

    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference_triton"])
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--shape", default=None, help="B,H,N,dk,dv instead of a named workload")
    ap.add_argument("--function", default="linear", choices=["linear", "normalized", "taylor"],
                    help="linear: LinearAttention / LinearAttentionSmallVHD (the benchmark); normalized: "
                         "LinearAttentionNormalized; taylor: TaylorLinearAttention on raw 16-dim q, k "
                         "(both through .apply + torch.autograd.grad, one GPU, device timing only)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="N>1: strong (default) = the workload's batch*heads are split over the GPUs; "
                         "weak = every GPU runs the whole workload (global batch = B x N)")
    ap.add_argument("--sharding", default=None, choices=["batch_head", "sequence"],
                    help="N>1: batch_head (default) or sequence (default for cfg5): every GPU holds "
                         "N/W tokens of every head and the per-GPU states are exclusive-scanned")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="sequence sharding: peer = state kernels store straight into the peers' memory over "
                         "NVLink and wait on flags (one fused kernel, no NCCL); nccl = all-gather + local sum")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true",
                    help="N>1: skip the weak-scaling and sequence-sharded secondary measurements")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every kernel from Python instead of replaying a captured CUDA graph per pass")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    shape, wname = parse_shape(args)

    if args.impl == "reference":
        run_reference(args, rank, shape, wname, emit)
        return
    if args.impl == "reference_triton":
        run_triton_reference(args, rank, shape, wname, emit)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the sm_100a kernels have no CPU fallback")
    import torch.distributed as dist

    from flashlinear import LinearAttention, LinearAttentionSmallVHD
    from flashy_linear_attention_b200 import _lib, ops
    from flashy_linear_attention_b200.host import HostPipeline
    from flashy_linear_attention_b200.sharding import (
        PeerShardedLinearAttention,
        PeerStateExchange,
        SequenceShardedLinearAttention,
        exclusive_state_scan,
        shard_batch_heads,
    )

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lib = _lib.load()
    stream = torch.cuda.current_stream(device)

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    def max_over_ranks(values):
        t = torch.tensor(values, device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def rel_errors(got, want):
        """(max relative error, Frobenius relative error) of one tensor against its reference."""
        g, w = got.float(), want.float()
        return ((g - w).abs().max() / w.abs().max()).item(), (torch.linalg.norm(g - w) / torch.linalg.norm(w)).item()

    # ------------------------------------------------------------------------------------------
    # One measurement: `mode` is "single" (one GPU), "strong" / "weak" (batch*head sharding) or
    # "sequence". Returns the timing, this rank's shapes and, for the sharded modes, the parity of
    # this rank's shard against the unsharded job on the same data.
    # ------------------------------------------------------------------------------------------
    def measure(shape, mode, steps, warmup, exchange="peer", want_clocks=False, keep=None):
        B, H, N, dk, dv = shape
        q, k, v, dy = make_inputs(B, H, N, dk, dv, device)
        seq_sharded = mode == "sequence"
        parity = None
        full_ref = None
        if mode in ("strong", "sequence"):
            # the unsharded job on the same data (every rank computes it; rank r then checks shard r)
            s_full = torch.empty(B * H, dk, dv, dtype=torch.float32, device=device) \
                if ops.backward_uses_final_state(q, v) else None
            o_full = ops.causal_dot_product_fwd(q, k, v, s_final=s_full)
            g_full = ops.causal_dot_product_bwd(dy, q, k, v, s_last=s_full)
            full_ref = (o_full,) + tuple(g_full)
            del s_full
        if seq_sharded:
            lo, hi = rank * N // world, (rank + 1) * N // world
            cut = lambda t: t[:, :, lo:hi].contiguous()  # noqa: E731
        elif mode == "strong":
            cut = lambda t: shard_batch_heads(t, rank, world).contiguous()  # noqa: E731
        else:
            cut = lambda t: t  # noqa: E731
        if full_ref is not None:
            full_ref = tuple(cut(t) for t in full_ref)
        q, k, v, dy = (cut(t) for t in (q, k, v, dy))
        Bl, Hl, Nl = q.shape[0], q.shape[1], q.shape[2]
        torch.cuda.empty_cache()

        # The forward also writes its final state (fp32, batch*heads x dk x dv) when the backward
        # can use it to sweep q, k, v, dO once -- what LinearAttention.apply + backward do.
        s_state = seg_states = None
        if seq_sharded or ops.backward_uses_final_state(q, v):
            s_state = torch.empty(Bl * Hl, dk, dv, dtype=torch.float32, device=device)
            if not seq_sharded:  # few heads per GPU: boundary states handed from forward to backward
                seg_states = ops.segment_states_buffer(q, v)
        ctx = {}
        peer_ex = None
        if seq_sharded and exchange == "peer":
            peer_ex = PeerStateExchange(Bl, Hl, dk, dv, device)
        repack = dk % 8 != 0  # rows the kernels cannot address in place (273-dim features)

        def step_fwd():
            if not seq_sharded and repack:
                # what LinearAttentionSmallVHD.apply does: q and k are copied to 16-byte-aligned rows
                # once (two launches of the library's pad kernel); the backward reuses the copies
                ctx["qp"], ctx["kp"] = ops.kernel_view(q), ops.kernel_view(k)
                ctx["out"] = ops.causal_dot_product_fwd(ctx["qp"], ctx["kp"], v)
                return 2 + lib.fla_sm100_last_launch_count()
            if not seq_sharded:
                ctx["out"] = ops.causal_dot_product_fwd(q, k, v, s_final=s_state, seg_states=seg_states)
                return lib.fla_sm100_last_launch_count()
            if peer_ex is not None:
                # state pass + ONE kernel that scans, stores to the peers, waits and adds their totals
                ws, ctx["prefix"], ctx["after"] = peer_ex.state_and_exchange(k, v, reverse=False)
                n = lib.fla_sm100_last_launch_count()
                ctx["out"] = ops.causal_dot_product_fwd(q, k, v, segment_workspace=ws)
                return n + lib.fla_sm100_last_launch_count()
            # sequence sharding: local state -> exclusive scan over ranks (one all-gather) -> forward
            s_local, ws = ops.chunk_state(k, v, keep_workspace=True)
            n = lib.fla_sm100_last_launch_count()
            ctx["prefix"] = exclusive_state_scan(s_local)
            ctx["out"] = ops.causal_dot_product_fwd(q, k, v, s_init=ctx["prefix"] if rank > 0 else None,
                                                    segment_workspace=ws if ws.numel() > 0 else None)
            ctx["after"] = torch.add(ctx["prefix"], s_local, out=s_state)  # state after this GPU's tokens
            return n + lib.fla_sm100_last_launch_count()

        def step_bwd():
            if not seq_sharded and repack:
                ctx["grads"] = ops.causal_dot_product_bwd(dy, ctx["qp"], ctx["kp"], v, keep_padded=True)
                return lib.fla_sm100_last_launch_count()
            if not seq_sharded:
                ctx["grads"] = ops.causal_dot_product_bwd(dy, q, k, v, s_last=s_state, seg_states=seg_states)
                return lib.fla_sm100_last_launch_count()
            if peer_ex is not None:
                _, r_suffix, _ = peer_ex.state_and_exchange(q, dy, reverse=True)
                n = lib.fla_sm100_last_launch_count()
            else:
                r_local = ops.chunk_state(q, dy)
                n = lib.fla_sm100_last_launch_count()
                r_suffix = exclusive_state_scan(r_local, reverse=True)
            ctx["grads"] = ops.causal_dot_product_bwd(dy, q, k, v, s_init=ctx["prefix"] if rank > 0 else None,
                                                      r_init=r_suffix if rank < world - 1 else None,
                                                      s_last=ctx["after"])
            return n + lib.fla_sm100_last_launch_count()

        sampler = ClockSampler(local_rank) if (want_clocks and rank == 0) else None
        if sampler:
            sampler.start()
        for _ in range(warmup):
            launches_f = step_fwd()
            launches_b = step_bwd()
        barrier()
        ops.check_status(device)
        if full_ref is not None:
            errs = [rel_errors(g, w) for g, w in zip((ctx["out"],) + tuple(ctx["grads"]), full_ref)]
            mr, fr = max_over_ranks([max(e[0] for e in errs), max(e[1] for e in errs)])
            parity = {"mode": mode, "against": "the unsharded job on the same data, every rank's shard of "
                      "out, dQ, dK, dV; max over tensors and ranks", "max_rel": mr, "frob": fr,
                      "tolerance": PARITY_TOL, "ok": bool(mr <= PARITY_TOL and fr <= PARITY_TOL)}
            full_ref = None
        # The launches are captured in CUDA graphs and replayed: for the headline time one graph that
        # holds `per_graph` whole steps back to back (what a training step with several attention
        # layers looks like to the GPU; a graph launch costs ~5 us, which at 16 heads per GPU is 4 %
        # of a step), one graph per pass for the forward / backward split (timed in a second loop,
        # with an event between the passes). The sequence-sharded path is captured too
        # when it uses the fused peer exchange (its exchange count lives on the device); the NCCL
        # arm stays eager.
        launch_mode = "eager"
        run_fwd, run_bwd = step_fwd, step_bwd

        per_graph = next(g for g in (10, 5, 4, 2, 1) if steps % g == 0)

        def step_both():
            for _ in range(per_graph):
                step_fwd()
                step_bwd()

        run_step = step_both
        if (not seq_sharded or peer_ex is not None) and not args.no_graph:
            try:
                from flashy_linear_attention_b200.graphs import capture_step
                g_fwd, g_bwd, g_step = capture_step(step_fwd), capture_step(step_bwd), capture_step(step_both)
                run_fwd, run_bwd, run_step = g_fwd, g_bwd, g_step
                launch_mode = f"CUDA graph replay, {per_graph} steps per graph"
                for _ in range(3):
                    run_fwd(); run_bwd(); run_step()
                barrier()
                ops.check_status(device)
            except Exception as exc:  # capture is an optimisation of the host side only
                launch_mode = f"eager (graph capture failed: {type(exc).__name__})"
                run_fwd, run_bwd, run_step = step_fwd, step_bwd, step_both
        t0_ev, t1_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t_region0 = time.time()
        t0_ev.record(stream)
        for i in range(steps // per_graph):
            run_step()
        t1_ev.record(stream)
        barrier()
        clocks = sampler.stop(t_region0, time.time()) if sampler else None
        ops.check_status(device)
        total_ms = t0_ev.elapsed_time(t1_ev)
        # forward / backward split: same kernels, one graph per pass, an event between the passes
        split_steps = min(steps, 50)
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(split_steps)]
        for i in range(split_steps):
            ev[i][0].record(stream)
            run_fwd()
            ev[i][1].record(stream)
            run_bwd()
            ev[i][2].record(stream)
        barrier()
        ops.check_status(device)
        fwd_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / split_steps
        bwd_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / split_steps
        total_ms, fwd_ms, bwd_ms = max_over_ranks([total_ms, fwd_ms, bwd_ms])
        res = {
            "ms_per_step": total_ms / steps, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "steps": steps, "warmup": warmup,
            "launches_per_step": launches_f + launches_b, "launch_mode": launch_mode, "clocks": clocks,
            "local_shape": (Bl, Hl, Nl, dk, dv), "parity_check": parity,
            "working_set_mb": 8 * q.numel() * 2 / 1e6 if dk == dv else (4 * q.numel() + 4 * v.numel()) * 2 / 1e6,
            "exchange": (None if not seq_sharded else
                         "by the state kernel itself (stores into the peers' HBM over NVLink + flags)"
                         if peer_ex is not None else "with one NCCL all-gather per pass"),
        }
        if keep is not None:
            keep.update({"q": q, "k": k, "v": v, "dy": dy, "peer_ex": peer_ex})
        elif peer_ex is not None:
            peer_ex.close()
        return res

    def roofline_of(res, peak):
        Bl, Hl, Nl, dk, dv = res["local_shape"]
        fwd_b, bwd_b = algorithmic_bytes(Bl, Hl, Nl, dk, dv)  # this rank's share
        achieved = (fwd_b + bwd_b) / ((res["fwd_ms"] + res["bwd_ms"]) * 1e-3) / 1e9
        return fwd_b, bwd_b, achieved, achieved / peak

    # ------------------------------------------------------------------------------------------
    # other Functions of the library, through autograd (one GPU)
    # ------------------------------------------------------------------------------------------
    if args.function != "linear":
        from flashy_linear_attention_b200.functions import LinearAttentionNormalized, TaylorLinearAttention

        B, H, N, dk, dv = shape
        if args.function == "taylor":
            gen = torch.Generator(device=device).manual_seed(0)
            q = torch.randn(B, H, N, 16, device=device, generator=gen).to(torch.bfloat16)
            k = torch.randn(B, H, N, 16, device=device, generator=gen).to(torch.bfloat16)
            v = torch.randn(B, H, N, dv, device=device, generator=gen).to(torch.bfloat16)
            dy = torch.randn(B, H, N, dv, device=device, generator=gen).to(torch.bfloat16)
            fn = TaylorLinearAttention
        else:
            q, k, v, dy = make_inputs(B, H, N, dk, dv, device)
            fn = LinearAttentionNormalized
        q, k, v = (t.requires_grad_(True) for t in (q, k, v))
        warmup, steps = max(args.warmup, 3), args.steps
        for _ in range(warmup):
            torch.autograd.grad(fn.apply(q, k, v), (q, k, v), dy)
        barrier()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        fwd_ms = bwd_ms = 0.0
        for _ in range(steps):
            e[0].record(stream)
            out = fn.apply(q, k, v)
            e[1].record(stream)
            torch.autograd.grad(out, (q, k, v), dy)
            e[2].record(stream)
            torch.cuda.synchronize(device)
            fwd_ms += e[0].elapsed_time(e[1]) / steps
            bwd_ms += e[1].elapsed_time(e[2]) / steps
        ops.check_status(device)
        emit({"metric": METRIC, "value": B * N / ((fwd_ms + bwd_ms) * 1e-3) / 1e6, "unit": UNIT, "n_gpus": 1,
              "steps": steps, "warmup": warmup, "ms_per_step": fwd_ms + bwd_ms, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
              "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
              "config": {"workload": f"{wname}: {fn.__name__}.apply + torch.autograd.grad, B={B} H={H} N={N} "
                                     f"dk={dk} dv={dv}, eager launches, per-step synchronisation"}})
        return

    B, H, N, dk, dv = shape
    sharding = args.sharding or ("sequence" if wname == "cfg5" else "batch_head")
    if world == 1:
        mode = "single"
    elif sharding == "sequence":
        mode = "sequence"
    else:
        mode = args.scaling
    warmup = max(args.warmup, 3)
    steps = args.steps
    kept = {}
    head = measure(shape, mode, steps, warmup, exchange=args.exchange, want_clocks=True, keep=kept)
    q, k, v, dy, peer_ex = (kept[n] for n in ("q", "k", "v", "dy", "peer_ex"))
    seq_sharded = mode == "sequence"
    strong = mode in ("strong", "sequence")
    Bl, Hl, Nl = head["local_shape"][:3]
    global_batch = B if (strong or world == 1) else B * world
    ms_per_step = head["ms_per_step"]
    value = global_batch * N / (ms_per_step * 1e-3) / 1e6

    # ---------------------------------------------------------------- the Functions, device-resident
    # LinearAttention.apply + torch.autograd.grad on device tensors, launched eagerly from Python:
    # the public call a training step makes. The gap to `value` is host-side launch cost.
    autograd_line = None
    if not seq_sharded:
        fn = LinearAttentionSmallVHD if dk != dv else LinearAttention
        aq, ak, av = (t.detach().requires_grad_(True) for t in (q, k, v))
        for _ in range(3):
            torch.autograd.grad(fn.apply(aq, ak, av), (aq, ak, av), dy)
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_steps = max(1, min(steps, 50))
        a0.record(stream)
        for _ in range(a_steps):
            torch.autograd.grad(fn.apply(aq, ak, av), (aq, ak, av), dy)
        a1.record(stream)
        barrier()
        a_ms = max_over_ranks([a0.elapsed_time(a1) / a_steps])[0]
        autograd_line = {"api": f"flashlinear.{fn.__name__}.apply + torch.autograd.grad, device tensors, eager launches",
                         "ms_per_step": a_ms, "value": global_batch * N / (a_ms * 1e-3) / 1e6, "unit": UNIT,
                         "steps": a_steps}
        del aq, ak, av

    # ---------------------------------------------------------------- end to end, host buffers
    e2e_steps = max(1, min(args.e2e_steps, steps))
    host_in = [torch.empty(x.shape, dtype=x.dtype, pin_memory=True).copy_(x) for x in (q, k, v, dy)]
    host_out = [torch.empty(x.shape, dtype=x.dtype, pin_memory=True) for x in (v, q, k, v)]
    h2d = sum(x.numel() * x.element_size() for x in host_in)
    d2h = sum(x.numel() * x.element_size() for x in host_out)

    pipeline = None if seq_sharded else HostPipeline(device)

    def e2e_autograd_step():
        dq_, dk_, dv_, ddy = (x.to(device, non_blocking=True) for x in host_in)
        dq_.requires_grad_(True); dk_.requires_grad_(True); dv_.requires_grad_(True)
        if seq_sharded and peer_ex is not None:
            out = PeerShardedLinearAttention.apply(dq_, dk_, dv_, peer_ex)
        elif seq_sharded:
            out = SequenceShardedLinearAttention.apply(dq_, dk_, dv_, None)
        else:
            out = (LinearAttentionSmallVHD if dk != dv else LinearAttention).apply(dq_, dk_, dv_)
        grads = torch.autograd.grad(out, (dq_, dk_, dv_), ddy)
        for dst, src in zip(host_out, (out,) + tuple(grads)):
            dst.copy_(src.detach(), non_blocking=True)

    def e2e_pipelined_step():
        # slabs of heads cross PCIe in both directions while the kernels run on the slab between
        pipeline.fwd_bwd(*host_in, *host_out)

    def time_e2e(step_fn):
        step_fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            step_fn()
        e1.record(stream)
        barrier()
        ms = max_over_ranks([e0.elapsed_time(e1) / e2e_steps])[0]
        return global_batch * N / (ms * 1e-3) / 1e6

    e2e_autograd = time_e2e(e2e_autograd_step)
    e2e_value = time_e2e(e2e_pipelined_step) if pipeline is not None else e2e_autograd
    ops.check_status(device)
    h2d_total = torch.tensor([h2d, d2h], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(h2d_total, op=dist.ReduceOp.SUM)
    h2d_all, d2h_all = (int(x) for x in h2d_total.tolist())
    if peer_ex is not None:
        peer_ex.close()
    del host_in, host_out, q, k, v, dy, kept, pipeline
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- secondary measurements (N > 1)
    peak, peak_src = measured_peaks()
    secondary = {}
    if world > 1 and not args.no_secondary and wname in ("cfg2", "cfg3") and mode == "strong":
        sec_steps = max(10, steps // 4)
        w = measure(shape, "weak", sec_steps, warmup)
        _, _, ach, frac = roofline_of(w, peak)
        secondary["weak"] = {
            "scaling": "weak", "workload": f"{wname} per GPU (global batch {B * world})",
            "value": B * world * N / (w["ms_per_step"] * 1e-3) / 1e6, "unit": UNIT,
            "ms_per_step": w["ms_per_step"], "steps": sec_steps, "roofline_frac_per_gpu": frac}
        torch.cuda.empty_cache()
    if world > 1 and not args.no_secondary and wname != "cfg5":
        sec_steps = max(10, steps // 4)
        s5 = measure(WORKLOADS["cfg5"], "sequence", sec_steps, warmup, exchange="peer")
        b5, h5, n5 = WORKLOADS["cfg5"][:3]
        fwd_b, bwd_b, ach, frac = roofline_of(s5, peak)
        secondary["cfg5_seq"] = {
            "workload": f"cfg5: B={b5} H={h5} N={n5} dk=dv=128, sequence sharded over {world} GPUs "
                        f"({s5['local_shape'][2]} tokens of every head per GPU), states exchanged {s5['exchange']}",
            "scaling": "strong", "value": b5 * n5 / (s5["ms_per_step"] * 1e-3) / 1e6, "unit": UNIT,
            "ms_per_step": s5["ms_per_step"], "fwd_ms": s5["fwd_ms"], "bwd_ms": s5["bwd_ms"], "steps": sec_steps,
            "launch": s5["launch_mode"], "launches_per_step": s5["launches_per_step"],
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": frac,
                         "algorithmic_bytes_per_step_per_gpu": fwd_b + bwd_b},
            "parity_check": s5["parity_check"]}
        torch.cuda.empty_cache()

    # The run fails on the headline's parity only. A secondary measurement that misses the tolerance
    # keeps its "ok": false in the line (and a note on stderr) without taking the headline down.
    failed = [name for name, pc in [("headline", head["parity_check"])] if pc is not None and not pc["ok"]]
    sec_pc = secondary.get("cfg5_seq", {}).get("parity_check")
    if rank == 0 and sec_pc is not None and not sec_pc["ok"]:
        print(f"bench.py: secondary cfg5_seq parity above tolerance: {sec_pc}", file=sys.stderr)

    if rank == 0:
        fwd_b, bwd_b, achieved, frac = roofline_of(head, peak)
        fwd_f, bwd_f = algorithmic_flops(Bl, Hl, Nl, dk, dv)
        tpeak, tpeak_src = measured_tensor_peak()
        fwd_ms, bwd_ms = head["fwd_ms"], head["bwd_ms"]
        traffic = NCU_TRAFFIC_BYTES_PER_STEP.get(wname) if world == 1 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if strong else args.scaling, "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": f"{wname}: {'LinearAttentionSmallVHD' if dk != dv else 'LinearAttention'} "
                            f"fwd+bwd B={B} H={H} N={N} dk={dk} dv={dv} per "
                            f"{'job' if strong or world == 1 else 'GPU'}, "
                            + ("q,k=2nd-order Taylor features of N(0,1)^16" if dk == 273 else "q,k=elu(N(0,1))+1")
                            + ", v,dO~N(0,1), seed 0",
                "global_batch": global_batch, "seq_len": N,
                "parallelism": (f"sequence sharded over {world} GPUs: {Nl} tokens of every head per GPU; per-GPU "
                                f"dk x dv fp32 states exchanged {head['exchange']}")
                if seq_sharded else
                f"batch*head sharded over {world} GPU(s): {Bl}x{Hl} heads per GPU, no collective",
                "l2": (f"per-GPU working set {head['working_set_mb']:.0f} MB exceeds the 126 MB L2; no flush between steps"
                       if head["working_set_mb"] > 126 else
                       f"per-GPU working set {head['working_set_mb']:.0f} MB does NOT exceed the 126 MB L2 and is not "
                       "flushed between steps"),
                "chunk": 128,
                "launch": head["launch_mode"],
            },
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_all,
                    "d2h_bytes_per_step": d2h_all, "steps": e2e_steps,
                    "api": ("SequenceShardedLinearAttention.apply + torch.autograd.grad, pinned host buffers"
                            if seq_sharded else
                            "flashy_linear_attention_b200.host.HostPipeline.fwd_bwd: pinned host buffers, slabs "
                            "of 16 heads, copies in both directions overlapped with the kernels"),
                    "unpipelined": {"value": e2e_autograd, "api": "flashlinear.LinearAttention.apply + "
                                    "torch.autograd.grad: copy in, compute, copy out, one stream"}},
            "gpu_launches": head["launches_per_step"] * steps,
            "clocks": head["clocks"],
            "roofline": {
                "bound": "hbm", "kernel": (f"fla_chunk_kernel<{max(dk, dv)},{max(dk, dv)}> (fwd launch + bwd launch)"
                                             if max(dk, dv) <= 128 else
                                             "fla_pad_rows_kernel x2, fla_wide_kernel<3> (fwd, dV), "
                                             "fla_chunk_kernel<128,128> on 128-column output slices (dQ, dK)"),
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": frac,
                "peak_source": peak_src,
                "algorithmic_bytes_per_step": fwd_b + bwd_b,
                "traffic": traffic,
                "traffic_source": ("ncu DRAM byte count of the two launches at half the sequence length, doubled; a "
                                   "constant, not measured in this run" if traffic is not None else None),
                "fwd": {"ms": fwd_ms, "GBps": fwd_b / (fwd_ms * 1e-3) / 1e9, "frac": fwd_b / (fwd_ms * 1e-3) / 1e9 / peak,
                        "Mtokens_per_s": global_batch * N / (fwd_ms * 1e-3) / 1e6},
                "bwd": {"ms": bwd_ms, "GBps": bwd_b / (bwd_ms * 1e-3) / 1e9, "frac": bwd_b / (bwd_ms * 1e-3) / 1e9 / peak},
                # the same step against the tensor-pipe bound (the path is HBM-bound; shown beside it)
                "tensor": {"achieved": (fwd_f + bwd_f) / ((fwd_ms + bwd_ms) * 1e-3) / 1e12, "peak": tpeak,
                           "unit": "TFLOP/s", "frac": (fwd_f + bwd_f) / ((fwd_ms + bwd_ms) * 1e-3) / 1e12 / tpeak,
                           "peak_source": tpeak_src, "algorithmic_flops_per_step": fwd_f + bwd_f},
            },
        }
        if autograd_line is not None:
            line["autograd"] = autograd_line
        if head["parity_check"] is not None:
            line["parity_check"] = head["parity_check"]
        if secondary:
            line["secondary"] = secondary
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_sample(B, H, N, dk, dv)
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise SystemExit(f"bench.py: parity check failed for {failed} (tolerance {PARITY_TOL})")


if __name__ == "__main__":
    main()
