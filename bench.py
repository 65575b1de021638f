"""Benchmark of the causal linear attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload cfg3]

One "step" = one forward + one backward of `LinearAttention` over the whole workload.
Headline workload (cfg3): bf16, B=4, H=32, N=8192, dk=dv=128; q, k = elu(N(0,1)) + 1,
v, dO ~ N(0,1), seeded synthetic data. Metric: Mtokens/s = B*N / step time, whole job.

At N > 1 (launched by torch.distributed.run, one rank per GPU) the heads are independent, so the
job is sharded by batch*head with no data-path collective: by default every GPU runs the whole
workload (weak scaling, global batch = B x N); `--scaling strong` splits the B*H heads of the one
workload over the GPUs instead. Timing is barrier + max over ranks; one JSON line on rank 0.

`--impl reference` times the reference's naive PyTorch path (restated in oracle/torch_naive.py) on
the host cores, on a bounded sample of the same workload.
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
    "cfg3_small": (4, 32, 1024, 128, 128),  # cfg3's head count at N=1024: sized for ncu captures
    "cfg3_half": (4, 32, 4096, 128, 128),   # cfg3 at half the sequence length (1 GB resident)
    "cfg4": (8, 16, 2048, 273, 64),  # LinearAttentionSmallVHD, 2nd-order Taylor features of 16 dims
    "cfg5": (1, 32, 65536, 128, 128),
    "cfg5_quarter": (1, 32, 16384, 128, 128),  # cfg5's head count at N=16384 (1 GB resident): for ncu captures
}
METRIC = "fwd+bwd Mtokens/s, N=8K D=128 bf16, 1/2/4/8 B200; % tensor/HBM roofline"
UNIT = "Mtokens/s"

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of the forward and backward launches
# of fla_chunk_kernel<128,128> at cfg3, from the ncu capture summarised under profiles/.
# Other workloads have no capture and report null.
NCU_TRAFFIC_BYTES_PER_STEP = {"cfg3": 2.909e9}


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
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_min_mhz": min(sm) if sm else None,
            "sm_max_mhz": max(smax) if smax else None,
            "samples": len(sm),
            "scope": scope,
            "reasons": sorted(reasons),
        }


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


def run_reference(args, rank, world, emit):
    if rank != 0:
        return
    B, H, N, dk, dv = WORKLOADS[args.workload]
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
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: B={B} H={H} N={N} dk={dk} dv={dv}",
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": used, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


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
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="N>1: weak = every GPU runs the whole workload (global batch = B x N); "
                         "strong = the workload's batch*heads are split over the GPUs")
    ap.add_argument("--sharding", default=None, choices=["batch_head", "sequence"],
                    help="N>1: batch_head (default) or sequence (default for cfg5): every GPU holds "
                         "N/W tokens of every head and the per-GPU states are exclusive-scanned")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="sequence sharding: peer = state kernels store straight into the peers' memory over "
                         "NVLink and wait on flags (one fused kernel, no NCCL); nccl = all-gather + local sum")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every kernel from Python instead of replaying a captured CUDA graph per pass")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world, emit)
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

    B, H, N, dk, dv = WORKLOADS[args.workload]
    q, k, v, dy = make_inputs(B, H, N, dk, dv, device)
    sharding = args.sharding or ("sequence" if args.workload == "cfg5" else "batch_head")
    seq_sharded = sharding == "sequence" and world > 1
    strong = (args.scaling == "strong" or seq_sharded) and world > 1
    if seq_sharded:
        lo, hi = rank * N // world, (rank + 1) * N // world
        q, k, v, dy = (t[:, :, lo:hi].contiguous() for t in (q, k, v, dy))
    elif strong:
        q, k, v, dy = (shard_batch_heads(t, rank, world).contiguous() for t in (q, k, v, dy))
    Bl, Hl, Nl = q.shape[0], q.shape[1], q.shape[2]
    global_batch = B if (strong or world == 1) else B * world
    torch.cuda.empty_cache()
    warmup = max(args.warmup, 3)
    steps = args.steps
    stream = torch.cuda.current_stream(device)

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    # ---------------------------------------------------------------- kernel-level timing
    # The forward also writes its final state (fp32, batch*heads x dk x dv) when the backward can
    # use it to sweep q, k, v, dO once -- what LinearAttention.apply + backward do.
    s_state = None
    if seq_sharded or ops.backward_uses_final_state(q, v):
        s_state = torch.empty(Bl * Hl, dk, dv, dtype=torch.float32, device=device)
    seq_ctx = {}
    peer_ex = None
    if seq_sharded and args.exchange == "peer":
        peer_ex = PeerStateExchange(Bl, Hl, dk, dv, device)

    repack = dk % 8 != 0  # rows the kernels cannot address in place (273-dim features)

    def step_fwd():
        if not seq_sharded and repack:
            # what LinearAttentionSmallVHD.apply does: q and k are copied to 16-byte-aligned rows
            # once (two launches of the library's pad kernel); the backward reuses the copies
            seq_ctx["qp"], seq_ctx["kp"] = ops.kernel_view(q), ops.kernel_view(k)
            ops.causal_dot_product_fwd(seq_ctx["qp"], seq_ctx["kp"], v)
            return 2 + lib.fla_sm100_last_launch_count()
        if not seq_sharded:
            ops.causal_dot_product_fwd(q, k, v, s_final=s_state)
            return lib.fla_sm100_last_launch_count()
        if peer_ex is not None:
            # state pass + ONE kernel that scans, stores to the peers, waits and adds their totals
            ws, seq_ctx["prefix"], seq_ctx["after"] = peer_ex.state_and_exchange(k, v, reverse=False)
            n = lib.fla_sm100_last_launch_count()
            ops.causal_dot_product_fwd(q, k, v, segment_workspace=ws)
            return n + lib.fla_sm100_last_launch_count()
        # sequence sharding: local state -> exclusive scan over ranks (one all-gather) -> forward
        s_local, ws = ops.chunk_state(k, v, keep_workspace=True)
        n = lib.fla_sm100_last_launch_count()
        seq_ctx["prefix"] = exclusive_state_scan(s_local)
        ops.causal_dot_product_fwd(q, k, v, s_init=seq_ctx["prefix"] if rank > 0 else None,
                                   segment_workspace=ws if ws.numel() > 0 else None)
        seq_ctx["after"] = torch.add(seq_ctx["prefix"], s_local, out=s_state)  # state after this GPU's tokens
        return n + lib.fla_sm100_last_launch_count()

    def step_bwd():
        if not seq_sharded and repack:
            ops.causal_dot_product_bwd(dy, seq_ctx["qp"], seq_ctx["kp"], v, keep_padded=True)
            return lib.fla_sm100_last_launch_count()
        if not seq_sharded:
            ops.causal_dot_product_bwd(dy, q, k, v, s_last=s_state)
            return lib.fla_sm100_last_launch_count()
        if peer_ex is not None:
            _, r_suffix, _ = peer_ex.state_and_exchange(q, dy, reverse=True)
            n = lib.fla_sm100_last_launch_count()
        else:
            r_local = ops.chunk_state(q, dy)
            n = lib.fla_sm100_last_launch_count()
            r_suffix = exclusive_state_scan(r_local, reverse=True)
        ops.causal_dot_product_bwd(dy, q, k, v, s_init=seq_ctx["prefix"] if rank > 0 else None,
                                   r_init=r_suffix if rank < world - 1 else None, s_last=seq_ctx["after"])
        return n + lib.fla_sm100_last_launch_count()

    launches = 0
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(warmup):
        launches_f = step_fwd()
        launches_b = step_bwd()
    barrier()
    ops.check_status(device)
    # The launches of a pass are captured in a CUDA graph and replayed (one graph per pass, so that
    # the forward / backward split can still be timed with events). The sequence-sharded path is
    # captured too when it uses the fused peer exchange (its exchange count lives on the device);
    # the NCCL arm stays eager.
    launch_mode = "eager"
    if (not seq_sharded or peer_ex is not None) and not args.no_graph:
        try:
            from flashy_linear_attention_b200.graphs import capture_step
            g_fwd, g_bwd = capture_step(step_fwd), capture_step(step_bwd)
            step_fwd, step_bwd = g_fwd, g_bwd
            launch_mode = "one CUDA graph replay per pass"
            for _ in range(3):
                step_fwd(); step_bwd()
            barrier()
            ops.check_status(device)
        except Exception as exc:  # capture is an optimisation of the host side only
            launch_mode = f"eager (graph capture failed: {type(exc).__name__})"
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    barrier()
    t_region0 = time.time()
    for i in range(steps):
        ev[i][0].record(stream)
        step_fwd()
        ev[i][1].record(stream)
        step_bwd()
        ev[i][2].record(stream)
    barrier()
    clocks = sampler.stop(t_region0, time.time()) if rank == 0 else None
    ops.check_status(device)
    total_ms = ev[0][0].elapsed_time(ev[-1][2])
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / steps
    launches = (launches_f + launches_b) * steps
    t = torch.tensor([total_ms, fwd_ms, bwd_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, fwd_ms, bwd_ms = (float(x) for x in t.tolist())
    ms_per_step = total_ms / steps
    value = global_batch * N / (ms_per_step * 1e-3) / 1e6

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
        ms = torch.tensor([e0.elapsed_time(e1) / e2e_steps], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return global_batch * N / (float(ms.item()) * 1e-3) / 1e6

    e2e_autograd = time_e2e(e2e_autograd_step)
    e2e_value = time_e2e(e2e_pipelined_step) if pipeline is not None else e2e_autograd
    ops.check_status(device)
    h2d_total = torch.tensor([h2d, d2h], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(h2d_total, op=dist.ReduceOp.SUM)
    h2d_all, d2h_all = (int(x) for x in h2d_total.tolist())

    if rank == 0:
        peak, peak_src = measured_peaks()
        fwd_b, bwd_b = algorithmic_bytes(Bl, Hl, Nl, dk, dv)  # this rank's share
        fwd_f, bwd_f = algorithmic_flops(Bl, Hl, Nl, dk, dv)
        tpeak, tpeak_src = measured_tensor_peak()
        achieved = (fwd_b + bwd_b) / ((fwd_ms + bwd_ms) * 1e-3) / 1e9
        traffic = NCU_TRAFFIC_BYTES_PER_STEP.get(args.workload) if world == 1 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": f"{args.workload}: {'LinearAttentionSmallVHD' if dk != dv else 'LinearAttention'} "
                            f"fwd+bwd B={B} H={H} N={N} dk={dk} dv={dv} per "
                            f"{'job' if strong or world == 1 else 'GPU'}, "
                            + ("q,k=2nd-order Taylor features of N(0,1)^16" if dk == 273 else "q,k=elu(N(0,1))+1")
                            + ", v,dO~N(0,1), seed 0",
                "global_batch": global_batch, "seq_len": N,
                "parallelism": (f"sequence sharded over {world} GPUs: {Nl} tokens of every head per GPU; per-GPU "
                                f"dk x dv fp32 states exchanged "
                                + ("by the state kernel itself (stores into the peers' HBM over NVLink + flags)"
                                   if peer_ex is not None else "with one NCCL all-gather per pass"))
                if seq_sharded else
                f"batch*head sharded over {world} GPU(s): {Bl}x{Hl} heads per GPU, no collective",
                "l2": f"per-GPU working set {8 * q.numel() * 2 / 1e6:.0f} MB exceeds the 126 MB L2; no flush between steps",
                "chunk": 128,
                "launch": launch_mode,
            },
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_all,
                    "d2h_bytes_per_step": d2h_all, "steps": e2e_steps,
                    "api": ("SequenceShardedLinearAttention.apply + torch.autograd.grad, pinned host buffers"
                            if seq_sharded else
                            "flashy_linear_attention_b200.host.HostPipeline.fwd_bwd: pinned host buffers, slabs "
                            "of 16 heads, copies in both directions overlapped with the kernels"),
                    "unpipelined": {"value": e2e_autograd, "api": "flashlinear.LinearAttention.apply + "
                                    "torch.autograd.grad: copy in, compute, copy out, one stream"}},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {
                "bound": "hbm", "kernel": (f"fla_chunk_kernel<{max(dk, dv)},{max(dk, dv)}> (fwd launch + bwd launch)"
                                             if max(dk, dv) <= 128 else
                                             "fla_pad_rows_kernel x2, fla_wide_kernel<3> (fwd, dV), "
                                             "fla_chunk_kernel<128,128> on 128-column output slices (dQ, dK)"),
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": peak_src,
                "algorithmic_bytes_per_step": fwd_b + bwd_b,
                "traffic": traffic,
                "fwd": {"ms": fwd_ms, "GBps": fwd_b / (fwd_ms * 1e-3) / 1e9, "frac": fwd_b / (fwd_ms * 1e-3) / 1e9 / peak,
                        "Mtokens_per_s": global_batch * N / (fwd_ms * 1e-3) / 1e6},
                "bwd": {"ms": bwd_ms, "GBps": bwd_b / (bwd_ms * 1e-3) / 1e9, "frac": bwd_b / (bwd_ms * 1e-3) / 1e9 / peak},
                # the same step against the tensor-pipe bound (the path is HBM-bound; shown beside it)
                "tensor": {"achieved": (fwd_f + bwd_f) / ((fwd_ms + bwd_ms) * 1e-3) / 1e12, "peak": tpeak,
                           "unit": "TFLOP/s", "frac": (fwd_f + bwd_f) / ((fwd_ms + bwd_ms) * 1e-3) / 1e12 / tpeak,
                           "peak_source": tpeak_src, "algorithmic_flops_per_step": fwd_f + bwd_f},
            },
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_sample(B, H, N, dk, dv)
        emit(line)
    if peer_ex is not None:
        peer_ex.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
