"""world_size-2 (and 4) gloo tests on CPU of the multi-GPU host logic: the exclusive / reverse
exclusive scan of per-rank states, sequence-sharded attention assembled from shard-local results
(the shard-local arithmetic is done by the oracle here), and failure of a rank that never joins."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port, timeout_s=60):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _scan_worker(rank, world, port):
    sys.path.insert(0, ROOT)
    from flashy_linear_attention_b200.sharding import exclusive_state_scan

    _init(rank, world, port)
    local = torch.full((3, 4, 5), float(rank + 1))
    fwd = exclusive_state_scan(local)
    rev = exclusive_state_scan(local, reverse=True)
    assert torch.equal(fwd, torch.full((3, 4, 5), float(sum(range(1, rank + 1)))))
    assert torch.equal(rev, torch.full((3, 4, 5), float(sum(range(rank + 2, world + 1)))))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_exclusive_state_scan_gloo(world):
    mp.spawn(_scan_worker, args=(world, _free_port()), nprocs=world, join=True)


def _seq_shard_worker(rank, world, port):
    sys.path.insert(0, ROOT)
    from flashy_linear_attention_b200.sharding import exclusive_state_scan
    from oracle import linear_attention_oracle as orc

    _init(rank, world, port)
    rng = np.random.default_rng(0)  # same data on every rank; each takes its token shard
    n, d = 256, 16
    q = orc.elu_plus_one(rng.standard_normal((1, 2, n, d)))
    k = orc.elu_plus_one(rng.standard_normal((1, 2, n, d)))
    v = rng.standard_normal((1, 2, n, d))
    dy = rng.standard_normal((1, 2, n, d))
    lo, hi = rank * n // world, (rank + 1) * n // world
    ql, kl, vl, dyl = (t[..., lo:hi, :] for t in (q, k, v, dy))
    s_local = torch.from_numpy(np.matmul(np.swapaxes(kl, -1, -2), vl))
    r_local = torch.from_numpy(np.matmul(np.swapaxes(ql, -1, -2), dyl))
    s_prefix = exclusive_state_scan(s_local).numpy()
    r_suffix = exclusive_state_scan(r_local, reverse=True).numpy()
    out, _ = orc.chunked_fwd(ql, kl, vl, chunk=64, s_init=s_prefix)
    dq, dk, dv, _ = orc.chunked_bwd(ql, kl, vl, dyl, chunk=64, s_init=s_prefix, r_init=r_suffix)
    full = orc.linear_ref(q, k, v)
    fq, fk, fv = orc.linear_ref_grads(q, k, v, dy)
    for mine, ref in ((out, full), (dq, fq), (dk, fk), (dv, fv)):
        assert orc.max_rel_error(mine, ref[..., lo:hi, :]) < 1e-12
    dist.destroy_process_group()


def test_sequence_sharding_assembles_the_full_result_gloo():
    mp.spawn(_seq_shard_worker, args=(2, _free_port()), nprocs=2, join=True)


def _missing_rank_worker(rank, world, port):
    # rank 1 never joins the collective; rank 0 must get an error after the timeout, not hang
    sys.path.insert(0, ROOT)
    from flashy_linear_attention_b200.sharding import exclusive_state_scan

    _init(rank, world, port, timeout_s=3)
    if rank == 1:
        dist.destroy_process_group()
        return
    with pytest.raises(Exception):
        exclusive_state_scan(torch.ones(4))
    os._exit(0)


def test_scan_fails_instead_of_hanging_when_a_rank_leaves():
    mp.spawn(_missing_rank_worker, args=(2, _free_port()), nprocs=2, join=True)
