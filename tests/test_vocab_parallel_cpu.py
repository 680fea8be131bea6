"""Host-side logic of the vocabulary-parallel fused loss on 2 CPU ranks (gloo): the packed
per-row statistics are all-gathered and merged exactly as the op does it, the partial
d(hidden) are all-reduced, dW stays local.  The per-shard device arithmetic is stood in for
by the numpy oracle, so this runs without a GPU."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from bastile_b200.ops.fused_linear_cross_entropy import merge_shard_stats

        rng = np.random.default_rng(0)  # same data on every rank
        bt, h, v = 48, 32, 96
        x = rng.standard_normal((bt, h)).astype(np.float32)
        w = (rng.standard_normal((v, h)) * 0.3).astype(np.float32)
        t = rng.integers(0, v, bt)
        t[::5] = -100
        vs = v // world
        w_loc = w[rank * vs:(rank + 1) * vs]
        stats, logits = oracle.lce_shard_stats(x, w_loc, t, -100, rank * vs)
        mine = torch.tensor(stats, dtype=torch.float32)
        gathered = torch.empty(world, bt, 3)
        dist.all_gather_into_tensor(gathered.view(-1), mine.view(-1))
        merged = merge_shard_stats(gathered).numpy().astype(np.float64)
        valid = t != -100
        scale = 1.0 / valid.sum()
        probs = np.exp(logits - merged[:, :1]) / merged[:, 1:2]
        loc = t - rank * vs
        own = valid & (loc >= 0) & (loc < vs)
        probs[np.arange(bt)[own], loc[own]] -= 1.0
        probs[~valid] = 0.0
        dlog = probs * scale
        dx = torch.tensor(dlog @ w_loc.astype(np.float64), dtype=torch.float32)
        dist.all_reduce(dx)
        dw_loc = dlog.T @ x.astype(np.float64)
        loss = float(np.where(valid, merged[:, 0] + np.log(merged[:, 1]) - merged[:, 2], 0.0).sum() * scale)
        l_ref, dx_ref, dw_ref = oracle.lce_fwd_bwd(x, w, t, -100, "mean")
        ok = (abs(loss - float(l_ref)) < 1e-5 and np.allclose(dx.numpy(), dx_ref, atol=1e-5)
              and np.allclose(dw_loc, dw_ref[rank * vs:(rank + 1) * vs], atol=1e-5))
        q.put((rank, bool(ok), loss, float(l_ref)))
    finally:
        dist.destroy_process_group()


def test_vocab_parallel_merge_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, loss, ref in results:
        assert ok, f"rank {rank}: loss {loss} vs {ref}"


def test_merge_shard_stats_matches_oracle_merge():
    from bastile_b200.ops.fused_linear_cross_entropy import merge_shard_stats

    rng = np.random.default_rng(1)
    st = rng.standard_normal((4, 17, 3)).astype(np.float32)
    st[..., 1] = np.abs(st[..., 1]) + 0.1
    got = merge_shard_stats(torch.tensor(st)).numpy()
    want = oracle.merge_shard_stats(st)
    lse_got = got[:, 0] + np.log(got[:, 1])
    lse_want = want[:, 0] + np.log(want[:, 1])
    np.testing.assert_allclose(lse_got, lse_want, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(got[:, 2], want[:, 2], rtol=1e-5, atol=1e-5)
