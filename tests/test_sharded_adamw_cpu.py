"""Bookkeeping of ShardedAdamW on 2 CPU ranks (gloo): bucket layout, parameters re-laid as views,
gradients consumed by the hooks, reduction + update of the rank's slice + re-assembly, partial
buckets.  The CUDA kernels are stood in for by the numpy oracle through ``update_fn``; the result
must equal one process running torch.optim.AdamW on the averaged gradients."""

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


def _oracle_update(bucket, step, hyper, master_weights):
    p = bucket.flat_p[bucket.lo:bucket.hi]
    g = bucket.flat_g[bucket.lo:bucket.hi]
    st = bucket.state
    src = st["master"] if master_weights else p
    b1, b2 = hyper["betas"]
    pn, m, v = oracle.adamw_step(src.double().numpy(), g.double().numpy(), st["exp_avg"].double().numpy(),
                                 st["exp_avg_sq"].double().numpy(), step, hyper["lr"], b1, b2, hyper["eps"],
                                 hyper["weight_decay"])
    st["exp_avg"].copy_(torch.from_numpy(m))
    st["exp_avg_sq"].copy_(torch.from_numpy(v))
    if master_weights:
        st["master"].copy_(torch.from_numpy(pn))
    p.copy_(torch.from_numpy(pn))


def _net():
    torch.manual_seed(7)
    return torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.Tanh(), torch.nn.Linear(40, 40, bias=False),
                               torch.nn.Tanh(), torch.nn.Linear(40, 8))


def _data(step, rank):
    g = torch.Generator().manual_seed(100 + 10 * step + rank)
    return torch.randn(16, 24, generator=g), torch.randn(16, 8, generator=g)


HP = dict(lr=5e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)


def _worker(rank, world, port, q, master):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from bastile_b200.optim import ShardedAdamW

        net = _net()
        # bucket_mb=0: a bucket closes after every parameter -> several buckets, each padded and split
        opt = ShardedAdamW(net.parameters(), bucket_mb=0, master_weights=master, update_fn=_oracle_update, **HP)
        assert len(opt.buckets) == 5 and all(b.numel % (128 * world) == 0 for b in opt.buckets)
        assert all(p.data_ptr() == b.flat_p[o:].data_ptr() for b in opt.buckets for p, o in zip(b.params, b.offsets))
        for step in range(3):
            x, y = _data(step, rank)
            opt.zero_grad()
            if step == 2:  # the last layer's bias gets no gradient: its bucket is never launched
                out = net[:4](x)
                (out.pow(2).mean()).backward()
            else:
                torch.nn.functional.mse_loss(net(x), y).backward()
            assert all(p.grad is None for p in net.parameters())
            opt.step()
        final = [p.detach().clone() for p in net.parameters()]
        with pytest.raises(RuntimeError):  # two backward passes in one step
            x, y = _data(0, rank)
            torch.nn.functional.mse_loss(net[:2](x).sum(1, keepdim=True), y[:, :1]).backward()
            torch.nn.functional.mse_loss(net[:2](x).sum(1, keepdim=True), y[:, :1]).backward()
        q.put((rank, final, opt.state_bytes()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("master", [False, True])
def test_sharded_adamw_two_gloo_ranks_match_single_process(master):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, master)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted((q.get(timeout=120) for _ in procs), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0

    ref = _net()
    ropt = torch.optim.AdamW(ref.parameters(), **HP)
    for step in range(3):
        ropt.zero_grad(set_to_none=True)
        loss = 0.0
        for rank in range(world):
            x, y = _data(step, rank)
            if step == 2:
                loss = loss + ref[:4](x).pow(2).mean() / world
            else:
                loss = loss + torch.nn.functional.mse_loss(ref(x), y) / world
        loss.backward()
        ropt.step()
    for rank, params, state_bytes in results:
        for got, want in zip(params, ref.parameters()):
            np.testing.assert_allclose(got.numpy(), want.detach().numpy(), rtol=2e-5, atol=2e-6)
        total = sum(p.numel() for p in ref.parameters())
        per_elem = 12 if master else 8
        assert state_bytes < per_elem * (total / world + 5 * 128 * world)  # 1/N of the state, plus padding
    # every rank ends with the same parameters
    for a, b in zip(results[0][1], results[1][1]):
        assert torch.equal(a, b)


def test_bucket_plan_tapers_and_keeps_large_and_twin_tensors_apart_and_together():
    """Buckets fill in reverse registration order; the parameters whose gradients arrive last get
    quarter-size buckets, a tensor as large as a bucket sits alone, and two same-shaped neighbours
    (gate | up) are never split, so a stacked gradient finds both destinations side by side."""
    from bastile_b200.optim import ShardedAdamW

    def mat(rows):  # fp32 [rows, 1024] = 4 * rows KiB
        return torch.nn.Parameter(torch.zeros(rows, 1024))

    # "embedding" 5 MiB, then 8 "layers" of q 1 MiB | gate 1.5 | up 1.5 | norm, then "head" 5 MiB
    params = [mat(1280)]
    for _ in range(8):
        params += [mat(256), mat(384), mat(384), torch.nn.Parameter(torch.zeros(256))]
    params.append(mat(1280))
    opt = ShardedAdamW(params, bucket_mb=4, update_fn=lambda *a: None)
    try:
        index = {id(p): i for i, p in enumerate(params)}
        plan = [[index[id(p)] for p in b.params] for b in opt.buckets]
        sizes = [sum(params[i].numel() * 4 for i in b) for b in plan]
        assert plan[0] == [len(params) - 1] and plan[-1] == [0]          # head and embedding alone
        assert sorted(i for b in plan for i in b) == list(range(len(params)))
        for b in plan:                                                   # gate | up: same bucket, adjacent, in order
            for i in b:
                if params[i].shape == (384, 1024) and params[i - 1].shape == (384, 1024):
                    assert b[b.index(i) - 1] == i - 1
            assert b == sorted(b)                                        # registration order inside a bucket
        early = [s for s, b in zip(sizes[1:-1], plan[1:-1]) if min(b) > 16]
        late = [s for s, b in zip(sizes[1:-1], plan[1:-1]) if max(b) <= 4]
        assert early and len(late) >= 2 and max(late) < min(early)       # the tail's buckets are the small ones
        assert all(s >= 4 << 20 for s in early) and all(s < 4 << 20 for s in late)
        # every parameter is a view into its bucket at an aligned offset
        for b in opt.buckets:
            for p, o in zip(b.params, b.offsets):
                assert o % 128 == 0 and p.data_ptr() == b.flat_p[o:].data_ptr()
    finally:
        opt.close()
