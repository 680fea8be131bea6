"""ShardedAdamW on 2 GPUs over NCCL (skipped with fewer): reduce-scatter / update / all-gather of
every bucket queued underneath the backward pass must give what DistributedDataParallel followed by
the plain AdamW step gives."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _net(dtype):
    torch.manual_seed(11)
    return torch.nn.Sequential(torch.nn.Linear(512, 1024, bias=True), torch.nn.GELU(),
                               torch.nn.Linear(1024, 1024, bias=False), torch.nn.LayerNorm(1024),
                               torch.nn.Linear(1024, 256, bias=False)).cuda().to(dtype)


def _worker(rank, world, port, q, dtype_name, master):
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from bastile_b200.optim import AdamW, ShardedAdamW

        dtype = getattr(torch, dtype_name)
        hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
        a, b = _net(dtype), _net(dtype)
        ddp = DDP(a, device_ids=[rank])
        opt_a = AdamW(a.parameters(), master_weights=master, **hp)
        opt_b = ShardedAdamW(b.parameters(), bucket_mb=1, master_weights=master, group=dist.group.WORLD, **hp)
        assert len(opt_b.buckets) >= 2
        g = torch.Generator(device=dev).manual_seed(50 + rank)  # different data per rank
        for _ in range(4):
            x = torch.randn(128, 512, device=dev, generator=g).to(dtype)
            opt_a.zero_grad(set_to_none=True)
            ddp(x).float().pow(2).mean().backward()
            opt_a.step()
            opt_b.zero_grad()
            b(x).float().pow(2).mean().backward()
            opt_b.step()
        torch.cuda.synchronize()
        worst = 0.0
        for pa, pb in zip(a.parameters(), b.parameters()):
            scale = float(pa.detach().float().abs().max()) + 1e-12
            worst = max(worst, float((pa.detach().float() - pb.detach().float()).abs().max()) / scale)
        # every rank holds the same parameters after the all-gather
        flat = torch.cat([p.detach().float().flatten() for p in b.parameters()])
        other = flat.clone()
        dist.broadcast(other, src=0)
        same = bool(torch.equal(flat, other))
        q.put((rank, worst, same))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("dtype_name,master,tol", [("float32", False, 1e-4), ("bfloat16", False, 2e-2),
                                                   ("bfloat16", True, 2e-2)])
def test_sharded_adamw_two_gpus_matches_ddp(dtype_name, master, tol):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, dtype_name, master)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, worst, same in results:
        assert same, f"rank {rank}: parameters differ between ranks after the all-gather"
        assert worst <= tol, f"rank {rank}: worst relative parameter difference {worst}"
