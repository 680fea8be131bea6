"""Vocabulary-parallel fused loss on 2 GPUs over NCCL (skipped with fewer): every rank holds half
of the lm_head rows, results must equal the single-GPU op and the oracle."""

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import oracle
        from bastile_b200 import _lib
        from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy

        g = torch.Generator().manual_seed(3)  # identical inputs on every rank
        bt, h, v = 700, 256, 3040  # 1520 columns per rank: ragged 256-wide tiles
        x = torch.randn(bt, h, generator=g).to(dev, torch.bfloat16)
        w = (torch.randn(v, h, generator=g) * 0.05).to(dev, torch.bfloat16)
        t = torch.randint(0, v, (bt,), generator=g).to(dev)
        t[::11] = -100
        vs = v // world
        xs = x.clone().requires_grad_(True)
        wl = w[rank * vs:(rank + 1) * vs].clone().requires_grad_(True)
        loss = fused_linear_cross_entropy(xs, wl, t, chunk_size=256, vocab_parallel_group=dist.group.WORLD,
                                          vocab_start=rank * vs)
        loss.backward()
        _lib.check_status(dev, "vocab-parallel loss")
        l_ref, dx_ref, dw_ref = oracle.lce_fwd_bwd(x.float().cpu().numpy(), w.float().cpu().numpy(), t.cpu().numpy(),
                                                   -100, "mean")
        sx, sw = float(np.abs(dx_ref).max()), float(np.abs(dw_ref).max())
        ok_loss = abs(loss.item() - float(l_ref)) <= 2e-3 * abs(float(l_ref))
        ok_dx = np.allclose(xs.grad.float().cpu().numpy(), dx_ref, rtol=2e-2, atol=2e-2 * sx)
        ok_dw = np.allclose(wl.grad.float().cpu().numpy(), dw_ref[rank * vs:(rank + 1) * vs], rtol=2e-2, atol=2e-2 * sw)
        # token-sharded form: every rank brings its own half of the rows
        half = bt // world
        xs2 = x[rank * half:(rank + 1) * half].clone().requires_grad_(True)
        wl2 = w[rank * vs:(rank + 1) * vs].clone().requires_grad_(True)
        loss2 = fused_linear_cross_entropy(xs2, wl2, t[rank * half:(rank + 1) * half], chunk_size=256,
                                           vocab_parallel_group=dist.group.WORLD, vocab_start=rank * vs,
                                           shard_tokens=True, grad_hidden_scale=2.0)
        loss2.backward()
        _lib.check_status(dev, "token-sharded vocab-parallel loss")
        ok_loss &= abs(loss2.item() - float(l_ref)) <= 2e-3 * abs(float(l_ref))
        ok_dx &= np.allclose(xs2.grad.float().cpu().numpy(), 2.0 * dx_ref[rank * half:(rank + 1) * half], rtol=2e-2,
                             atol=4e-2 * sx)
        ok_dw &= np.allclose(wl2.grad.float().cpu().numpy(), dw_ref[rank * vs:(rank + 1) * vs], rtol=2e-2, atol=2e-2 * sw)
        # chunks that lie inside one rank's block of rows: every chunk's d(hidden) is reduced to its owner
        # while the next chunk computes (175 divides the 350 rows a rank brings)
        xs3 = x[rank * half:(rank + 1) * half].clone().requires_grad_(True)
        wl3 = w[rank * vs:(rank + 1) * vs].clone().requires_grad_(True)
        loss3 = fused_linear_cross_entropy(xs3, wl3, t[rank * half:(rank + 1) * half], chunk_size=175,
                                           vocab_parallel_group=dist.group.WORLD, vocab_start=rank * vs,
                                           shard_tokens=True, grad_hidden_scale=1.0, vocab_size=v)
        loss3.backward()
        _lib.check_all_status()
        ok_loss &= abs(loss3.item() - float(l_ref)) <= 2e-3 * abs(float(l_ref))
        ok_dx &= np.allclose(xs3.grad.float().cpu().numpy(), dx_ref[rank * half:(rank + 1) * half], rtol=2e-2,
                             atol=2e-2 * sx)
        ok_dw &= np.allclose(wl3.grad.float().cpu().numpy(), dw_ref[rank * vs:(rank + 1) * vs], rtol=2e-2, atol=2e-2 * sw)
        q.put((rank, ok_loss, ok_dx, ok_dw, loss.item(), float(l_ref)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_vocab_parallel_loss_two_gpus_nccl():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok_loss, ok_dx, ok_dw, loss, ref in results:
        assert ok_loss and ok_dx and ok_dw, f"rank {rank}: loss {loss} vs {ref}; dx {ok_dx} dw {ok_dw}"
