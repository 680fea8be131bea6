"""AdamW: the numpy oracle against torch.optim.AdamW on CPU, and the CUDA kernel against both."""

import numpy as np
import pytest
import torch

import oracle
from conftest import assert_close


def test_oracle_matches_torch_adamw_cpu():
    torch.manual_seed(0)
    p = torch.randn(257, dtype=torch.float64, requires_grad=True)
    opt = torch.optim.AdamW([p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    pn, m, v = p.detach().numpy().copy(), np.zeros(257), np.zeros(257)
    for step in range(1, 5):
        g = torch.randn(257, dtype=torch.float64)
        p.grad = g.clone()
        opt.step()
        pn, m, v = oracle.adamw_step(pn, g.numpy(), m, v, step, 1e-2, 0.9, 0.95, 1e-8, 0.1)
        np.testing.assert_allclose(p.detach().numpy(), pn, rtol=1e-12, atol=1e-12)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cuda_adamw_matches_oracle_and_torch(dtype):
    from bastile_b200.optim import AdamW

    torch.manual_seed(1)
    shapes = [(4096,), (128,), (300, 1000), (1024, 4096), (7,), (65536,), (65537,)]
    params = [torch.randn(s, device="cuda").to(dtype).requires_grad_(True) for s in shapes]
    ref_params = [p.detach().clone().requires_grad_(True) for p in params]
    hp = dict(lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.05)
    ours, ref = AdamW(params, **hp), torch.optim.AdamW(ref_params, **hp)
    state = [(p.detach().double().cpu().numpy(), np.zeros(s), np.zeros(s)) for p, s in zip(params, shapes)]
    for step in range(1, 4):
        for i, (p, r) in enumerate(zip(params, ref_params)):
            g = torch.randn_like(p)
            p.grad, r.grad = g.clone(), g.clone()
            if dtype == torch.float32:
                state[i] = oracle.adamw_step(*state[i][:1], g.double().cpu().numpy(), *state[i][1:], step, hp["lr"], 0.9,
                                             0.95, 1e-8, 0.05)
        ours.step()
        ref.step()
    for i, (p, r) in enumerate(zip(params, ref_params)):
        if dtype == torch.float32:
            assert_close(p, state[i][0], what=f"param {i} vs oracle", rtol=1e-5, atol=1e-6)
            assert_close(ours.state[p]["exp_avg_sq"], state[i][2], what=f"v {i}", rtol=1e-5, atol=1e-7)
            assert_close(p, r, what=f"param {i} vs torch", rtol=1e-5, atol=1e-6)
        else:  # bf16 storage: one ulp of rounding per step on both sides
            assert_close(p, r, what=f"param {i} vs torch", rtol=2e-2, atol=2e-2)
            assert_close(ours.state[p]["exp_avg"], ref.state[r]["exp_avg"], what=f"m {i}", rtol=2e-2, atol=2e-3)
    assert set(ours.state[params[0]]) == {"step", "exp_avg", "exp_avg_sq"}


@pytest.mark.gpu
def test_overlap_backward_gives_the_same_bits_as_the_plain_step():
    """Updates queued from post-accumulate-grad hooks on a side stream (large tensors) plus the
    rest in step(): every parameter and moment ends up bit-identical to the plain optimizer."""
    from bastile_b200.optim import _OVERLAP_MIN_NUMEL, AdamW

    def build():
        torch.manual_seed(3)
        return torch.nn.Sequential(torch.nn.Linear(1024, 2048, bias=True), torch.nn.GELU(),
                                   torch.nn.Linear(2048, 1024, bias=False), torch.nn.LayerNorm(1024),
                                   torch.nn.Linear(1024, 1024, bias=False)).cuda().to(torch.bfloat16)

    nets = [build(), build()]
    assert any(p.numel() >= _OVERLAP_MIN_NUMEL for p in nets[0].parameters())
    assert any(p.numel() < _OVERLAP_MIN_NUMEL for p in nets[0].parameters())
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opts = [AdamW(nets[0].parameters(), **hp), AdamW(nets[1].parameters(), overlap_backward=True, **hp)]
    torch.manual_seed(4)
    xs = [torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16) for _ in range(4)]
    for x in xs:
        for net, opt in zip(nets, opts):
            opt.zero_grad(set_to_none=True)
            net(x).float().pow(2).mean().backward()
            opt.step()
    assert len(opts[1]._early) == 0 and len(opts[1]._side_streams) == 1
    torch.cuda.synchronize()
    for (name, a), b in zip(nets[0].named_parameters(), nets[1].parameters()):
        assert torch.equal(a, b), name
        assert torch.equal(opts[0].state[a]["exp_avg"], opts[1].state[b]["exp_avg"]), name
        assert torch.equal(opts[0].state[a]["exp_avg_sq"], opts[1].state[b]["exp_avg_sq"]), name
        assert opts[0].state[a]["step"] == opts[1].state[b]["step"] == len(xs)
    with pytest.raises(RuntimeError):
        opts[1].step(closure=lambda: None)


def test_overlap_backward_is_inert_without_cuda_gradients():
    """On CPU tensors the hooks do nothing (and the optimizer refuses the step as before)."""
    from bastile_b200.optim import AdamW

    w = torch.nn.Parameter(torch.randn(2048, 1024))
    opt = AdamW([w], overlap_backward=True)
    (w * w).sum().backward()
    assert not opt._early and not opt._side_streams
    with pytest.raises(RuntimeError):
        opt.step()


@pytest.mark.gpu
def test_overlap_backward_with_tied_weights_matches_plain_step_bit_for_bit():
    """A weight used twice in the graph (tied embedding / output projection): autograd sums both
    contributions before the single accumulation that fires the hook, so the early update sees the
    complete gradient."""
    from bastile_b200.optim import _OVERLAP_MIN_NUMEL, AdamW

    class Tied(torch.nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(5)
            self.emb = torch.nn.Embedding(2048, 1024)
            self.mid = torch.nn.Linear(1024, 1024, bias=False)

        def forward(self, ids):
            return torch.nn.functional.linear(torch.tanh(self.mid(self.emb(ids))), self.emb.weight)

    nets = [Tied().cuda().to(torch.bfloat16), Tied().cuda().to(torch.bfloat16)]
    assert nets[0].emb.weight.numel() >= _OVERLAP_MIN_NUMEL
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opts = [AdamW(nets[0].parameters(), **hp), AdamW(nets[1].parameters(), overlap_backward=True, **hp)]
    torch.manual_seed(6)
    for _ in range(3):
        ids = torch.randint(0, 2048, (4, 64), device="cuda")
        for net, opt in zip(nets, opts):
            opt.zero_grad(set_to_none=True)
            torch.nn.functional.cross_entropy(net(ids).float().view(-1, 2048), ids.view(-1)).backward()
            opt.step()
    torch.cuda.synchronize()
    for (name, a), b in zip(nets[0].named_parameters(), nets[1].parameters()):
        assert torch.equal(a, b), name
    # a second backward pass before step() is refused, not silently half-applied
    ids = torch.randint(0, 2048, (4, 64), device="cuda")
    opts[1].zero_grad(set_to_none=True)
    torch.nn.functional.cross_entropy(nets[1](ids).float().view(-1, 2048), ids.view(-1)).backward()
    with pytest.raises(RuntimeError):
        torch.nn.functional.cross_entropy(nets[1](ids).float().view(-1, 2048), ids.view(-1)).backward()
    opts[1].step()


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1 << 20, 4099, 7])
def test_cuda_adamw_master_weights_match_oracle(n):
    """bf16 parameter / gradient, fp32 master and moments (bt_adamw_master_step) against the float64 oracle."""
    from bastile_b200.optim import AdamW

    torch.manual_seed(8)
    p = torch.randn(n, device="cuda").to(torch.bfloat16).requires_grad_(True)
    hp = dict(lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.05)
    opt = AdamW([p], master_weights=True, **hp)
    pn, m, v = p.detach().double().cpu().numpy(), np.zeros(n), np.zeros(n)
    for step in range(1, 5):
        g = torch.randn(n, device="cuda").to(torch.bfloat16)
        p.grad = g.clone()
        opt.step()
        pn, m, v = oracle.adamw_step(pn, g.double().cpu().numpy(), m, v, step, hp["lr"], 0.9, 0.95, 1e-8, 0.05)
    st = opt.state[p]
    assert set(st) == {"step", "exp_avg", "exp_avg_sq", "master"} and st["master"].dtype == torch.float32
    assert_close(st["master"], pn, what="master", rtol=1e-5, atol=1e-6)
    assert_close(st["exp_avg"], m, what="m", rtol=1e-5, atol=1e-7)
    assert_close(st["exp_avg_sq"], v, what="v", rtol=1e-5, atol=1e-7)
    assert torch.equal(p.detach(), st["master"].to(torch.bfloat16))  # the 16-bit copy is the rounded master


@pytest.mark.gpu
@pytest.mark.parametrize("master", [False, True])
def test_sharded_adamw_single_rank_matches_plain_adamw(master):
    """One rank: ShardedAdamW is a flat, overlapped AdamW - same bits as AdamW on the same model."""
    from bastile_b200.optim import AdamW, ShardedAdamW

    def build():
        torch.manual_seed(9)
        return torch.nn.Sequential(torch.nn.Linear(1024, 2048, bias=True), torch.nn.GELU(),
                                   torch.nn.Linear(2048, 1024, bias=False), torch.nn.LayerNorm(1024),
                                   torch.nn.Linear(1024, 512, bias=False)).cuda().to(torch.bfloat16)

    nets = [build(), build()]
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opts = [AdamW(nets[0].parameters(), master_weights=master, **hp),
            ShardedAdamW(nets[1].parameters(), bucket_mb=4, master_weights=master, **hp)]
    assert len(opts[1].buckets) >= 2
    torch.manual_seed(10)
    for _ in range(4):
        x = torch.randn(256, 1024, device="cuda", dtype=torch.bfloat16)
        for net, opt in zip(nets, opts):
            opt.zero_grad(set_to_none=True)
            net(x).float().pow(2).mean().backward()
            opt.step()
    torch.cuda.synchronize()
    for (name, a), b in zip(nets[0].named_parameters(), nets[1].parameters()):
        if a.numel() > 65536:  # both sides take the 16-byte vector path: same instructions, same bits
            assert torch.equal(a, b), name
        else:  # AdamW batches small tensors into a scalar kernel whose fp32 contraction may differ by an ulp
            assert_close(a, b, what=name, rtol=1e-2, atol=1e-3)
    opts[1].close()


@pytest.mark.gpu
def test_sharded_adamw_gradient_sinks_are_written_directly():
    """The MLP block and the fused loss write their weight gradients straight into ShardedAdamW's
    flat buckets (no copy in the hook); parameters after a few steps equal the plain optimizer's."""
    from types import SimpleNamespace

    from bastile_b200 import _lib
    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy
    from bastile_b200.ops.swiglu import B200SwiGLUMLP
    from bastile_b200.optim import AdamW, ShardedAdamW

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(14)
            self.mlp = B200SwiGLUMLP(SimpleNamespace(hidden_size=256, intermediate_size=768, hidden_act="silu"))
            self.head = torch.nn.Linear(256, 1000, bias=False)

        def forward(self, x, y):
            return fused_linear_cross_entropy(x + self.mlp(x), self.head.weight, y)

    nets = [Net().cuda().to(torch.bfloat16), Net().cuda().to(torch.bfloat16)]
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    # one bucket: gate | up lie back to back in it, so the stacked dWg | dWu product can go there too
    opts = [AdamW(nets[0].parameters(), **hp), ShardedAdamW(nets[1].parameters(), bucket_mb=64, **hp)]
    seen = []
    orig = opts[1]._on_grad

    def spy(p):
        b, i = opts[1]._where[p]
        seen.append(p.grad.data_ptr() == b.flat_g[b.offsets[i]:].data_ptr())
        orig(p)

    for h in opts[1]._hooks:
        h.remove()
    opts[1]._hooks = [p.register_post_accumulate_grad_hook(spy) for p in nets[1].parameters()]
    torch.manual_seed(15)
    for _ in range(3):
        x = torch.randn(300, 256, device="cuda", dtype=torch.bfloat16)
        y = torch.randint(0, 1000, (300,), device="cuda")
        for net, opt in zip(nets, opts):
            opt.zero_grad(set_to_none=True)
            net(x, y).backward()
            opt.step()
    _lib.check_all_status()
    assert sum(seen) == len(seen) == 3 * 4, f"gradients written in place: {sum(seen)} of {len(seen)}"  # gate, up, down, head
    for (name, a), b in zip(nets[0].named_parameters(), nets[1].parameters()):
        assert_close(a, b, what=name, rtol=1e-2, atol=1e-3)
    opts[1].close()
    assert not any(id(v) in {id(d) for bk in opts[1].buckets for d in bk.sinks} for v in _lib._grad_sinks.values())


@pytest.mark.gpu
def test_sharded_single_rank_whole_model_projection_gradients_land_in_the_buckets():
    """A small Qwen3 under apply(fused_layers=True) (projections in "acc" mode) with ShardedAdamW:
    the weight gradients of q/k/v/o, gate/up/down and lm_head are written where the optimizer
    reduces them, without a copy, and training matches the plain optimizer on unfused projections."""
    from transformers import Qwen3Config, Qwen3ForCausalLM

    import bastile_b200
    from bastile_b200 import _lib
    from bastile_b200.optim import AdamW, ShardedAdamW

    cfg = Qwen3Config(vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6,
                      tie_word_embeddings=False, use_cache=False)
    cfg._attn_implementation = "sdpa"
    hp = dict(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ids = [torch.randint(0, 1024, (2, 64), generator=torch.Generator().manual_seed(s)).cuda() for s in (1, 2, 3)]
    finals, in_place, first_grads = {}, {}, {"off": {}, "acc": {}}
    try:
        for mode in ("off", "acc"):
            bastile_b200.reset()
            bastile_b200.apply(fused_layers=True, gemm_projections=mode)
            torch.manual_seed(9)
            model = Qwen3ForCausalLM(cfg).cuda().to(torch.bfloat16).train()
            if mode == "off":
                opt = AdamW(model.parameters(), **hp)
            else:
                opt = ShardedAdamW(model.parameters(), bucket_mb=64, **hp)
                names = {p: n for n, p in model.named_parameters()}
                orig = opt._on_grad

                def spy(p, opt=opt, names=names, orig=orig):
                    b, i = opt._where[p]
                    in_place.setdefault(names[p], []).append(p.grad.data_ptr() == b.flat_g[b.offsets[i]:].data_ptr())
                    first_grads["acc"].setdefault(names[p], p.grad.detach().float().clone())
                    orig(p)

                for h in opt._hooks:
                    h.remove()
                opt._hooks = [p.register_post_accumulate_grad_hook(spy) for p in model.parameters()]
            for step, x in enumerate(ids):
                opt.zero_grad(set_to_none=True)
                model(input_ids=x, labels=x).loss.backward()
                if mode == "off" and step == 0:
                    first_grads["off"] = {n: p.grad.detach().float().clone() for n, p in model.named_parameters()}
                opt.step()
            _lib.check_all_status()
            finals[mode] = {n: p.detach().float().clone() for n, p in model.named_parameters()}
            opt.close()
    finally:
        bastile_b200.reset()
    for n, hits in in_place.items():
        if n.endswith(("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "down_proj.weight",
                       "lm_head.weight")):
            assert all(hits) and len(hits) == 3, (n, hits)
    assert set(first_grads["acc"]) == set(first_grads["off"])
    for n, g in first_grads["off"].items():  # same weights, same batch: the gradients of the first step
        assert_close(first_grads["acc"][n], g.cpu().numpy(), what=f"grad {n}", rtol=2e-2,
                     atol=2e-2 * float(g.abs().max()) + 1e-6)
    for n in finals["off"]:  # three Adam steps move an element by at most 3 * lr whatever its gradient
        assert_close(finals["acc"][n], finals["off"][n].cpu().numpy(), what=n, rtol=2e-2, atol=8e-3)
