"""The CPU oracle against the golden fixtures (reference / HF eager outputs) and
against torch autograd on the reference's own unit-test shapes.  CPU only."""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle
from conftest import assert_close, load_golden

TOL = dict(rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("name", ["loss_fp32", "grads", "ignore_index", "three_d", "sum", "all_ignored", "ragged"])
@pytest.mark.parametrize("n_shards", [1, 2])
def test_lce_oracle_matches_reference_fixture(name, n_shards):
    g = load_golden(f"lce_{name}.npz")
    v = g["w"].shape[0]
    if v % n_shards:
        pytest.skip("vocabulary not divisible")
    loss, dx, dw = oracle.lce_fwd_bwd(g["x"], g["w"], g["t"], -100, str(g["reduction"]), n_shards=n_shards)
    assert abs(float(loss) - float(g["loss"])) <= 1e-4 * max(1.0, abs(float(g["loss"])))
    assert_close(dx, g["dx"], what="dx", **TOL)
    assert_close(dw, g["dw"], what="dw", **TOL)


def test_rmsnorm_oracle_matches_hf_fixture():
    g = load_golden("rmsnorm_hf.npz")
    y, rstd = oracle.rms_norm_fwd(g["x"], g["w"], float(g["eps"]))
    assert_close(y, g["y"], what="y", **TOL)
    dx, dw = oracle.rms_norm_bwd(g["dy"], g["x"], g["w"], rstd)
    assert_close(dx, g["dx"], what="dx", **TOL)
    assert_close(dw, g["dw"], what="dw", rtol=1e-4, atol=1e-4)


def test_rope_oracle_matches_hf_fixture():
    g = load_golden("rope_hf.npz")
    qo, ko = oracle.rope(g["q"], g["k"], g["cos"], g["sin"])
    assert_close(qo, g["q_out"], what="q_out", **TOL)
    assert_close(ko, g["k_out"], what="k_out", **TOL)
    dq, dk = oracle.rope(g["dq_out"], g["dk_out"], g["cos"], g["sin"], negate_sin=True)
    assert_close(dq, g["dq"], what="dq", **TOL)
    assert_close(dk, g["dk"], what="dk", **TOL)


def test_rope_only_first_half_of_cos_sin_is_used():
    g = load_golden("rope_hf.npz")
    half = g["cos"].shape[-1] // 2
    a = oracle.rope(g["q"], g["k"], g["cos"], g["sin"])
    b = oracle.rope(g["q"], g["k"], g["cos"][..., :half], g["sin"][..., :half])
    np.testing.assert_array_equal(a[0], b[0])
    np.testing.assert_array_equal(a[1], b[1])


def test_mlp_oracle_matches_hf_fixture():
    g = load_golden("mlp_hf.npz")
    y, gate, up, h = oracle.mlp_fwd(g["x"], g["wg"], g["wu"], g["wd"])
    assert_close(y, g["y"], what="y", rtol=1e-4, atol=1e-4)
    dx, dwg, dwu, dwd = oracle.mlp_bwd(g["dy"], g["x"], g["wg"], g["wu"], g["wd"])
    for name, val in (("dx", dx), ("dwg", dwg), ("dwu", dwu), ("dwd", dwd)):
        assert_close(val, g[name], what=name, rtol=1e-4, atol=1e-4)
    # the elementwise op alone
    assert_close(oracle.swiglu_fwd(gate, up), h, what="h", **TOL)


# ---- the reference's unit-test shapes, against torch autograd ------------------------

def test_rmsnorm_reference_test_shapes():
    torch.manual_seed(0)
    x = torch.randn(4, 128, 1024)  # tests/ops/test_rms_norm.py:10-33
    w = torch.ones(1024)
    y, _ = oracle.rms_norm_fwd(x.numpy(), w.numpy(), 1e-6)
    ref = w * x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
    assert_close(y, ref, what="fwd", rtol=1e-3, atol=1e-3)
    x = torch.randn(2, 64, 512, requires_grad=True)  # :36-71
    w = torch.ones(512, requires_grad=True)
    (w * x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)).sum().backward()
    dx, dw = oracle.rms_norm_bwd(np.ones((2, 64, 512), np.float32), x.detach().numpy(), w.detach().numpy())
    assert_close(dx, x.grad, what="dx", rtol=1e-2, atol=1e-2)
    assert_close(dw, w.grad, what="dw", rtol=1e-3, atol=1e-3)


def test_swiglu_reference_test_shapes():
    torch.manual_seed(0)
    g = torch.randn(2, 32, 256, requires_grad=True)  # tests/ops/test_swiglu.py:32-59
    u = torch.randn(2, 32, 256, requires_grad=True)
    out = F.silu(g) * u
    out.sum().backward()
    assert_close(oracle.swiglu_fwd(g.detach().numpy(), u.detach().numpy()), out, what="fwd", rtol=1e-3, atol=1e-3)
    dg, du = oracle.swiglu_bwd(np.ones((2, 32, 256), np.float32), g.detach().numpy(), u.detach().numpy())
    assert_close(dg, g.grad, what="dgate", rtol=1e-2, atol=1e-2)
    assert_close(du, u.grad, what="dup", rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("reduction", ["mean", "sum"])
def test_lce_against_torch_autograd(reduction):
    torch.manual_seed(42)
    x = torch.randn(32, 256, requires_grad=True)  # tests/ops/test_fused_linear_cross_entropy.py:18-34
    w = torch.randn(1024, 256, requires_grad=True)
    t = torch.randint(0, 1024, (32,))
    t[::3] = -100
    loss = F.cross_entropy(F.linear(x, w), t, ignore_index=-100, reduction=reduction)
    loss.backward()
    l, dx, dw = oracle.lce_fwd_bwd(x.detach().numpy(), w.detach().numpy(), t.numpy(), -100, reduction, n_shards=4)
    assert abs(float(l) - loss.item()) <= 1e-3 * abs(loss.item())
    assert_close(dx, x.grad, what="dx", rtol=1e-3, atol=1e-4)  # torch side is fp32
    assert_close(dw, w.grad, what="dw", rtol=1e-3, atol=1e-4)


def test_tiny_qwen3_fixture_is_reproducible():
    """Seeded CPU construction of the tiny model gives the weights the fixture was made with."""
    from golden.make_golden import build_tiny_qwen3, tiny_qwen3_inputs

    g = load_golden("tiny_qwen3.npz")
    model = build_tiny_qwen3()
    ids, labels = tiny_qwen3_inputs()
    np.testing.assert_array_equal(ids.numpy(), g["ids"])
    np.testing.assert_array_equal(labels.numpy(), g["labels"])
    norms = np.array([p.norm().item() for p in model.parameters()])
    np.testing.assert_allclose(norms, g["param_norms"], rtol=1e-6)
    out = model(input_ids=ids, labels=labels)
    assert abs(out.loss.item() - float(g["loss"])) < 1e-5


def test_fused_oracle_forms_match_hf_eager_autograd():
    """The restatements of the fused forms (residual add + norm; q/k-norm + RoPE) against the HF
    eager modules they stand for, forward and autograd backward, in fp32 on the CPU - the same
    pin as for the four patched ops themselves."""
    import transformers.models.qwen3.modeling_qwen3 as q3

    torch.manual_seed(7)
    # residual + x -> Qwen3RMSNorm, gradient arriving on both the norm output and the stream
    m, n = 37, 256
    x = torch.randn(m, n, requires_grad=True)
    r = torch.randn(m, n, requires_grad=True)
    norm = q3.Qwen3RMSNorm(n, eps=1e-6)
    with torch.no_grad():
        norm.weight.copy_(1 + 0.1 * torch.randn(n))
    stream = r + x
    y = norm(stream)
    dy, ds = torch.randn(m, n), torch.randn(m, n)
    torch.autograd.backward([y, stream], [dy, ds])
    w = norm.weight.detach().numpy()
    y_o, s_o, rstd = oracle.add_rms_norm_fwd(x.detach().numpy(), r.detach().numpy(), w, 1e-6)
    dx_o, dw_o = oracle.add_rms_norm_bwd(dy.numpy(), ds.numpy(), s_o, w, rstd)
    assert_close(torch.as_tensor(y_o), y.detach().numpy(), what="y", rtol=1e-5, atol=1e-5)
    assert_close(torch.as_tensor(s_o), stream.detach().numpy(), what="stream", rtol=1e-6, atol=1e-6)
    assert_close(torch.as_tensor(dx_o), x.grad.numpy(), what="dx", rtol=1e-4, atol=1e-5)
    assert_close(torch.as_tensor(dx_o), r.grad.numpy(), what="dresidual", rtol=1e-4, atol=1e-5)
    assert_close(torch.as_tensor(dw_o), norm.weight.grad.numpy(), what="dw", rtol=1e-4, atol=1e-4)

    # q_norm / k_norm then apply_rotary_pos_emb, as Qwen3Attention.forward chains them
    b, t, h, d = 2, 19, 3, 64
    xq = torch.randn(b, t, h, d, requires_grad=True)
    qn = q3.Qwen3RMSNorm(d, eps=1e-6)
    with torch.no_grad():
        qn.weight.copy_(1 + 0.1 * torch.randn(d))
    inv = 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    emb = torch.outer(torch.arange(t, dtype=torch.float32), inv)
    emb = torch.cat((emb, emb), -1)
    cos, sin = emb.cos()[None].expand(b, -1, -1), emb.sin()[None].expand(b, -1, -1)
    q_rot, _ = q3.apply_rotary_pos_emb(qn(xq).transpose(1, 2), torch.zeros(b, 1, t, d), cos, sin)
    dq = torch.randn(b, h, t, d)
    q_rot.backward(dq)
    wq = qn.weight.detach().numpy()
    o_o, _ = oracle.head_norm_rope_fwd(xq.detach().numpy(), wq, cos.numpy(), sin.numpy(), 1e-6)
    dx_o, dw_o = oracle.head_norm_rope_bwd(dq.transpose(1, 2).numpy(), xq.detach().numpy(), wq, cos.numpy(),
                                           sin.numpy(), 1e-6)
    assert_close(torch.as_tensor(o_o), q_rot.detach().transpose(1, 2).numpy(), what="q rotated", rtol=1e-5, atol=1e-5)
    assert_close(torch.as_tensor(dx_o), xq.grad.numpy(), what="dq", rtol=1e-4, atol=1e-5)
    assert_close(torch.as_tensor(dw_o), qn.weight.grad.numpy(), what="dw", rtol=1e-4, atol=1e-4)
