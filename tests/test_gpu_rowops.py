"""RMSNorm, RoPE and elementwise SwiGLU kernels through the C ABI, against the CPU oracle,
the golden fixtures and the reference's own unit-test shapes/tolerances."""

import numpy as np
import pytest
import torch

import oracle
from conftest import BF16_TOL, FP32_TOL, assert_close, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _t(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=torch.float32).to(DEV, dtype)


# ------------------------------------------------------------------------ RMSNorm
@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, BF16_TOL), (torch.float16, BF16_TOL)])
@pytest.mark.parametrize("m,n", [(1, 8), (5, 64), (37, 128), (300, 128), (64, 192), (33, 1024), (130, 2048),
                                 (67, 4096), (9, 8192), (3, 5120), (4, 100), (7, 4099), (2, 16384), (0, 128)])
def test_rmsnorm_fwd_bwd_vs_oracle(m, n, dtype, tol):
    from bastile_b200.ops.rms_norm import rms_norm

    torch.manual_seed(m * 1000 + n)
    x = torch.randn(m, n, device=DEV).to(dtype).requires_grad_(True)
    w = (1 + 0.02 * torch.randn(n, device=DEV)).to(dtype).requires_grad_(True)
    dy = torch.randn(m, n, device=DEV).to(dtype)
    y = rms_norm(x, w, eps=1e-6)
    y.backward(dy)
    xo, wo, dyo = (t.detach().float().cpu().numpy() for t in (x, w, dy))
    y_ref, rstd = oracle.rms_norm_fwd(xo, wo, 1e-6)
    dx_ref, dw_ref = oracle.rms_norm_bwd(dyo, xo, wo, rstd)
    assert y.dtype == dtype and x.grad.dtype == dtype and w.grad.dtype == dtype
    assert_close(y, y_ref, what="y", **tol)
    assert_close(x.grad, dx_ref, what="dx", **tol)
    # dw sums m rounded products: allow the 16-bit rounding of the result plus accumulation noise
    dw_tol = dict(rtol=tol["rtol"], atol=max(tol["atol"], 2e-2 * np.sqrt(max(m, 1)) if dtype != torch.float32 else 1e-4))
    assert_close(w.grad, dw_ref, what="dw", **dw_tol)


def test_rmsnorm_golden_hf_fixture():
    from bastile_b200.ops.rms_norm import rms_norm

    g = load_golden("rmsnorm_hf.npz")
    x = _t(g["x"]).requires_grad_(True)
    w = _t(g["w"]).requires_grad_(True)
    y = rms_norm(x, w, eps=float(g["eps"]))
    y.backward(_t(g["dy"]))
    assert_close(y, g["y"], what="y", **FP32_TOL)
    assert_close(x.grad, g["dx"], what="dx", **FP32_TOL)
    assert_close(w.grad, g["dw"], what="dw", rtol=1e-4, atol=1e-4)


def test_rmsnorm_reference_unit_tests():
    """tests/ops/test_rms_norm.py of the reference, same shapes and tolerances."""
    from bastile_b200.ops.rms_norm import rms_norm

    x = torch.randn(4, 128, 1024, device=DEV)
    w = torch.ones(1024, device=DEV)
    ref = w * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6))
    torch.testing.assert_close(rms_norm(x, w, eps=1e-6), ref, rtol=1e-3, atol=1e-3)

    x = torch.randn(2, 64, 512, device=DEV, requires_grad=True)
    w = torch.ones(512, device=DEV, requires_grad=True)
    rms_norm(x, w, eps=1e-6).sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    (wr * (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6))).sum().backward()
    torch.testing.assert_close(x.grad, xr.grad, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(w.grad, wr.grad, rtol=1e-2, atol=1e-2)

    x = torch.randn(128, 2048, device=DEV, dtype=torch.bfloat16)
    w = torch.ones(2048, device=DEV, dtype=torch.bfloat16)
    ref = (w.float() * (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6))).to(x.dtype)
    torch.testing.assert_close(rms_norm(x, w, eps=1e-6), ref, rtol=1e-2, atol=1e-2)


def test_rmsnorm_strided_rows_and_4d_input():
    from bastile_b200.ops.rms_norm import rms_norm

    torch.manual_seed(5)
    big = torch.randn(50, 512, device=DEV, dtype=torch.bfloat16)
    x = big[:, :128]  # row stride 512
    w = torch.ones(128, device=DEV, dtype=torch.bfloat16)
    y_ref, _ = oracle.rms_norm_fwd(x.float().cpu().numpy(), w.float().cpu().numpy())
    assert_close(rms_norm(x, w), y_ref, what="strided", **BF16_TOL)
    x4 = torch.randn(2, 9, 8, 128, device=DEV, dtype=torch.bfloat16)  # q_norm layout [B,T,heads,128]
    y4_ref, _ = oracle.rms_norm_fwd(x4.float().cpu().numpy(), w.float().cpu().numpy())
    assert_close(rms_norm(x4, w), y4_ref, what="4d", **BF16_TOL)


def test_rmsnorm_bwd_scratch_is_left_zero_and_reusable():
    from bastile_b200 import _lib
    from bastile_b200.ops.rms_norm import rms_norm

    outs = []
    for _ in range(3):
        torch.manual_seed(9)
        x = torch.randn(257, 4096, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        w = torch.ones(4096, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        rms_norm(x, w).sum().backward()
        outs.append(w.grad.float().clone())
    ws = _lib.zero_workspace(torch.device(DEV, torch.cuda.current_device()), 16)
    torch.cuda.synchronize()
    assert int(ws.count_nonzero()) == 0
    assert_close(outs[1], outs[0], what="rerun", rtol=1e-2, atol=1e-1)
    assert_close(outs[2], outs[0], what="rerun", rtol=1e-2, atol=1e-1)


def test_rmsnorm_full_size_properties():
    """Per-op benchmark shape x[8192,4096] bf16: scale equivariance and unit RMS of y/w."""
    from bastile_b200.ops.rms_norm import rms_norm

    torch.manual_seed(1)
    x = torch.randn(8192, 4096, device=DEV, dtype=torch.bfloat16)
    w = (1 + 0.02 * torch.randn(4096, device=DEV)).to(torch.bfloat16)
    y = rms_norm(x, w, eps=1e-6)
    rms = (y.float() / w.float()).pow(2).mean(-1).sqrt()
    assert float((rms - 1).abs().max()) < 2e-2
    y2 = rms_norm(x * 4, w, eps=1e-6)  # exact power-of-two scaling of the input leaves y unchanged
    assert float((y2.float() - y.float()).abs().max()) <= 2e-2
    idx = torch.randint(0, 8192, (64,), device=DEV)
    y_ref, _ = oracle.rms_norm_fwd(x[idx].float().cpu().numpy(), w.float().cpu().numpy())
    assert_close(y[idx], y_ref, what="rows", **BF16_TOL)


# --------------------------------------------------------------------------- RoPE
def _cos_sin(t, d, theta=1e6, dtype=torch.float32, batch=1):
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    emb = torch.outer(torch.arange(t, dtype=torch.float32), inv)
    emb = torch.cat((emb, emb), -1)
    return (emb.cos()[None].expand(batch, -1, -1).contiguous().to(DEV, dtype),
            emb.sin()[None].expand(batch, -1, -1).contiguous().to(DEV, dtype))


def test_rope_golden_hf_fixture_fwd_bwd():
    from bastile_b200.ops.rope import apply_rotary_pos_emb

    g = load_golden("rope_hf.npz")
    q = _t(g["q"]).requires_grad_(True)
    k = _t(g["k"]).requires_grad_(True)
    qo, ko = apply_rotary_pos_emb(q.clone(), k.clone(), _t(g["cos"]), _t(g["sin"]))
    assert_close(qo, g["q_out"], what="q_out", **FP32_TOL)
    assert_close(ko, g["k_out"], what="k_out", **FP32_TOL)
    qc, kc = q * 1.0, k * 1.0  # non-leaf copies that the op may overwrite in place
    qo, ko = apply_rotary_pos_emb(qc, kc, _t(g["cos"]), _t(g["sin"]))
    torch.autograd.backward([qo, ko], [_t(g["dq_out"]), _t(g["dk_out"])])
    assert_close(q.grad, g["dq"], what="dq", **FP32_TOL)
    assert_close(k.grad, g["dk"], what="dk", **FP32_TOL)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_TOL), (torch.bfloat16, BF16_TOL), (torch.float16, BF16_TOL)])
@pytest.mark.parametrize("b,hq,hk,t,d,hf_layout", [(2, 8, 8, 64, 64, False), (1, 32, 8, 130, 128, True),
                                                   (3, 5, 3, 17, 128, True), (2, 4, 2, 9, 24, False), (1, 1, 1, 1, 2, False)])
def test_rope_vs_oracle_inplace_and_strided(b, hq, hk, t, d, hf_layout, dtype, tol):
    from bastile_b200.ops.rope import apply_rotary_pos_emb

    torch.manual_seed(b + hq + t + d)
    if hf_layout:  # [B,T,H,D] storage handed over as a transposed [B,H,T,D] view
        q = torch.randn(b, t, hq, d, device=DEV).to(dtype).transpose(1, 2)
        k = torch.randn(b, t, hk, d, device=DEV).to(dtype).transpose(1, 2)
    else:
        q = torch.randn(b, hq, t, d, device=DEV).to(dtype)
        k = torch.randn(b, hk, t, d, device=DEV).to(dtype)
    cos, sin = _cos_sin(t, d, dtype=dtype)
    q_ref, k_ref = oracle.rope(q.float().cpu().numpy(), k.float().cpu().numpy(), cos.float().cpu().numpy(),
                               sin.float().cpu().numpy())
    qo, ko = apply_rotary_pos_emb(q, k, cos, sin)
    assert qo.shape == q.shape and ko.shape == k.shape
    assert_close(qo, q_ref, what="q", **tol)
    assert_close(ko, k_ref, what="k", **tol)
    # rotated in place, like the reference
    assert qo.data_ptr() == q.data_ptr() and ko.data_ptr() == k.data_ptr()
    # forward followed by the backward rotation (sin negated) is the identity up to rounding
    q0 = q_ref.copy()
    dq, dk = oracle.rope(q0, k_ref, cos.float().cpu().numpy(), sin.float().cpu().numpy(), negate_sin=True)
    assert np.isfinite(dq).all() and np.isfinite(dk).all()


def test_rope_reference_unit_tests():
    """tests/ops/test_rope.py: shapes preserved, finite grads, random cos/sin of shape [B,T,D]."""
    from bastile_b200.ops.rope import apply_rotary_pos_emb

    q = torch.randn(2, 4, 32, 64, device=DEV, requires_grad=True)
    k = torch.randn(2, 4, 32, 64, device=DEV, requires_grad=True)
    cos = torch.randn(2, 32, 64, device=DEV)
    sin = torch.randn(2, 32, 64, device=DEV)
    qn, kn, cn, sn = (a.detach().cpu().numpy().copy() for a in (q, k, cos, sin))
    qo, ko = apply_rotary_pos_emb(q * 1.0, k * 1.0, cos, sin)
    assert qo.shape == q.shape and ko.shape == k.shape
    q_ref, k_ref = oracle.rope(qn, kn, cn, sn)  # per-batch cos/sin, first half only
    assert_close(qo, q_ref, what="q", **FP32_TOL)
    (qo.sum() + ko.sum()).backward()
    assert torch.isfinite(q.grad).all() and torch.isfinite(k.grad).all()
    dq_ref, dk_ref = oracle.rope(np.ones_like(qn), np.ones_like(kn), cn, sn, negate_sin=True)
    assert_close(q.grad, dq_ref, what="dq", **FP32_TOL)
    assert_close(k.grad, dk_ref, what="dk", **FP32_TOL)


def test_rope_full_size_roundtrip():
    """Benchmark shape q[1,32,8192,128], k[1,8,8192,128]: norm preservation and fwd->bwd round trip."""
    from bastile_b200 import _lib
    from bastile_b200.ops.rope import _launch

    torch.manual_seed(1)
    q = torch.randn(1, 32, 8192, 128, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(1, 8, 8192, 128, device=DEV, dtype=torch.bfloat16)
    cos, sin = _cos_sin(8192, 128, dtype=torch.bfloat16)
    q0, k0 = q.clone(), k.clone()
    _launch(q, k, q, k, cos, sin, negate=False)
    half = 64
    n0 = q0.float()[..., :half].pow(2) + q0.float()[..., half:].pow(2)
    n1 = q.float()[..., :half].pow(2) + q.float()[..., half:].pow(2)
    # |x|^2 of each rotated pair is preserved up to the bf16 rounding of cos/sin and of the outputs
    assert float(((n1 - n0).abs() - 3e-2 * n0).max()) < 3e-2
    idx = torch.tensor([0, 1, 4095, 8191], device=DEV)
    q_ref, k_ref = oracle.rope(q0[:, :, idx].float().cpu().numpy(), k0[:, :, idx].float().cpu().numpy(),
                               cos[:, idx].float().cpu().numpy(), sin[:, idx].float().cpu().numpy())
    assert_close(q[:, :, idx], q_ref, what="q rows", **BF16_TOL)
    assert_close(k[:, :, idx], k_ref, what="k rows", **BF16_TOL)
    qb, kb = torch.empty_like(q), torch.empty_like(k)
    _launch(q, k, qb, kb, cos, sin, negate=True)
    assert float((qb.float() - q0.float()).abs().max()) < 6e-2
    assert float((kb.float() - k0.float()).abs().max()) < 6e-2


# ----------------------------------------------------------------- SwiGLU (elementwise)
@pytest.mark.parametrize("dtype,tol", [(torch.float32, dict(rtol=1e-4, atol=1e-5)), (torch.bfloat16, BF16_TOL),
                                       (torch.float16, BF16_TOL)])
@pytest.mark.parametrize("shape", [(4, 64, 512), (2, 32, 256), (7, 12288), (5, 100), (3, 33), (0, 64), (1, 8)])
def test_swiglu_fwd_bwd_vs_oracle(shape, dtype, tol):
    from bastile_b200.ops.swiglu import SwiGLUFunction

    torch.manual_seed(sum(shape))
    g = torch.randn(*shape, device=DEV).to(dtype).requires_grad_(True)
    u = torch.randn(*shape, device=DEV).to(dtype).requires_grad_(True)
    dy = torch.randn(*shape, device=DEV).to(dtype)
    out = SwiGLUFunction.apply(g, u)
    out.backward(dy)
    gn, un, dn = (a.detach().float().cpu().numpy() for a in (g, u, dy))
    assert_close(out, oracle.swiglu_fwd(gn, un), what="out", **tol)
    dg_ref, du_ref = oracle.swiglu_bwd(dn, gn, un)
    assert_close(g.grad, dg_ref, what="dgate", **tol)
    assert_close(u.grad, du_ref, what="dup", **tol)


def test_swiglu_reference_unit_tests():
    """tests/ops/test_swiglu.py: fp32, vs F.silu(gate) * up and autograd, 1e-3 / 1e-2."""
    import torch.nn.functional as F

    from bastile_b200.ops.swiglu import SwiGLUFunction

    gate = torch.randn(4, 64, 512, device=DEV)
    up = torch.randn(4, 64, 512, device=DEV)
    torch.testing.assert_close(SwiGLUFunction.apply(gate, up), F.silu(gate) * up, rtol=1e-3, atol=1e-3)
    g = torch.randn(2, 32, 256, device=DEV, requires_grad=True)
    u = torch.randn(2, 32, 256, device=DEV, requires_grad=True)
    SwiGLUFunction.apply(g, u).sum().backward()
    gr, ur = g.detach().clone().requires_grad_(True), u.detach().clone().requires_grad_(True)
    (F.silu(gr) * ur).sum().backward()
    torch.testing.assert_close(g.grad, gr.grad, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(u.grad, ur.grad, rtol=1e-2, atol=1e-2)


def test_swiglu_bf16_forward_bits_match_eager_rounding():
    """silu is rounded to bf16 before the multiply, like the op being replaced."""
    import torch.nn.functional as F

    from bastile_b200.ops.swiglu import swiglu

    torch.manual_seed(3)
    g = torch.randn(64, 1024, device=DEV, dtype=torch.bfloat16)
    u = torch.randn(64, 1024, device=DEV, dtype=torch.bfloat16)
    eager = F.silu(g) * u
    ours = swiglu(g, u)
    ulp_off = (ours.view(torch.int16).int() - eager.view(torch.int16).int()).abs()
    assert float((ulp_off > 1).float().mean()) < 1e-3  # approximate exp may move silu by one ulp, rarely
