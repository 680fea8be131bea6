"""Whole-tensor parity at the benchmark shapes.

The numpy oracle cannot evaluate 8192 x 4096 x 12288 or 16384 x 4096 x 151936 in reasonable time, so
the full-size results are compared, element by element and complete, with an fp32 evaluation of the
same formulas in torch on the GPU (TF32 off).  Each such evaluation is first pinned to the oracle at a
small shape inside the same test, so the chain is: reference lines -> oracle -> torch fp32 -> kernels.
Tolerance: the 16-bit bar, rtol 2e-2 and atol 2e-2 of the tensor's largest magnitude."""

import numpy as np
import pytest
import torch

import oracle
from conftest import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


@pytest.fixture(autouse=True)
def _exact_fp32_matmul():
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = prev
    torch.cuda.empty_cache()


def gpu_close(actual, expected, what, rtol=2e-2, atol_rel=2e-2):
    """|a - e| <= atol_rel * max|e| + rtol * |e| for every element, evaluated on the device."""
    a, e = actual.detach().float(), expected.detach().float()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(e.shape)}"
    assert bool(torch.isfinite(a).all()), f"{what}: non-finite values"
    bound = atol_rel * float(e.abs().max()) + rtol * e.abs()
    bad = (a - e).abs() > bound
    n_bad = int(bad.sum())
    if n_bad:
        idx = torch.nonzero(bad)[0].tolist()
        raise AssertionError(f"{what}: {n_bad}/{bad.numel()} elements off; first at {idx}: got "
                             f"{float(a[tuple(idx)])!r}, want {float(e[tuple(idx)])!r}")


def npf(t):
    return t.detach().float().cpu().numpy()


# ------------------------------------------------------------------ fp32 evaluations in torch
def ref_rms(x, w, dy, eps=1e-6):
    x32 = x.float().requires_grad_(True)
    w32 = w.float().requires_grad_(True)
    y = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps) * w32
    y.backward(dy.float())
    return y.detach(), x32.grad, w32.grad


def ref_head_norm_rope(x, w, cos, sin, dout, eps=1e-6):
    """x [B,T,H,D]: per-head RMSNorm with w, then rotate-half RoPE with cos/sin [1,T,D]."""
    x32 = x.float().requires_grad_(True)
    w32 = w.float().requires_grad_(True)
    n = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps) * w32
    c, s = cos.float()[:, :, None, :], sin.float()[:, :, None, :]
    d = x.shape[-1]
    rot = torch.cat((-n[..., d // 2:], n[..., : d // 2]), dim=-1)
    out = n * c + rot * s
    out.backward(dout.float())
    return out.detach(), x32.grad, w32.grad


def ref_mlp(x, wg, wu, wd, dy):
    t = [a.float().requires_grad_(True) for a in (x, wg, wu, wd)]
    y = (torch.nn.functional.silu(t[0] @ t[1].T) * (t[0] @ t[2].T)) @ t[3].T
    y.backward(dy.float())
    return (y.detach(), *[a.grad for a in t])


def ref_lce(x, w, labels, ignore_index=-100, chunk=2048):
    """mean cross-entropy of x @ w.T and its gradients, fp32, `chunk` rows of logits at a time."""
    x32, w32 = x.float(), w.float()
    valid = labels != ignore_index
    n_valid = int(valid.sum())
    scale = 1.0 / max(n_valid, 1)
    dx = torch.empty_like(x32)
    dw = torch.zeros_like(w32)
    loss = torch.zeros((), dtype=torch.float64, device=x.device)
    for s in range(0, x.shape[0], chunk):
        xs, ls, vs = x32[s:s + chunk], labels[s:s + chunk], valid[s:s + chunk]
        logits = xs @ w32.T
        lse = torch.logsumexp(logits, dim=-1)
        tgt = logits.gather(1, ls.clamp(min=0)[:, None])[:, 0]
        loss += torch.where(vs, lse - tgt, torch.zeros_like(lse)).double().sum()
        p = torch.exp(logits - lse[:, None])
        del logits
        rows = torch.nonzero(vs)[:, 0]
        p[rows, ls[rows]] -= 1.0
        p[~vs] = 0.0
        p *= scale
        dx[s:s + chunk] = p @ w32
        dw += p.T @ xs
        del p
    return float(loss) * scale, dx, dw


def _rope_tables(t, d, dev):
    inv = 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    emb = torch.outer(torch.arange(t, dtype=torch.float32), inv)
    emb = torch.cat((emb, emb), -1)
    return emb.cos()[None].to(dev, BF), emb.sin()[None].to(dev, BF)


# ------------------------------------------------------------------ RMSNorm
@pytest.mark.parametrize("m,n", [(8192, 4096), (262144, 128)])
def test_rmsnorm_full_size_complete(m, n):
    from bastile_b200.ops.rms_norm import rms_norm

    torch.manual_seed(1)
    # pin the torch evaluation to the oracle
    xs, ws, ds = torch.randn(48, n, device=DEV), 1 + 0.02 * torch.randn(n, device=DEV), torch.randn(48, n, device=DEV)
    y_t, dx_t, dw_t = ref_rms(xs, ws, ds)
    y_o, rstd = oracle.rms_norm_fwd(npf(xs), npf(ws), 1e-6)
    dx_o, dw_o = oracle.rms_norm_bwd(npf(ds), npf(xs), npf(ws), rstd)
    assert_close(y_t, y_o, what="torch fp32 y vs oracle", rtol=1e-4, atol=1e-5)
    assert_close(dx_t, dx_o, what="torch fp32 dx vs oracle", rtol=1e-4, atol=1e-4)
    assert_close(dw_t, dw_o, what="torch fp32 dw vs oracle", rtol=1e-4, atol=1e-4)

    x = torch.randn(m, n, device=DEV, dtype=BF).requires_grad_(True)
    w = (1 + 0.02 * torch.randn(n, device=DEV)).to(BF).requires_grad_(True)
    dy = torch.randn(m, n, device=DEV, dtype=BF)
    y = rms_norm(x, w, 1e-6)
    y.backward(dy)
    y_r, dx_r, dw_r = ref_rms(x.detach(), w.detach(), dy)
    gpu_close(y, y_r, "y")
    gpu_close(x.grad, dx_r, "dx")
    gpu_close(w.grad, dw_r, "dw")


# ------------------------------------------------------------------ q/k-norm + RoPE
def test_qk_norm_rope_full_size_complete():
    from bastile_b200.ops.fused_layers import qk_norm_rope

    torch.manual_seed(1)
    d = 128
    # pin: [1, 16, 4, 128] against the oracle's head_norm_rope
    cos_s, sin_s = _rope_tables(16, d, DEV)
    xs = torch.randn(1, 16, 4, d, device=DEV)
    ws = 1 + 0.1 * torch.randn(d, device=DEV)
    ds = torch.randn(1, 16, 4, d, device=DEV)
    o_t, dx_t, dw_t = ref_head_norm_rope(xs, ws, cos_s, sin_s, ds)
    o_o = oracle.head_norm_rope_fwd(npf(xs), npf(ws), npf(cos_s), npf(sin_s), 1e-6)
    o_o = o_o[0] if isinstance(o_o, tuple) else o_o
    dx_o, dw_o = oracle.head_norm_rope_bwd(npf(ds), npf(xs), npf(ws), npf(cos_s), npf(sin_s), 1e-6)[:2]
    assert_close(o_t, o_o, what="torch fp32 out vs oracle", rtol=1e-4, atol=1e-4)
    assert_close(dx_t, dx_o, what="torch fp32 dx vs oracle", rtol=1e-4, atol=1e-4)
    assert_close(dw_t, dw_o, what="torch fp32 dw vs oracle", rtol=1e-4, atol=1e-3)

    t = 8192
    cos, sin = _rope_tables(t, d, DEV)
    q = torch.randn(1, t, 32, d, device=DEV, dtype=BF).requires_grad_(True)
    k = torch.randn(1, t, 8, d, device=DEV, dtype=BF).requires_grad_(True)
    wq = (1 + 0.1 * torch.randn(d, device=DEV)).to(BF).requires_grad_(True)
    wk = (1 + 0.1 * torch.randn(d, device=DEV)).to(BF).requires_grad_(True)
    dq, dk = torch.randn_like(q), torch.randn_like(k)
    qo, ko = qk_norm_rope(q, k, wq, wk, cos, sin)
    torch.autograd.backward([qo, ko], [dq, dk])
    for name, x, w, dout, out in (("q", q, wq, dq, qo), ("k", k, wk, dk, ko)):
        o_r, dx_r, dw_r = ref_head_norm_rope(x.detach(), w.detach(), cos, sin, dout)
        gpu_close(out, o_r, f"{name} out")
        gpu_close(x.grad, dx_r, f"d{name}")
        gpu_close(w.grad, dw_r, f"dw{name}")


# ------------------------------------------------------------------ SwiGLU MLP block
def test_mlp_full_size_complete():
    """y, dx, dWg, dWu, dWd of the 8192 x 4096 x 12288 block, every element."""
    from bastile_b200 import _lib
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction

    torch.manual_seed(1)
    # pin at a small shape
    xs, wgs, wus = torch.randn(40, 64, device=DEV), torch.randn(96, 64, device=DEV) * 0.1, torch.randn(96, 64, device=DEV) * 0.1
    wds, ds = torch.randn(64, 96, device=DEV) * 0.1, torch.randn(40, 64, device=DEV)
    y_t, dx_t, dwg_t, dwu_t, dwd_t = ref_mlp(xs, wgs, wus, wds, ds)
    y_o = oracle.mlp_fwd(npf(xs), npf(wgs), npf(wus), npf(wds))[0]
    dx_o, dwg_o, dwu_o, dwd_o = oracle.mlp_bwd(npf(ds), npf(xs), npf(wgs), npf(wus), npf(wds))
    for a, b, what in ((y_t, y_o, "y"), (dx_t, dx_o, "dx"), (dwg_t, dwg_o, "dwg"), (dwu_t, dwu_o, "dwu"),
                       (dwd_t, dwd_o, "dwd")):
        assert_close(a, b, what=f"torch fp32 {what} vs oracle", rtol=1e-4, atol=1e-4)

    x = torch.randn(8192, 4096, device=DEV, dtype=BF).requires_grad_(True)
    wg = (torch.randn(12288, 4096, device=DEV) * 0.02).to(BF).requires_grad_(True)
    wu = (torch.randn(12288, 4096, device=DEV) * 0.02).to(BF).requires_grad_(True)
    wd = (torch.randn(4096, 12288, device=DEV) * 0.02).to(BF).requires_grad_(True)
    dy = torch.randn(8192, 4096, device=DEV, dtype=BF)
    y = SwiGLUMLPFunction.apply(x, wg, wu, wd)
    y.backward(dy)
    _lib.check_status(x.device, "full-size MLP")
    y_r, dx_r, dwg_r, dwu_r, dwd_r = ref_mlp(x.detach(), wg.detach(), wu.detach(), wd.detach(), dy)
    gpu_close(y, y_r, "y")
    gpu_close(x.grad, dx_r, "dx")
    gpu_close(wg.grad, dwg_r, "dWg")
    gpu_close(wu.grad, dwu_r, "dWu")
    gpu_close(wd.grad, dwd_r, "dWd")


# ------------------------------------------------------------------ fused linear + cross-entropy
def test_lce_full_size_complete():
    """loss, d hidden and d weight of 16384 x 4096 x 151936 (151936 = 593 * 256 + 128: the last
    column tile is ragged), every element, 5 % of the labels ignored."""
    from bastile_b200 import _lib
    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy

    torch.manual_seed(1)
    # pin at a small shape (two row chunks, ignored rows)
    xs, ws = torch.randn(70, 48, device=DEV), torch.randn(200, 48, device=DEV) * 0.3
    ts = torch.randint(0, 200, (70,), device=DEV)
    ts[::9] = -100
    l_t, dx_t, dw_t = ref_lce(xs, ws, ts, chunk=32)
    l_o, dx_o, dw_o = oracle.lce_fwd_bwd(npf(xs), npf(ws), ts.cpu().numpy(), -100, "mean")
    assert abs(l_t - float(l_o)) <= 1e-5 * abs(float(l_o))
    assert_close(dx_t, dx_o, what="torch fp32 dx vs oracle", rtol=1e-4, atol=1e-6)
    assert_close(dw_t, dw_o, what="torch fp32 dw vs oracle", rtol=1e-4, atol=1e-6)

    rows, hdim, vocab = 16384, 4096, 151936
    x = torch.randn(rows, hdim, device=DEV, dtype=BF).requires_grad_(True)
    w = (torch.randn(vocab, hdim, device=DEV) * 0.02).to(BF).requires_grad_(True)
    t = torch.randint(0, vocab, (rows,), device=DEV)
    t[torch.rand(rows, device=DEV) < 0.05] = -100
    t[:4] = torch.tensor([0, 255, vocab - 1, vocab - 128], device=DEV)  # first tile, last (ragged) tile
    loss = fused_linear_cross_entropy(x, w, t)
    loss.backward()
    _lib.check_all_status()
    l_r, dx_r, dw_r = ref_lce(x.detach(), w.detach(), t)
    assert abs(float(loss) - l_r) <= 1e-3 * abs(l_r), (float(loss), l_r)
    gpu_close(x.grad, dx_r, "d hidden")
    ignored = t == -100
    assert float(x.grad[ignored].float().abs().max()) == 0.0
    gpu_close(w.grad, dw_r, "d weight")
    # the rows that carry a -1 term (labels of a few tokens) and the ragged tail, at a tighter absolute bar
    sel = torch.cat((t[:64][t[:64] >= 0], torch.arange(vocab - 128, vocab, device=DEV), torch.arange(0, 256, device=DEV)))
    gpu_close(w.grad[sel], dw_r[sel], "d weight (label rows, first tile, ragged tail)")
