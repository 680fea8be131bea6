"""The fusions across op boundaries (`apply(fused_layers=True)`): add + RMSNorm, q/k-norm + RoPE,
residual in the down projection - against the CPU oracle, against the separate kernels (bit for
bit where the rounding points are the same), and on the tiny Qwen3 against the HF eager fixture."""

import numpy as np
import pytest
import torch

import oracle
from conftest import BF16_TOL, FP32_TOL, assert_close, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"

DTYPES = [(torch.float32, FP32_TOL), (torch.bfloat16, BF16_TOL), (torch.float16, BF16_TOL)]


def _np(t):
    return t.detach().float().cpu().numpy()


def _round_like(dtype):
    return lambda a: torch.as_tensor(np.asarray(a, np.float32)).to(dtype).float().numpy()


def _cos_sin(t, d, theta=1e6, dtype=torch.float32, batch=1):
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    emb = torch.outer(torch.arange(t, dtype=torch.float32), inv)
    emb = torch.cat((emb, emb), -1)
    return (emb.cos()[None].expand(batch, -1, -1).contiguous().to(DEV, dtype),
            emb.sin()[None].expand(batch, -1, -1).contiguous().to(DEV, dtype))


# ------------------------------------------------------------------ add + RMSNorm
@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("m,n", [(1, 8), (37, 128), (300, 128), (33, 1024), (130, 2048), (67, 4096), (9, 8192),
                                 (3, 5120), (4, 100), (7, 4099), (2, 16384), (0, 128)])
def test_add_rmsnorm_vs_oracle_and_separate_kernels(m, n, dtype, tol):
    from bastile_b200.ops.fused_layers import add_rms_norm
    from bastile_b200.ops.rms_norm import rms_norm

    torch.manual_seed(m * 1000 + n + 1)
    x = torch.randn(m, n, device=DEV).to(dtype).requires_grad_(True)
    r = torch.randn(m, n, device=DEV).to(dtype).requires_grad_(True)
    w = (1 + 0.02 * torch.randn(n, device=DEV)).to(dtype).requires_grad_(True)
    dy = torch.randn(m, n, device=DEV).to(dtype)
    ds = torch.randn(m, n, device=DEV).to(dtype)
    y, stream = add_rms_norm(x, r, w, 1e-6)
    torch.autograd.backward([y, stream], [dy, ds])
    assert y.dtype == dtype and stream.dtype == dtype

    y_ref, s_ref, rstd = oracle.add_rms_norm_fwd(_np(x), _np(r), _np(w), 1e-6, round_to=_round_like(dtype))
    dx_ref, dw_ref = oracle.add_rms_norm_bwd(_np(dy), _np(ds), s_ref, _np(w), rstd)
    assert_close(stream, s_ref, what="stream", **tol)
    assert_close(y, y_ref, what="y", **tol)
    assert_close(x.grad, dx_ref, what="dx", **tol)
    assert torch.equal(x.grad, r.grad)
    dw_tol = dict(rtol=tol["rtol"], atol=max(tol["atol"], 2e-2 * np.sqrt(max(m, 1)) if dtype != torch.float32 else 1e-4))
    assert_close(w.grad, dw_ref, what="dw", **dw_tol)

    # the same thing from the separate kernels: torch add, then the plain norm
    x2, r2, w2 = (t.detach().clone().requires_grad_(True) for t in (x, r, w))
    s2 = x2 + r2
    y2 = rms_norm(s2, w2, 1e-6)
    torch.autograd.backward([y2, s2], [dy, ds])
    assert torch.equal(stream, s2) and torch.equal(y, y2)
    assert_close(w.grad, _np(w2.grad), what="dw vs separate", **dw_tol)  # atomics: order varies
    # dx: the fused kernel adds the stream gradient before the single rounding, autograd after it
    assert_close(x.grad, _np(x2.grad), what="dx vs separate", **tol)


def test_add_rmsnorm_without_residual_merges_the_stream_gradient():
    from bastile_b200.ops.fused_layers import add_rms_norm

    torch.manual_seed(5)
    x = torch.randn(3, 50, 256, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    w = torch.ones(256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    h = x * 1.0
    y, stream = add_rms_norm(h, None, w, 1e-6)
    assert stream.data_ptr() == h.data_ptr()
    dy, ds = torch.randn_like(y), torch.randn_like(y)
    torch.autograd.backward([y, stream], [dy, ds])
    rstd = oracle.rms_norm_fwd(_np(x), _np(w))[1]
    dx_ref, _ = oracle.add_rms_norm_bwd(_np(dy), _np(ds), _np(x), _np(w), rstd)
    assert_close(x.grad, dx_ref, what="dx", **BF16_TOL)
    # only one of the two outputs used downstream
    for use_y in (True, False):
        x.grad = None
        y, stream = add_rms_norm(x * 1.0, None, w, 1e-6)
        (y if use_y else stream).backward(dy)
        ref = oracle.rms_norm_bwd(_np(dy), _np(x), _np(w), rstd)[0] if use_y else _np(dy)
        assert_close(x.grad, ref, what=f"dx use_y={use_y}", **BF16_TOL)


def test_add_rmsnorm_full_size():
    """8192 x 4096 bf16, the per-layer shape of Qwen3-8B at sequence length 8192."""
    from bastile_b200.ops.fused_layers import add_rms_norm
    from bastile_b200.ops.rms_norm import rms_norm

    torch.manual_seed(1)
    m, n = 8192, 4096
    x = torch.randn(m, n, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(m, n, device=DEV, dtype=torch.bfloat16)
    w = (1 + 0.02 * torch.randn(n, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    dy, ds = torch.randn_like(x), torch.randn_like(x)
    y, stream = add_rms_norm(x, r, w, 1e-6)
    torch.autograd.backward([y, stream], [dy, ds])
    x2, w2 = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    s2 = x2 + r
    y2 = rms_norm(s2, w2, 1e-6)
    torch.autograd.backward([y2, s2], [dy, ds])
    assert torch.equal(stream, s2) and torch.equal(y, y2)
    assert_close(w.grad, _np(w2.grad), what="dw", rtol=2e-2, atol=2e-2 * float(w2.grad.float().abs().max()))
    idx = torch.tensor([0, 1, 4095, 8191], device=DEV)
    assert_close(x.grad[idx], _np(x2.grad[idx]), what="dx rows", **BF16_TOL)


# ------------------------------------------------------------------ q/k-norm + RoPE
@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("b,t,hq,hk,d", [(1, 130, 32, 8, 128), (2, 17, 8, 8, 128), (3, 9, 5, 3, 64), (1, 1, 1, 1, 128),
                                         (2, 33, 3, 1, 32), (1, 700, 6, 2, 256)])
def test_qk_norm_rope_vs_oracle_and_separate_kernels(b, t, hq, hk, d, dtype, tol):
    from bastile_b200.ops.fused_layers import _head_rows_supported, qk_norm_rope
    from bastile_b200.ops.rms_norm import rms_norm
    from bastile_b200.ops.rope import apply_rotary_pos_emb

    if not _head_rows_supported(d, dtype):
        pytest.skip("head rows of this size go through the separate kernels")
    torch.manual_seed(b + t + hq + d)
    # projection outputs [B, T, H*D] viewed per head, as Qwen3Attention builds them
    xq = torch.randn(b, t, hq * d, device=DEV).to(dtype).requires_grad_(True)
    xk = torch.randn(b, t, hk * d, device=DEV).to(dtype).requires_grad_(True)
    wq = (1 + 0.1 * torch.randn(d, device=DEV)).to(dtype).requires_grad_(True)
    wk = (1 + 0.1 * torch.randn(d, device=DEV)).to(dtype).requires_grad_(True)
    cos, sin = _cos_sin(t, d, dtype=dtype, batch=b if b == 2 else 1)
    dqo = torch.randn(b, hq, t, d, device=DEV).to(dtype)  # attention hands back [B,H,T,D]
    dko = torch.randn(b, hk, t, d, device=DEV).to(dtype)
    qo, ko = qk_norm_rope(xq.view(b, t, hq, d), xk.view(b, t, hk, d), wq, wk, cos, sin, 1e-6, 1e-5)
    qo, ko = qo.transpose(1, 2), ko.transpose(1, 2)
    torch.autograd.backward([qo, ko], [dqo, dko])

    rnd = _round_like(dtype)
    for x, w, out, dout, h, eps in ((xq, wq, qo, dqo, hq, 1e-6), (xk, wk, ko, dko, hk, 1e-5)):
        x4 = _np(x).reshape(b, t, h, d)
        o_ref, _ = oracle.head_norm_rope_fwd(x4, _np(w), _np(cos), _np(sin), eps, round_to=rnd)
        dx_ref, dw_ref = oracle.head_norm_rope_bwd(_np(dout).transpose(0, 2, 1, 3), x4, _np(w), _np(cos), _np(sin),
                                                   eps, round_to=rnd)
        assert_close(out.transpose(1, 2), o_ref, what="out", **tol)
        assert_close(x.grad.view(b, t, h, d), dx_ref, what="dx", **tol)
        dw_tol = dict(rtol=tol["rtol"],
                      atol=max(tol["atol"], 2e-2 * np.sqrt(b * t * h) if dtype != torch.float32 else 1e-4))
        assert_close(w.grad, dw_ref, what="dw", **dw_tol)

    # the separate kernels round at the same two places: identical bits
    xq2, xk2, wq2, wk2 = (a.detach().clone().requires_grad_(True) for a in (xq, xk, wq, wk))
    q2 = rms_norm(xq2.view(b, t, hq, d), wq2, 1e-6).transpose(1, 2)
    k2 = rms_norm(xk2.view(b, t, hk, d), wk2, 1e-5).transpose(1, 2)
    qo2, ko2 = apply_rotary_pos_emb(q2, k2, cos, sin)
    torch.autograd.backward([qo2, ko2], [dqo, dko])
    assert torch.equal(qo, qo2) and torch.equal(ko, ko2)
    assert torch.equal(xq.grad, xq2.grad) and torch.equal(xk.grad, xk2.grad)


def test_qk_norm_rope_full_size_matches_separate_kernels():
    """q and k of Qwen3-8B at sequence length 8192: 32 and 8 heads of 128."""
    from bastile_b200.ops.fused_layers import qk_norm_rope
    from bastile_b200.ops.rms_norm import rms_norm
    from bastile_b200.ops.rope import apply_rotary_pos_emb

    torch.manual_seed(2)
    b, t, hq, hk, d = 1, 8192, 32, 8, 128
    bf = torch.bfloat16
    xq = torch.randn(b, t, hq * d, device=DEV, dtype=bf, requires_grad=True)
    xk = torch.randn(b, t, hk * d, device=DEV, dtype=bf, requires_grad=True)
    wq = (1 + 0.1 * torch.randn(d, device=DEV)).to(bf).requires_grad_(True)
    wk = (1 + 0.1 * torch.randn(d, device=DEV)).to(bf).requires_grad_(True)
    cos, sin = _cos_sin(t, d, dtype=bf)
    dqo = torch.randn(b, hq, t, d, device=DEV, dtype=bf)
    dko = torch.randn(b, hk, t, d, device=DEV, dtype=bf)
    qo, ko = qk_norm_rope(xq.view(b, t, hq, d), xk.view(b, t, hk, d), wq, wk, cos, sin)
    qo, ko = qo.transpose(1, 2), ko.transpose(1, 2)
    torch.autograd.backward([qo, ko], [dqo, dko])
    xq2, xk2, wq2, wk2 = (a.detach().clone().requires_grad_(True) for a in (xq, xk, wq, wk))
    q2 = rms_norm(xq2.view(b, t, hq, d), wq2, 1e-6).transpose(1, 2)
    k2 = rms_norm(xk2.view(b, t, hk, d), wk2, 1e-6).transpose(1, 2)
    qo2, ko2 = apply_rotary_pos_emb(q2, k2, cos, sin)
    torch.autograd.backward([qo2, ko2], [dqo, dko])
    assert torch.equal(qo, qo2) and torch.equal(ko, ko2)
    assert torch.equal(xq.grad, xq2.grad) and torch.equal(xk.grad, xk2.grad)
    for w, w2 in ((wq, wq2), (wk, wk2)):
        assert_close(w.grad, _np(w2.grad), what="dw", rtol=2e-2, atol=2e-2 * float(w2.grad.float().abs().max()))


def test_qk_norm_rope_rejects_unsupported_head_rows():
    from bastile_b200 import _lib

    lib = _lib.get_lib()
    x = torch.randn(1, 4, 2, 24, device=DEV, dtype=torch.bfloat16)
    out, rstd = torch.empty_like(x), torch.empty(8, device=DEV)
    w = torch.ones(24, device=DEV, dtype=torch.bfloat16)
    cos, sin = _cos_sin(4, 24, dtype=torch.bfloat16)
    s3 = _lib.I64x3(*x.stride()[:3])
    rc = lib.bt_qk_norm_rope_fwd(x.data_ptr(), x.data_ptr(), w.data_ptr(), w.data_ptr(), cos.data_ptr(),
                                 sin.data_ptr(), out.data_ptr(), out.data_ptr(), rstd.data_ptr(), rstd.data_ptr(), 1, 4,
                                 2, 2, 24, s3, s3, s3, s3, _lib.I64x2(cos.stride(0), cos.stride(1)), 1, 1e-6, 1e-6, 0,
                                 _lib.stream_ptr(x.device))
    assert rc == -1 and b"not supported" in lib.bt_last_error()


# ------------------------------------------------------------------ residual in the down projection
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_mlp_with_residual_vs_oracle(dtype):
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction

    torch.manual_seed(3)
    t, hidden, inter = 200, 256, 640
    x = torch.randn(t, hidden, device=DEV).to(dtype).requires_grad_(True)
    r = torch.randn(t, hidden, device=DEV).to(dtype).requires_grad_(True)
    wg, wu = (torch.randn(inter, hidden, device=DEV).mul(0.05).to(dtype).requires_grad_(True) for _ in range(2))
    wd = torch.randn(hidden, inter, device=DEV).mul(0.05).to(dtype).requires_grad_(True)
    dy = torch.randn(t, hidden, device=DEV).to(dtype)
    y = SwiGLUMLPFunction.apply(x, wg, wu, wd, r)
    y.backward(dy)
    y_ref = oracle.mlp_fwd(_np(x), _np(wg), _np(wu), _np(wd))[0] + _np(r)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype != torch.float32 else dict(rtol=5e-3, atol=5e-3)
    assert_close(y, y_ref, what="y", **tol)
    assert torch.equal(r.grad, dy)
    x2, wg2, wu2, wd2 = (a.detach().clone().requires_grad_(True) for a in (x, wg, wu, wd))
    SwiGLUMLPFunction.apply(x2, wg2, wu2, wd2).backward(dy)
    assert torch.equal(x.grad, x2.grad) and torch.equal(wd.grad, wd2.grad) and torch.equal(wg.grad, wg2.grad)


# ------------------------------------------------------------------ projections sharing their input
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("dx_only", [False, True])
@pytest.mark.parametrize("widths", [(512, 128, 128), (256,), (384, 128), (128, 128, 128, 256)])
def test_shared_input_linear_vs_float64(widths, dtype, dx_only):
    """y_i = x W_i^T, dx = sum_i dy_i W_i (accumulated inside the GEMMs), dW_i = dy_i^T x."""
    from bastile_b200 import _lib
    from bastile_b200.ops.fused_layers import shared_input_linear

    torch.manual_seed(len(widths) * 7 + widths[0])
    rows, hidden = 333, 256
    x = torch.randn(3, rows // 3, hidden, device=DEV).to(dtype).requires_grad_(True)
    ws = [torch.randn(n, hidden, device=DEV).mul(0.05).to(dtype).requires_grad_(True) for n in widths]
    dys = [torch.randn(3, rows // 3, n, device=DEV).to(dtype) for n in widths]
    ys = shared_input_linear(x, *ws, dx_only=dx_only)
    torch.autograd.backward(list(ys), dys)
    _lib.check_status(x.device, "shared_input_linear")
    x64 = x.detach().double().cpu().reshape(-1, hidden)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype != torch.float32 else dict(rtol=5e-3, atol=5e-3)
    dx_ref = torch.zeros_like(x64)
    for y, w, dy in zip(ys, ws, dys):
        w64, dy64 = w.detach().double().cpu(), dy.double().cpu().reshape(-1, w.shape[0])
        assert y.dtype == dtype and y.shape == (3, rows // 3, w.shape[0])
        assert_close(y.reshape(-1, w.shape[0]), (x64 @ w64.T).numpy(), what="y", **tol)
        dw_ref = (dy64.T @ x64).numpy()
        assert_close(w.grad, dw_ref, what="dW", rtol=tol["rtol"], atol=tol["atol"] * float(np.abs(dw_ref).max()))
        dx_ref += dy64 @ w64
    assert_close(x.grad.reshape(-1, hidden), dx_ref.numpy(), what="dx", rtol=tol["rtol"],
                 atol=tol["atol"] * float(dx_ref.abs().max()))


def test_shared_input_linear_partial_gradients():
    """An output that is not used downstream contributes nothing; weights can be frozen."""
    from bastile_b200.ops.fused_layers import shared_input_linear

    torch.manual_seed(11)
    x = torch.randn(64, 128, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w0 = torch.randn(256, 128, device=DEV, dtype=torch.bfloat16).mul(0.05).requires_grad_(True)
    w1 = torch.randn(128, 128, device=DEV, dtype=torch.bfloat16).mul(0.05)  # frozen
    y0, y1 = shared_input_linear(x, w0, w1)
    dy1 = torch.randn_like(y1)
    y1.backward(dy1)
    assert w0.grad is None
    ref = dy1.double() @ w1.double()
    assert_close(x.grad, ref.cpu().numpy(), what="dx", rtol=2e-2, atol=2e-2 * float(ref.abs().max()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("pairs", [1, 0])
@pytest.mark.parametrize("rows,hidden,nq,nk", [(333, 256, 512, 256), (1024, 512, 1024, 256), (40, 128, 256, 256)])
def test_qkv_projection_one_product_each_way_vs_float64(rows, hidden, nq, nk, dtype, pairs):
    """q/k/v projections over weights stacked in memory: forward with the result split over three
    dense tensors, dx with the A operand read from three gradient tensors along the contraction,
    the three weight gradients as one product with A in three pieces along M - against float64."""
    from bastile_b200 import _lib
    from bastile_b200.ops.fused_layers import QKVProjectionFunction, _qkv_fusable

    lib = _lib.get_lib()
    prev = lib.bt_set_gemm_cta_pairs(pairs)
    try:
        torch.manual_seed(rows + nq)
        x = torch.randn(rows, hidden, device=DEV).to(dtype).requires_grad_(True)
        buf = torch.randn(nq + 2 * nk, hidden, device=DEV).mul(0.05).to(dtype)
        ws = [buf[:nq].requires_grad_(True), buf[nq:nq + nk].requires_grad_(True), buf[nq + nk:].requires_grad_(True)]
        assert _qkv_fusable(x, *ws)
        dys = [torch.randn(rows, n, device=DEV).to(dtype) for n in (nq, nk, nk)]
        ys = QKVProjectionFunction.apply(x, *ws)
        assert all(y.is_contiguous() for y in ys)
        torch.autograd.backward(list(ys), dys)
        _lib.check_status(x.device, "qkv projection")
        x64 = x.detach().double().cpu()
        tol = dict(rtol=2e-2, atol=2e-2) if dtype != torch.float32 else dict(rtol=5e-3, atol=5e-3)
        dx_ref = torch.zeros_like(x64)
        for y, w, dy in zip(ys, ws, dys):
            w64, dy64 = w.detach().double().cpu(), dy.double().cpu()
            assert_close(y, (x64 @ w64.T).numpy(), what="y", **tol)
            dw_ref = (dy64.T @ x64).numpy()
            assert_close(w.grad, dw_ref, what="dW", rtol=tol["rtol"], atol=tol["atol"] * float(np.abs(dw_ref).max()))
            dx_ref += dy64 @ w64
        assert_close(x.grad, dx_ref.numpy(), what="dx", rtol=tol["rtol"], atol=tol["atol"] * float(dx_ref.abs().max()))
    finally:
        lib.bt_set_gemm_cta_pairs(prev)


def test_qkv_mode_whole_model_matches_separate_projections():
    """A small Qwen3 whose q/k/v widths the fused product takes (512 | 256 | 256): after
    stack_qkv_weights() the "qkv" mode must give the loss and gradients of the same model with
    nn.Linear projections, parameter names and shapes unchanged; a layer whose weights are not
    stacked falls back by itself."""
    from transformers import Qwen3Config, Qwen3ForCausalLM

    import bastile_b200
    from bastile_b200 import _lib
    from bastile_b200.ops import fused_layers

    cfg = Qwen3Config(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=8, num_key_value_heads=4, head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6,
                      tie_word_embeddings=False, use_cache=False)
    cfg._attn_implementation = "sdpa"
    ids = torch.randint(0, 1024, (2, 96), generator=torch.Generator().manual_seed(3)).to(DEV)
    results = {}
    try:
        for mode in ("off", "qkv"):
            bastile_b200.reset()
            bastile_b200.apply(fused_layers=True, gemm_projections=mode)
            torch.manual_seed(21)
            model = Qwen3ForCausalLM(cfg).to(DEV, torch.bfloat16).train()
            names = [n for n, _ in model.named_parameters()]
            if mode == "qkv":
                assert fused_layers.stack_qkv_weights(model) == 2
                att = model.model.layers[0].self_attn
                assert fused_layers._stacked(att.q_proj.weight, att.k_proj.weight, att.v_proj.weight)
                assert [n for n, _ in model.named_parameters()] == names
                # un-stack the second layer: it must take the separate projections again
                att1 = model.model.layers[1].self_attn
                att1.k_proj.weight.data = att1.k_proj.weight.data.clone()
                assert not fused_layers._stacked(att1.q_proj.weight, att1.k_proj.weight, att1.v_proj.weight)
            _lib.instr.reset(enabled=False)
            out = model(input_ids=ids, labels=ids)
            out.loss.backward()
            _lib.check_status(torch.device(DEV, torch.cuda.current_device()), mode)
            results[mode] = (float(out.loss.detach()), {n: p.grad.detach().float().clone() for n, p in model.named_parameters()})
    finally:
        bastile_b200.reset()
    (l0, g0), (l1, g1) = results["off"], results["qkv"]
    assert abs(l0 - l1) <= 1e-3 * abs(l0)
    for n in g0:
        scale = float(g0[n].abs().max()) + 1e-12
        assert float((g0[n] - g1[n]).abs().max()) <= 3e-2 * scale, n



def test_acc_mode_matches_separate_projections_and_fills_gradient_destinations():
    """gemm_projections="acc": the library GEMMs of nn.Linear with dx accumulated by the GEMMs.
    The forward is the same product; gradients agree with autograd's separate products + adds to
    bf16 rounding of the running sum; with a registered destination dW lands in it uncopied."""
    from bastile_b200 import _lib
    from bastile_b200.ops.fused_layers import AccumulatedInputGradFunction

    torch.manual_seed(5)
    x = torch.randn(2, 67, 256, device=DEV).to(torch.bfloat16).requires_grad_(True)
    ws = [(0.05 * torch.randn(n, 256, device=DEV)).to(torch.bfloat16).requires_grad_(True) for n in (512, 128, 128)]
    dys = [torch.randn(2, 67, n, device=DEV).to(torch.bfloat16) for n in (512, 128, 128)]
    ref = [torch.nn.functional.linear(x, w) for w in ws]
    torch.autograd.backward(ref, dys)
    want = [x.grad.clone()] + [w.grad.clone() for w in ws]
    x.grad = None
    for w in ws:
        w.grad = None
    dest = torch.zeros_like(ws[1])
    _lib.register_grad_sink(ws[1].data, dest)
    try:
        outs = AccumulatedInputGradFunction.apply(x, *ws)
        for o, r in zip(outs, ref):
            assert torch.equal(o, r)
        # v arrives as the transposed view attention hands back: not contiguous
        dys[2] = dys[2].view(2, 67, 2, 64).transpose(1, 2).contiguous().transpose(1, 2).reshape(2, 67, 128)
        torch.autograd.backward(outs, dys)
    finally:
        _lib.unregister_grad_sinks([dest])
    assert_close(x.grad, want[0].float().cpu().numpy(), what="dx", rtol=2e-2, atol=2e-2 * float(want[0].abs().max()))
    for w, g in zip(ws, want[1:]):
        assert_close(w.grad, g.float().cpu().numpy(), what="dw", rtol=1e-2, atol=1e-2 * float(g.abs().max()))
    assert ws[1].grad.data_ptr() == dest.data_ptr()
    # a gradient that never arrives (k unused) is skipped, not materialised
    x.grad = None
    q, k, v = AccumulatedInputGradFunction.apply(x, *ws)
    (q.float().sum() + v.float().sum()).backward()
    assert x.grad is not None and torch.isfinite(x.grad.float()).all()


# ------------------------------------------------------------------ whole model
@pytest.fixture(params=["off", "acc", "dx", "all", "qkv"])
def fused(request):
    """apply(fused_layers=True) in each mode of the q/k/v/o projections."""
    import bastile_b200

    bastile_b200.reset()
    applied = bastile_b200.apply(fused_layers=True, gemm_projections=request.param)
    yield applied
    bastile_b200.reset()


def _tiny_model(dtype):
    from golden.make_golden import build_tiny_qwen3, tiny_qwen3_config
    from transformers import Qwen3ForCausalLM

    import bastile_b200

    from bastile_b200.ops import fused_layers

    applied, mode = bastile_b200.get_patched_ops(), fused_layers._projection_mode
    bastile_b200.reset()
    stock = build_tiny_qwen3()  # CPU fp32, seed 0: the weights of the fixture
    bastile_b200.apply(fused_layers=True, gemm_projections=mode)
    assert bastile_b200.get_patched_ops() == applied
    model = Qwen3ForCausalLM(tiny_qwen3_config())
    model.load_state_dict(stock.state_dict())
    return model.to(DEV, dtype).train()


def test_apply_fused_layers_installs_and_reset_restores(fused):
    import transformers.models.qwen3.modeling_qwen3 as q3

    import bastile_b200
    from bastile_b200.ops import fused_layers

    assert fused == ["rms_norm_qwen3", "rope_qwen3", "swiglu_qwen3", "decoder_layer_qwen3", "attention_qwen3",
                     "fused_linear_cross_entropy"]
    assert q3.Qwen3DecoderLayer.forward is fused_layers.decoder_layer_forward
    assert q3.Qwen3Attention.forward is fused_layers.attention_forward
    bastile_b200.reset()
    assert q3.Qwen3DecoderLayer.forward is not fused_layers.decoder_layer_forward
    assert q3.Qwen3Attention.forward is not fused_layers.attention_forward
    assert fused_layers.installed() == []


def test_tiny_qwen3_fused_layers_match_hf_eager_fixture(fused):
    from golden.make_golden import tiny_qwen3_inputs

    from bastile_b200 import _lib

    g = load_golden("tiny_qwen3.npz")
    model = _tiny_model(torch.bfloat16)
    ids, labels = tiny_qwen3_inputs()
    out = model(input_ids=ids.to(DEV), labels=labels.to(DEV))
    out.loss.backward()
    _lib.check_status(torch.device(DEV, torch.cuda.current_device()), "tiny model, fused layers")
    loss_ref = float(g["loss"])
    assert abs(out.loss.item() - loss_ref) <= 5e-3 * loss_ref
    grads = dict(model.named_parameters())
    for name, ref_norm in zip([str(n) for n in g["names"]], g["grad_norms"]):
        gn = grads[name].grad.float().norm().item()
        assert np.isfinite(gn)
        assert abs(gn - ref_norm) <= 0.08 * ref_norm + 1e-4, f"{name}: grad norm {gn} vs {ref_norm}"
    for key in g.files:
        if not key.startswith("grad::"):
            continue
        pname = key[len("grad::"):]
        if pname.endswith("[:64,:64]"):
            got = grads[pname[:-len("[:64,:64]")]].grad[:64, :64]
        else:
            got = grads[pname].grad
        ref = g[key]
        assert_close(got, ref, what=pname, rtol=5e-2, atol=5e-2 * float(np.abs(ref).max()))


def test_tiny_qwen3_fused_layers_fp32_match_hf_eager_fixture(fused):
    from golden.make_golden import tiny_qwen3_inputs

    g = load_golden("tiny_qwen3.npz")
    model = _tiny_model(torch.float32)
    ids, labels = tiny_qwen3_inputs()
    out = model(input_ids=ids.to(DEV), labels=labels.to(DEV))
    out.loss.backward()
    assert abs(out.loss.item() - float(g["loss"])) <= 1e-3 * float(g["loss"])
    grads = dict(model.named_parameters())
    for name, ref_norm in zip([str(n) for n in g["names"]], g["grad_norms"]):
        gn = grads[name].grad.float().norm().item()
        assert abs(gn - ref_norm) <= 2e-2 * ref_norm + 1e-5, f"{name}: grad norm {gn} vs {ref_norm}"


def test_fused_layers_eval_forward_and_kv_cache_match_unfused():
    """Inference path (no labels, generation with a cache) through the fused forwards gives the
    logits of the unfused patched model."""
    from golden.make_golden import build_tiny_qwen3, tiny_qwen3_config, tiny_qwen3_inputs
    from transformers import Qwen3ForCausalLM

    import bastile_b200

    bastile_b200.reset()
    stock = build_tiny_qwen3()
    ids, _ = tiny_qwen3_inputs()
    logits = []
    try:
        for fused_on in (False, True):
            bastile_b200.reset()
            bastile_b200.apply(fused_layers=fused_on)
            model = Qwen3ForCausalLM(tiny_qwen3_config())
            model.load_state_dict(stock.state_dict())
            model = model.to(DEV, torch.bfloat16).eval()
            with torch.no_grad():
                full = model(input_ids=ids.to(DEV)).logits
                first = model(input_ids=ids[:, :100].to(DEV), use_cache=True)
                rest = model(input_ids=ids[:, 100:].to(DEV), past_key_values=first.past_key_values, use_cache=True)
            logits.append((full, torch.cat((first.logits, rest.logits), dim=1)))
    finally:
        bastile_b200.reset()
    (full_u, cached_u), (full_f, cached_f) = logits
    scale = float(full_u.float().abs().max())
    assert_close(full_f, _np(full_u), what="logits", rtol=2e-2, atol=2e-2 * scale)
    assert_close(cached_f, _np(full_f), what="cached vs full", rtol=3e-2, atol=3e-2 * scale)
    assert_close(cached_f, _np(cached_u), what="cached", rtol=2e-2, atol=2e-2 * scale)
