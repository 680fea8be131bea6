"""Fused linear + cross-entropy through the C ABI: golden fixtures from the reference's own
implementation, the reference's unit tests, ragged/edge cases, and the full-size properties."""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle
from conftest import LOSS_REL, assert_close, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=[(1, 0), (1, 1), (0, 0)], ids=["cta_pairs", "cta_pairs_dynamic_tiles", "single_cta"])
def gemm_mode(request):
    from bastile_b200 import _lib

    lib = _lib.get_lib()
    pairs, dynamic = request.param
    prev = lib.bt_set_gemm_cta_pairs(pairs), lib.bt_set_gemm_dynamic_tiles(dynamic)
    yield request.param
    lib.bt_set_gemm_cta_pairs(prev[0])
    lib.bt_set_gemm_dynamic_tiles(prev[1])


def _run(x, w, t, **kw):
    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy

    xs = x.clone().requires_grad_(True)
    ws = w.clone().requires_grad_(True)
    loss = fused_linear_cross_entropy(xs, ws, t, **kw)
    loss.backward()
    from bastile_b200 import _lib

    _lib.check_status(x.device, "fused_linear_cross_entropy")
    return loss, xs.grad, ws.grad


@pytest.mark.parametrize("name", ["loss_fp32", "grads", "ignore_index", "three_d", "sum", "all_ignored", "ragged"])
@pytest.mark.parametrize("chunk", [4096, 16])
def test_lce_golden_reference_fixtures(name, chunk):
    """Inputs rounded to bf16; expected values recomputed by the oracle on the rounded inputs
    (the oracle itself is pinned to the reference's fp32 outputs on the unrounded ones)."""
    g = load_golden(f"lce_{name}.npz")
    x = torch.as_tensor(g["x"]).to(DEV, torch.bfloat16)
    w = torch.as_tensor(g["w"]).to(DEV, torch.bfloat16)
    t = torch.as_tensor(g["t"]).to(DEV)
    red = str(g["reduction"])
    if bool(g["three_d"]):
        xin, tin = x.view(2, -1, x.shape[-1]), t.view(2, -1)
    else:
        xin, tin = x, t
    loss, dx, dw = _run(xin, w, tin, reduction=red, chunk_size=chunk)
    l_ref, dx_ref, dw_ref = oracle.lce_fwd_bwd(x.float().cpu().numpy(), w.float().cpu().numpy(), g["t"], -100, red)
    # logits are rounded to bf16 before the softmax (as in the reference), so the loss carries
    # that rounding: |logit| * 2^-9 per term, averaged
    assert abs(loss.item() - float(l_ref)) <= 5e-2 * max(1.0, abs(float(l_ref))) if red == "mean" else True
    assert loss.dtype == torch.float32
    assert_close(dx.reshape(dx_ref.shape), dx_ref, what="dx", rtol=2e-2, atol=2e-2 * max(1.0, float(np.abs(dx_ref).max())))
    assert_close(dw, dw_ref, what="dw", rtol=2e-2, atol=2e-2 * max(1.0, float(np.abs(dw_ref).max())))


def test_lce_reference_unit_tests_bf16():
    """tests/ops/test_fused_linear_cross_entropy.py:37-55 (bf16 loss, 5e-2) and the gradient,
    ignore_index, 3-D and v_chunk_size cases at the same shapes, with bf16 inputs."""
    torch.manual_seed(42)
    x = torch.randn(64, 256, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(1024, 256, device=DEV, dtype=torch.bfloat16)
    t = torch.randint(0, 1024, (64,), device=DEV)
    ref = F.cross_entropy(F.linear(x.float(), w.float()), t)
    loss, _, _ = _run(x, w, t)
    torch.testing.assert_close(loss.float(), ref, rtol=5e-2, atol=5e-2)
    loss_v, _, _ = _run(x, w, t, v_chunk_size=128)
    torch.testing.assert_close(loss_v.float(), ref, rtol=5e-2, atol=5e-2)
    t3 = t.clone()
    t3[::3] = -100
    ref3 = F.cross_entropy(F.linear(x.float(), w.float()), t3, ignore_index=-100)
    loss3, _, _ = _run(x, w, t3)
    torch.testing.assert_close(loss3.float(), ref3, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("bt,h,v,chunk", [(300, 256, 1000, 128), (1, 64, 8, 4096), (513, 128, 3000, 256),
                                          (64, 4096, 2048, 4096)])
def test_lce_small_weights_vs_oracle(bt, h, v, chunk, reduction, gemm_mode):
    """W ~ N(0, 0.02) as in training: loss within 1e-3 relative of the fp32 oracle."""
    torch.manual_seed(bt + v)
    x = torch.randn(bt, h, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(v, h, device=DEV) * 0.02).to(torch.bfloat16)
    t = torch.randint(0, v, (bt,), device=DEV)
    t[torch.rand(bt, device=DEV) < 0.05] = -100
    loss, dx, dw = _run(x, w, t, reduction=reduction, chunk_size=chunk)
    l_ref, dx_ref, dw_ref = oracle.lce_fwd_bwd(x.float().cpu().numpy(), w.float().cpu().numpy(), t.cpu().numpy(), -100,
                                               reduction)
    assert abs(loss.item() - float(l_ref)) <= LOSS_REL * abs(float(l_ref)) + 1e-6
    sx = max(float(np.abs(dx_ref).max()), 1e-6)
    sw = max(float(np.abs(dw_ref).max()), 1e-6)
    assert_close(dx, dx_ref, what="dx", rtol=2e-2, atol=2e-2 * sx)
    assert_close(dw, dw_ref, what="dw", rtol=2e-2, atol=2e-2 * sw)


def test_lce_upstream_gradient_scales_both_grads():
    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy

    torch.manual_seed(5)
    x = torch.randn(200, 128, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(600, 128, device=DEV) * 0.05).to(torch.bfloat16)
    t = torch.randint(0, 600, (200,), device=DEV)
    grads = []
    for k in (1.0, 3.0):
        xs, ws = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        (fused_linear_cross_entropy(xs, ws, t, chunk_size=64) * k).backward()
        grads.append((xs.grad.float(), ws.grad.float()))
    assert_close(grads[1][0], grads[0][0] * 3, what="dx", rtol=1e-2, atol=1e-5)
    assert_close(grads[1][1], grads[0][1] * 3, what="dw", rtol=1e-2, atol=1e-5)


def test_lce_bias_falls_back_to_linear_plus_cross_entropy_like_the_reference():
    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy

    torch.manual_seed(6)
    x = torch.randn(16, 64, device=DEV)
    w = torch.randn(32, 64, device=DEV)
    b = torch.randn(32, device=DEV)
    t = torch.randint(0, 32, (16,), device=DEV)
    torch.testing.assert_close(fused_linear_cross_entropy(x, w, t, bias=b), F.cross_entropy(F.linear(x, w, b), t))


def test_lce_reference_unit_tests_fp32_verbatim():
    """tests/ops/test_fused_linear_cross_entropy.py with its own fp32 inputs, shapes and tolerances
    (fp32 operands run on the tensor cores as tf32)."""
    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy

    def ref(x, w, t, **kw):
        return F.cross_entropy(F.linear(x, w), t, **kw)

    # :18-34 forward loss
    torch.manual_seed(42)
    x = torch.randn(32, 256, device=DEV, requires_grad=True)
    w = torch.randn(1024, 256, device=DEV, requires_grad=True)
    t = torch.randint(0, 1024, (32,), device=DEV)
    torch.testing.assert_close(fused_linear_cross_entropy(x, w, t), ref(x.detach(), w.detach(), t), rtol=1e-3, atol=1e-3)
    # :58-88 gradients
    torch.manual_seed(42)
    x = torch.randn(16, 128, device=DEV, requires_grad=True)
    w = torch.randn(512, 128, device=DEV, requires_grad=True)
    t = torch.randint(0, 512, (16,), device=DEV)
    xr, wr = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    ref(xr, wr, t).backward()
    fused_linear_cross_entropy(x, w, t).backward()
    assert torch.isfinite(x.grad).all() and torch.isfinite(w.grad).all()
    torch.testing.assert_close(x.grad, xr.grad, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(w.grad, wr.grad, rtol=1e-2, atol=1e-2)
    # :91-113 ignore_index
    torch.manual_seed(42)
    x = torch.randn(48, 128, device=DEV)
    w = torch.randn(512, 128, device=DEV)
    t = torch.randint(0, 512, (48,), device=DEV)
    t[::3] = -100
    torch.testing.assert_close(fused_linear_cross_entropy(x, w, t, ignore_index=-100), ref(x, w, t, ignore_index=-100),
                               rtol=1e-3, atol=1e-3)
    # :116-136 3-D input
    x3, t3 = torch.randn(2, 16, 128, device=DEV), torch.randint(0, 512, (2, 16), device=DEV)
    torch.testing.assert_close(fused_linear_cross_entropy(x3, w, t3), ref(x3.view(-1, 128), w, t3.view(-1)),
                               rtol=1e-3, atol=1e-3)
    # :139-159 v_chunk_size
    torch.testing.assert_close(fused_linear_cross_entropy(x, w, t, v_chunk_size=128), ref(x, w, t, ignore_index=-100),
                               rtol=1e-2, atol=1e-2)
    from bastile_b200 import _lib

    _lib.check_status(x.device, "fp32 fused loss")


@pytest.mark.parametrize("name", ["loss_fp32", "grads", "ignore_index", "sum", "ragged"])
def test_lce_golden_reference_fixtures_fp32(name):
    """The reference's own outputs (fp32, CPU) against the kernels fed the same fp32 inputs."""
    g = load_golden(f"lce_{name}.npz")
    x = torch.as_tensor(g["x"]).to(DEV)
    w = torch.as_tensor(g["w"]).to(DEV)
    t = torch.as_tensor(g["t"]).to(DEV)
    red = str(g["reduction"])
    loss, dx, dw = _run(x, w, t, reduction=red)
    assert abs(loss.item() - float(g["loss"])) <= 1e-3 * max(1.0, abs(float(g["loss"])))
    assert_close(dx, g["dx"], what="dx", rtol=1e-2, atol=1e-2 * max(1.0, float(np.abs(g["dx"]).max())))
    assert_close(dw, g["dw"], what="dw", rtol=1e-2, atol=1e-2 * max(1.0, float(np.abs(g["dw"]).max())))


def test_lce_vocab_shards_emulated_on_one_gpu():
    """The sharded path's device steps, run shard by shard on one GPU with the exchange done
    by torch ops: statistics merge, dlogits per shard, dx summed over shards, dW per shard."""
    from bastile_b200 import _lib
    from bastile_b200.ops.fused_linear_cross_entropy import merge_shard_stats

    lib = _lib.get_lib()
    torch.manual_seed(8)
    bt, h, v, n = 160, 128, 1520, 4  # 380 columns per shard: ragged tiles
    vs = v // n
    x = torch.randn(bt, h, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(v, h, device=DEV) * 0.05).to(torch.bfloat16)
    t = torch.randint(0, v, (bt,), device=DEV)
    t[::7] = -100
    dev = x.device
    st = _lib.status_word(dev)
    stream = _lib.stream_ptr(dev)
    ld = (vs + 7) // 8 * 8
    n_vt = int(lib.bt_lce_num_vtiles(vs))
    scal = torch.empty(3, device=DEV)
    _lib.check(lib.bt_lce_count_valid(t.data_ptr(), bt, -100, 1, scal[0:].data_ptr(), scal[1:].data_ptr(), v, st.data_ptr(), stream), "cv")
    logits, stats = [], []
    for r in range(n):
        lg = torch.empty(bt, ld, device=DEV, dtype=torch.bfloat16)
        ts = torch.empty(bt, n_vt, 2, device=DEV)
        tg = torch.empty(bt, device=DEV)
        rs = torch.empty(bt, 3, device=DEV)
        wr = w[r * vs:(r + 1) * vs].contiguous()
        _lib.check(lib.bt_lce_logits_stats(x.data_ptr(), wr.data_ptr(), t.data_ptr(), lg.data_ptr(), ts.data_ptr(),
                                           tg.data_ptr(), bt, h, vs, h, ld, r * vs, -100, 0, st.data_ptr(), stream), "ls")
        _lib.check(lib.bt_lce_row_stats(ts.data_ptr(), tg.data_ptr(), rs.data_ptr(), bt, n_vt, stream), "rs")
        logits.append(lg)
        stats.append(rs)
    merged = merge_shard_stats(torch.stack(stats))
    st_ref = np.stack([oracle.lce_shard_stats(x.float().cpu().numpy(), w[r * vs:(r + 1) * vs].float().cpu().numpy(),
                                              t.cpu().numpy(), -100, r * vs)[0] for r in range(n)])
    m_ref = oracle.merge_shard_stats(st_ref)
    lse = merged[:, 0] + merged[:, 1].log()
    assert_close(lse, m_ref[:, 0] + np.log(m_ref[:, 1]), what="lse", rtol=2e-3, atol=2e-2)
    assert_close(merged[:, 2], m_ref[:, 2], what="target logit", rtol=2e-2, atol=2e-2)
    loss_row = torch.empty(bt, device=DEV)
    dx = torch.zeros(bt, h, device=DEV)
    dws = []
    for r in range(n):
        wr = w[r * vs:(r + 1) * vs].contiguous()
        _lib.check(lib.bt_lce_dlogits(logits[r].data_ptr(), merged.data_ptr(), t.data_ptr(), loss_row.data_ptr(),
                                      scal[1:].data_ptr(), bt, vs, ld, r * vs, -100, 1, 0, stream), "dl")
        part = torch.empty(bt, h, device=DEV)
        _lib.check(lib.bt_gemm(logits[r].data_ptr(), wr.data_ptr(), part.data_ptr(), bt, h, vs, ld, h, h, 1, 0, 0, 2,
                               None, 0, None, st.data_ptr(), stream), "dx")
        dx += part
        dwr = torch.empty(vs, h, device=DEV, dtype=torch.bfloat16)
        _lib.check(lib.bt_gemm(logits[r].data_ptr(), x.data_ptr(), dwr.data_ptr(), vs, h, bt, ld, h, h, 0, 0, 0, 0,
                               None, 0, None, st.data_ptr(), stream), "dw")
        dws.append(dwr)
    _lib.check_status(dev, "sharded lce")
    l_ref, dx_ref, dw_ref = oracle.lce_fwd_bwd(x.float().cpu().numpy(), w.float().cpu().numpy(), t.cpu().numpy(), -100,
                                               "mean", n_shards=n)
    loss = loss_row.sum() * scal[1]
    assert abs(loss.item() - float(l_ref)) <= 2e-3 * abs(float(l_ref))
    assert_close(dx, dx_ref, what="dx", rtol=2e-2, atol=2e-2 * float(np.abs(dx_ref).max()))
    assert_close(torch.cat(dws), dw_ref, what="dw", rtol=2e-2, atol=2e-2 * float(np.abs(dw_ref).max()))


def test_lce_full_size_properties():
    """Benchmark shape hidden[16384,4096] x W[151936,4096], 5 % ignored: loss near ln(V) for
    small weights, sampled-row loss and dx against the oracle, zero gradient on ignored rows,
    rows of dW for unused vocabulary entries all <= 0 scaled softmax mass."""
    torch.manual_seed(2)
    bt, h, v = 16384, 4096, 151936
    x = torch.randn(bt, h, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(v, h, device=DEV, dtype=torch.bfloat16) * 0.02)
    t = torch.randint(0, v, (bt,), device=DEV)
    t[torch.rand(bt, device=DEV) < 0.05] = -100
    loss, dx, dw = _run(x, w, t)
    valid = t != -100
    assert torch.isfinite(dx).all() and torch.isfinite(dw).all()
    assert float(dx[~valid].abs().max()) == 0.0
    rows = torch.tensor([0, 5, 4095, 4096, 9000, 16383], device=DEV)
    rows = rows[valid[rows]]
    torch.backends.cuda.matmul.allow_tf32 = False
    logits = x[rows].float() @ w.float().T
    lse = torch.logsumexp(logits, dim=-1)
    row_loss = lse - logits[torch.arange(len(rows)), t[rows]]
    nv = int(valid.sum())
    p = torch.softmax(logits, -1)
    p[torch.arange(len(rows)), t[rows]] -= 1
    dx_ref = (p / nv) @ w.float()
    assert_close(dx[rows], dx_ref, what="dx rows", rtol=3e-2, atol=3e-2 * float(dx_ref.abs().max()))
    # full loss through a chunked fp32 evaluation on the GPU (no [BT,V] fp32 tensor at once)
    tot = 0.0
    for s in range(0, bt, 2048):
        lg = x[s:s + 2048].float() @ w.float().T
        tot += F.cross_entropy(lg, t[s:s + 2048], ignore_index=-100, reduction="sum").item()
    assert abs(loss.item() - tot / nv) <= LOSS_REL * tot / nv
    # gradient of the weight sums to ~0 over the vocabulary for every hidden unit (softmax - onehot sums to 0)
    col_sum = dw.float().sum(0)
    assert float(col_sum.abs().max()) < 5e-2


def test_lce_out_of_range_label_sets_status_bit():
    """A label >= V (or negative and not ignore_index) makes F.cross_entropy - which the reference
    calls for its loss (:127, :427) - assert on the device.  Here the call completes without waiting
    for the device and the stream's status word carries BT_STATUS_BAD_LABEL, which
    check_all_status() raises on; clean labels leave the word untouched."""
    from bastile_b200 import _lib
    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy

    torch.manual_seed(12)
    x = torch.randn(64, 128, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(512, 128, device=DEV) * 0.05).to(torch.bfloat16)
    t = torch.randint(0, 512, (64,), device=DEV)
    t[3] = -100
    fused_linear_cross_entropy(x, w, t)
    _lib.check_all_status()  # nothing set
    for bad in (512, -7):
        t2 = t.clone()
        t2[5] = bad
        fused_linear_cross_entropy(x, w, t2)
        with pytest.raises(_lib.BastileB200Error, match="label"):
            _lib.check_all_status()
        _lib.check_all_status()  # the word was cleared by the failed check


def test_lce_batched_slice_runs_without_flattening_copy():
    """hidden[:, :-1] of a [B, T, H] tensor with B > 1 cannot be flattened without a copy; with
    entries of >= 1024 rows the op walks the batch entries with their row stride instead (chunks
    never straddle two entries).  Results must equal the oracle's on the flattened rows, and the
    short-entry case (which copies) must agree too."""
    from bastile_b200.ops import fused_linear_cross_entropy as mod
    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy

    torch.manual_seed(13)
    for b, t, chunk in ((2, 1101, 4096), (3, 1030, 512), (4, 65, 4096)):
        h, v = 128, 777
        full = torch.randn(b, t, h, device=DEV, dtype=torch.bfloat16)
        x = full[:, :-1].detach().requires_grad_(True)  # a leaf that is itself a non-flattenable slice
        assert x.stride(0) != x.shape[1] * x.stride(1)
        w = (torch.randn(v, h, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_(True)
        y = torch.randint(0, v, (b, t - 1), device=DEV)
        y[:, ::13] = -100
        assert (t - 1 >= mod._SEGMENT_MIN_ROWS) == (t > 1000)
        loss = fused_linear_cross_entropy(x, w, y, chunk_size=chunk)
        loss.backward()
        l_ref, dx_ref, dw_ref = oracle.lce_fwd_bwd(x.detach().float().cpu().numpy().reshape(-1, h),
                                                   w.detach().float().cpu().numpy(), y.cpu().numpy().reshape(-1),
                                                   -100, "mean")
        assert abs(loss.item() - float(l_ref)) <= 2e-3 * abs(float(l_ref))
        assert x.grad.shape == x.shape
        assert_close(x.grad.reshape(-1, h), dx_ref, what=f"dx b={b}", rtol=2e-2, atol=2e-2 * float(np.abs(dx_ref).max()))
        assert_close(w.grad, dw_ref, what=f"dw b={b}", rtol=2e-2, atol=2e-2 * float(np.abs(dw_ref).max()))


def test_lce_stats_combine_matches_oracle_merge():
    """bt_lce_stats_combine (the cross-shard log-sum-exp merge as one kernel) against the oracle's
    merge and the torch form used on CPU ranks; shard blocks with a stride larger than rows * 3."""
    from bastile_b200 import _lib
    from bastile_b200.ops.fused_linear_cross_entropy import merge_shard_stats

    lib = _lib.get_lib()
    rng = np.random.default_rng(5)
    n_shards, rows, cap = 8, 1000, 1024
    st = rng.standard_normal((n_shards, cap, 3)).astype(np.float32) * 5
    st[..., 1] = np.abs(st[..., 1]) + 0.1
    st[..., 2] = 0.0
    st[rng.integers(0, n_shards, rows), np.arange(rows), 2] = rng.standard_normal(rows).astype(np.float32)
    g = torch.tensor(st, device=DEV)
    out = torch.empty(rows, 3, device=DEV)
    _lib.check(lib.bt_lce_stats_combine(g.data_ptr(), out.data_ptr(), rows, cap * 3, n_shards,
                                        _lib.stream_ptr(g.device)), "bt_lce_stats_combine")
    want = oracle.merge_shard_stats(st[:, :rows])
    got = out.cpu().numpy()
    np.testing.assert_allclose(got[:, 0] + np.log(got[:, 1]), want[:, 0] + np.log(want[:, 1]), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(got[:, 2], want[:, 2], rtol=1e-6, atol=1e-6)
    torch_form = merge_shard_stats(g[:, :rows]).cpu().numpy()
    np.testing.assert_allclose(got, torch_form, rtol=1e-5, atol=1e-5)
