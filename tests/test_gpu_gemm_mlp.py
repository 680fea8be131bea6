"""The tcgen05 GEMM core and the fused SwiGLU MLP through the C ABI, against the oracle."""

import numpy as np
import pytest
import torch

import oracle
from conftest import BF16_TOL, assert_close, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=[(1, 0), (1, 1), (0, 0)], ids=["cta_pairs", "cta_pairs_dynamic_tiles", "single_cta"])
def gemm_mode(request):
    """Run a test under both tilings of the tensor-core kernels (cta_group::2 pairs, the default,
    and one CTA per tile), the pairs also with tiles drawn from a global counter."""
    from bastile_b200 import _lib

    lib = _lib.get_lib()
    pairs, dynamic = request.param
    prev = lib.bt_set_gemm_cta_pairs(pairs), lib.bt_set_gemm_dynamic_tiles(dynamic)
    yield request.param
    lib.bt_set_gemm_cta_pairs(prev[0])
    lib.bt_set_gemm_dynamic_tiles(prev[1])


@pytest.mark.parametrize("M,N,K", [(2500, 5000, 64), (2500, 5000, 200), (4096, 6144, 1024), (20000, 300, 520)])
def test_dynamic_tile_handout_gives_the_same_bits(M, N, K):
    """More tiles than CTA pairs (so tiles really are drawn at run time), down to one k-block
    per tile: every output element comes from the same arithmetic as with the fixed deal."""
    from bastile_b200 import _lib

    lib = _lib.get_lib()
    torch.manual_seed(M + K)
    A = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    B = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    prev = lib.bt_set_gemm_dynamic_tiles(0)
    try:
        fixed = _gemm(A, B, M, N, K, 1, 1)
        lib.bt_set_gemm_dynamic_tiles(1)
        for _ in range(3):
            assert torch.equal(_gemm(A, B, M, N, K, 1, 1), fixed)
    finally:
        lib.bt_set_gemm_dynamic_tiles(prev)
    ref = A[:64].double() @ B[:512].double().T
    assert_close(fixed[:64, :512], ref.cpu().numpy(), what="D", rtol=2e-2, atol=2e-2 * max(1.0, np.sqrt(K) / 4))


def _gemm(A, B, M, N, K, ak, bk, out_dtype=None, addend=None, alpha=None):
    from bastile_b200 import _lib

    lib = _lib.get_lib()
    dev = A.device
    out_dtype = out_dtype or A.dtype
    D = torch.full((M, N), float("nan"), device=dev, dtype=out_dtype)
    st = _lib.status_word(dev)
    rc = lib.bt_gemm(A.data_ptr(), B.data_ptr(), D.data_ptr(), M, N, K, A.stride(0), B.stride(0), N, int(ak), int(bk),
                     _lib.dtype_code(A.dtype), _lib.dtype_code(out_dtype),
                     addend.data_ptr() if addend is not None else None, N,
                     alpha.data_ptr() if alpha is not None else None, st.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "bt_gemm")
    _lib.check_status(dev, "bt_gemm")
    return D


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("ak,bk", [(1, 1), (1, 0), (0, 1), (0, 0)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (136, 264, 72), (8, 8, 8), (300, 520, 1000), (1, 1000, 130),
                                   (640, 1024, 520)])
def test_gemm_layouts_and_ragged_shapes(M, N, K, ak, bk, dtype, gemm_mode):
    if (ak or bk) and K % 8:
        pytest.skip("K-major operands need a row stride that is a multiple of 8 elements")
    torch.manual_seed(M + N + K)
    A = torch.randn((M, K) if ak else (K, (M + 7) // 8 * 8), device=DEV).to(dtype)
    B = torch.randn((N, K) if bk else (K, (N + 7) // 8 * 8), device=DEV).to(dtype)
    Af = A.float().cpu().numpy() if ak else A.float().cpu().numpy().T[:M]
    Bf = B.float().cpu().numpy() if bk else B.float().cpu().numpy().T[:N]
    ref = Af.astype(np.float64) @ Bf.astype(np.float64).T
    D = _gemm(A, B, M, N, K, ak, bk)
    tol = dict(rtol=2e-2, atol=2e-2 * max(1.0, np.sqrt(K) / 4))
    assert_close(D, ref, what="D", **tol)


@pytest.mark.parametrize("ak,bk", [(1, 1), (1, 0), (0, 1), (0, 0)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 32), (136, 264, 72), (300, 520, 1000), (640, 1024, 516)])
def test_gemm_fp32_operands_as_tf32(M, N, K, ak, bk, gemm_mode):
    """fp32 storage, tf32 products, fp32 accumulation: against float64 with a tf32-sized tolerance."""
    torch.manual_seed(M + N + K)
    A = torch.randn((M, K) if ak else (K, (M + 3) // 4 * 4), device=DEV)
    B = torch.randn((N, K) if bk else (K, (N + 3) // 4 * 4), device=DEV)
    Af = A.double().cpu().numpy() if ak else A.double().cpu().numpy().T[:M]
    Bf = B.double().cpu().numpy() if bk else B.double().cpu().numpy().T[:N]
    ref = Af @ Bf.T
    D = _gemm(A, B, M, N, K, ak, bk, out_dtype=torch.float32)
    assert_close(D, ref, what="D", rtol=2e-3, atol=2e-3 * np.sqrt(K))


def test_mlp_fp32_vs_oracle():
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction

    x, wg, wu, wd, dy = _mlp_case(200, 256, 640, torch.float32, seed=9)
    xs, wgs, wus, wds = (a.clone().requires_grad_(True) for a in (x, wg, wu, wd))
    y = SwiGLUMLPFunction.apply(xs, wgs, wus, wds)
    y.backward(dy)
    f = lambda a: a.detach().cpu().numpy()  # noqa: E731
    y_ref = oracle.mlp_fwd(f(x), f(wg), f(wu), f(wd))[0]
    dx_ref, dwg_ref, dwu_ref, dwd_ref = oracle.mlp_bwd(f(dy), f(x), f(wg), f(wu), f(wd))
    for got, want, what in ((y, y_ref, "y"), (xs.grad, dx_ref, "dx"), (wgs.grad, dwg_ref, "dwg"),
                            (wus.grad, dwu_ref, "dwu"), (wds.grad, dwd_ref, "dwd")):
        assert got.dtype == torch.float32
        assert_close(got, want, what=what, rtol=5e-3, atol=5e-3 * max(1.0, float(np.abs(want).max())))


def test_gemm_fp32_out_addend_alpha_and_inplace_accumulate():
    torch.manual_seed(0)
    M, N, K = 200, 328, 264
    A = torch.randn(M, K, device=DEV).bfloat16()
    B = torch.randn(N, K, device=DEV).bfloat16()
    add = torch.randn(M, N, device=DEV)
    alpha = torch.tensor([0.25], device=DEV)
    ref = (A.float() @ B.float().T + add) * 0.25
    D = _gemm(A, B, M, N, K, 1, 1, out_dtype=torch.float32, addend=add, alpha=alpha)
    assert_close(D, ref, what="fp32 out", rtol=1e-4, atol=1e-3)
    D16 = _gemm(A, B, M, N, K, 1, 1, addend=add, alpha=alpha)
    assert_close(D16, ref, what="bf16 out", **BF16_TOL)
    # accumulate in place: addend aliases the fp32 result
    from bastile_b200 import _lib

    lib = _lib.get_lib()
    acc = add.clone()
    st = _lib.status_word(acc.device)
    for _ in range(2):
        _lib.check(lib.bt_gemm(A.data_ptr(), B.data_ptr(), acc.data_ptr(), M, N, K, K, K, N, 1, 1, 0, 2, acc.data_ptr(),
                               N, None, st.data_ptr(), _lib.stream_ptr(acc.device)), "bt_gemm")
    _lib.check_status(acc.device, "bt_gemm")
    assert_close(acc, add + 2 * (A.float() @ B.float().T), what="accumulate", rtol=1e-4, atol=2e-3)


def test_gemm_persistent_many_tiles_matches_fp32_reference(gemm_mode):
    """More tiles than SMs (several per CTA, both accumulator buffers, ring wrap-around)."""
    torch.manual_seed(1)
    M, N, K = 2048, 5120, 1024
    A = (torch.randn(M, K, device=DEV) * 0.1).bfloat16()
    B = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    D = _gemm(A, B, M, N, K, 1, 1)
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = A.float() @ B.float().T
    assert_close(D, ref, what="D", **BF16_TOL)


def test_gemm_rejects_bad_arguments():
    from bastile_b200 import _lib

    lib = _lib.get_lib()
    A = torch.randn(16, 20, device=DEV).bfloat16()  # row stride 20: not a multiple of 8
    B = torch.randn(16, 20, device=DEV).bfloat16()
    D = torch.empty(16, 16, device=DEV).bfloat16()
    st = _lib.status_word(A.device)
    rc = lib.bt_gemm(A.data_ptr(), B.data_ptr(), D.data_ptr(), 16, 16, 20, 20, 20, 16, 1, 1, 0, 0, None, 0, None,
                     st.data_ptr(), _lib.stream_ptr(A.device))
    assert rc == -1 and b"multiple of 8" in lib.bt_last_error()
    rc = lib.bt_gemm(A.data_ptr(), B.data_ptr(), D.data_ptr(), 16, 16, 16, 24, 24, 16, 1, 1, 2, 0, None, 0, None,
                     st.data_ptr(), _lib.stream_ptr(A.device))
    assert rc == -1  # fp32 operands give an fp32 result, nothing narrower


# ------------------------------------------------------------------------------ MLP
def _mlp_case(t, hidden, inter, dtype, seed=0, w_std=0.05):
    torch.manual_seed(seed)
    x = torch.randn(t, hidden, device=DEV).to(dtype)
    wg = (torch.randn(inter, hidden, device=DEV) * w_std).to(dtype)
    wu = (torch.randn(inter, hidden, device=DEV) * w_std).to(dtype)
    wd = (torch.randn(hidden, inter, device=DEV) * w_std).to(dtype)
    dy = torch.randn(t, hidden, device=DEV).to(dtype)
    return x, wg, wu, wd, dy


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("t,hidden,inter", [(21, 64, 160), (256, 256, 768), (300, 512, 1384), (1, 128, 256)])
def test_mlp_fwd_bwd_vs_oracle(t, hidden, inter, dtype, gemm_mode):
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction

    x, wg, wu, wd, dy = _mlp_case(t, hidden, inter, dtype)
    xs, wgs, wus, wds = (a.clone().requires_grad_(True) for a in (x, wg, wu, wd))
    y = SwiGLUMLPFunction.apply(xs, wgs, wus, wds)
    y.backward(dy)
    f = lambda a: a.detach().float().cpu().numpy()  # noqa: E731
    y_ref, _, _, _ = oracle.mlp_fwd(f(x), f(wg), f(wu), f(wd))
    dx_ref, dwg_ref, dwu_ref, dwd_ref = oracle.mlp_bwd(f(dy), f(x), f(wg), f(wu), f(wd))

    def tol(ref):
        s = float(np.abs(ref).max())
        return dict(rtol=2e-2, atol=2e-2 * max(1.0, s))

    assert_close(y, y_ref, what="y", **tol(y_ref))
    assert_close(xs.grad, dx_ref, what="dx", **tol(dx_ref))
    assert_close(wgs.grad, dwg_ref, what="dwg", **tol(dwg_ref))
    assert_close(wus.grad, dwu_ref, what="dwu", **tol(dwu_ref))
    assert_close(wds.grad, dwd_ref, what="dwd", **tol(dwd_ref))


def test_mlp_golden_hf_fixture():
    """HF eager Qwen3MLP outputs (fp32) vs the bf16 kernels on the same inputs."""
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction

    g = load_golden("mlp_hf.npz")
    t = lambda a: torch.as_tensor(a).to(DEV, torch.bfloat16)  # noqa: E731
    x, wg, wu, wd = (t(g[k]).requires_grad_(True) for k in ("x", "wg", "wu", "wd"))
    y = SwiGLUMLPFunction.apply(x, wg, wu, wd)
    y.backward(t(g["dy"]))
    assert_close(y, g["y"], what="y", **BF16_TOL)
    assert_close(x.grad, g["dx"], what="dx", **BF16_TOL)
    assert_close(wg.grad, g["dwg"], what="dwg", rtol=2e-2, atol=4e-2)
    assert_close(wu.grad, g["dwu"], what="dwu", rtol=2e-2, atol=4e-2)
    assert_close(wd.grad, g["dwd"], what="dwd", rtol=2e-2, atol=4e-2)


def test_mlp_module_matches_hf_eager_module():
    """B200SwiGLUMLP against transformers' Qwen3MLP with the same weights (bf16 on the GPU)."""
    import transformers.models.qwen3.modeling_qwen3 as q3
    from golden.make_golden import tiny_qwen3_config

    from bastile_b200.ops.swiglu import B200SwiGLUMLP

    import bastile_b200

    bastile_b200.reset()
    cfg = tiny_qwen3_config()
    torch.manual_seed(0)
    hf = q3.Qwen3MLP(cfg).to(DEV, torch.bfloat16)
    ours = B200SwiGLUMLP(cfg).to(DEV, torch.bfloat16)
    ours.load_state_dict(hf.state_dict())
    x = torch.randn(2, 128, cfg.hidden_size, device=DEV, dtype=torch.bfloat16)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya, yb = ours(xa), hf(xb)
    dy = torch.randn_like(ya)
    ya.backward(dy)
    yb.backward(dy)
    assert_close(ya, yb, what="y", **BF16_TOL)
    assert_close(xa.grad, xb.grad, what="dx", **BF16_TOL)
    for (n, pa), (_, pb) in zip(ours.named_parameters(), hf.named_parameters()):
        assert_close(pa.grad, pb.grad, what=n, rtol=2e-2, atol=5e-2)


def test_mlp_full_size_linearity_and_sampled_rows():
    """Benchmark shape x[8192,4096], intermediate 12288: sampled rows vs the oracle, and the
    backward's linearity in the upstream gradient."""
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction

    x, wg, wu, wd, dy = _mlp_case(8192, 4096, 12288, torch.bfloat16, seed=1, w_std=0.02)
    xs = x.clone().requires_grad_(True)
    wgs, wus, wds = (a.clone().requires_grad_(True) for a in (wg, wu, wd))
    y = SwiGLUMLPFunction.apply(xs, wgs, wus, wds)
    y.backward(dy)
    rows = torch.tensor([0, 1, 127, 128, 4095, 8191], device=DEV)
    f = lambda a: a.detach().float().cpu().numpy()  # noqa: E731
    y_ref, _, _, _ = oracle.mlp_fwd(f(x[rows]), f(wg), f(wu), f(wd))
    # gate/up/h are rounded to bf16 on the way (as in the op being replaced): scale atol by |y|
    assert_close(y[rows], y_ref, what="y rows", rtol=2e-2, atol=2e-2 * max(1.0, float(np.abs(y_ref).max()) / 2))
    # dx rows depend only on their own row of x and dy
    dx_ref, _, _, _ = oracle.mlp_bwd(f(dy[rows]), f(x[rows]), f(wg), f(wu), f(wd))
    assert_close(xs.grad[rows], dx_ref, what="dx rows", rtol=2e-2, atol=2e-2 * max(1.0, float(np.abs(dx_ref).max()) / 2))
    # a slice of dWd = dy^T h against fp32 matmul of the saved bf16 operands
    torch.backends.cuda.matmul.allow_tf32 = False
    h = torch.nn.functional.silu(x.float() @ wg.float().T[:, :256]) * (x.float() @ wu.float().T[:, :256])
    dwd_ref = dy.float().T @ h
    assert_close(wds.grad[:, :256], dwd_ref, what="dwd slice", rtol=2e-2, atol=2e-2 * float(dwd_ref.abs().max()))
    # linearity: backward(2*dy) == 2*backward(dy)
    xs2 = x.clone().requires_grad_(True)
    y2 = SwiGLUMLPFunction.apply(xs2, wg, wu, wd)
    y2.backward(dy * 2)
    assert_close(xs2.grad, xs.grad.float() * 2, what="linearity", rtol=1e-2, atol=1e-2)


def test_mlp_bwd_c_abi_with_separate_buffers_and_skipped_outputs():
    """bt_mlp_bwd called directly: dgate/dup and dWg/dWu in unrelated buffers (no stacked product),
    dWu skipped with NULL - results must equal the autograd path that uses the stacked buffers."""
    from bastile_b200 import _lib
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction

    lib = _lib.get_lib()
    t, hidden, inter = 200, 256, 640
    x, wg, wu, wd, dy = _mlp_case(t, hidden, inter, torch.bfloat16, seed=4)
    xs, wgs, wus, wds = (a.clone().requires_grad_(True) for a in (x, wg, wu, wd))
    SwiGLUMLPFunction.apply(xs, wgs, wus, wds).backward(dy)
    dev = x.device
    gate, up, h = (torch.empty(t, inter, device=dev, dtype=torch.bfloat16) for _ in range(3))
    y = torch.empty(t, hidden, device=dev, dtype=torch.bfloat16)
    st = _lib.status_word(dev)
    stream = _lib.stream_ptr(dev)
    _lib.check(lib.bt_mlp_fwd(x.data_ptr(), wg.data_ptr(), wu.data_ptr(), wd.data_ptr(), gate.data_ptr(), up.data_ptr(),
                              h.data_ptr(), y.data_ptr(), t, hidden, inter, hidden, None, 0, 0, st.data_ptr(), stream), "fwd")
    dgate, dup = (torch.empty(t, inter, device=dev, dtype=torch.bfloat16) for _ in range(2))
    dx = torch.empty_like(x)
    dwg, dwd = torch.empty_like(wg), torch.empty_like(wd)
    _lib.check(lib.bt_mlp_bwd(dy.data_ptr(), x.data_ptr(), wg.data_ptr(), wu.data_ptr(), wd.data_ptr(), gate.data_ptr(),
                              up.data_ptr(), h.data_ptr(), dgate.data_ptr(), dup.data_ptr(), dx.data_ptr(),
                              dwg.data_ptr(), None, dwd.data_ptr(), t, hidden, inter, hidden, hidden, inter, 0,
                              st.data_ptr(), stream), "bwd")
    _lib.check_status(dev, "mlp c abi")
    assert torch.equal(dx, xs.grad) and torch.equal(dwd, wds.grad)
    assert_close(dwg, wgs.grad, what="dWg", rtol=1e-2, atol=1e-2 * float(wgs.grad.float().abs().max()))


@pytest.mark.parametrize("pairs", [1, 0])
def test_tile_stores_give_the_same_bits_as_register_stores(pairs):
    """16-bit results staged in shared memory and written by tile stores (the default) against the
    per-thread stores: MLP forward/backward, the fused loss and a plain product, with ragged row and
    column counts (rows and columns past the tensor are clipped by the store)."""
    from bastile_b200 import _lib
    from bastile_b200.ops.fused_linear_cross_entropy import fused_linear_cross_entropy
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction

    lib = _lib.get_lib()
    prev_pairs = lib.bt_set_gemm_cta_pairs(pairs)
    prev = lib.bt_set_gemm_tile_stores(-1)
    results = {}
    try:
        for mode in (1, 0):
            lib.bt_set_gemm_tile_stores(mode)
            out = []
            for t, hidden, inter in ((333, 256, 640), (1000, 512, 1288), (7, 128, 136)):
                x, wg, wu, wd, dy = _mlp_case(t, hidden, inter, torch.bfloat16, seed=6)
                xs, wgs, wus, wds = (a.clone().requires_grad_(True) for a in (x, wg, wu, wd))
                y = SwiGLUMLPFunction.apply(xs, wgs, wus, wds)
                y.backward(dy)
                out += [y.detach(), xs.grad, wgs.grad, wus.grad, wds.grad]
            torch.manual_seed(7)
            for rows, hidden, vocab in ((300, 128, 1000), (77, 256, 4104)):
                x = torch.randn(rows, hidden, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
                w = (torch.randn(vocab, hidden, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_(True)
                tg = torch.randint(0, vocab, (rows,), device=DEV)
                tg[::5] = -100
                loss = fused_linear_cross_entropy(x, w, tg, chunk_size=128)
                loss.backward()
                out += [loss.detach(), x.grad, w.grad]
            a = torch.randn(515, 200, device=DEV, dtype=torch.float16)
            b = torch.randn(264, 200, device=DEV, dtype=torch.float16)
            d = torch.empty(515, 264, device=DEV, dtype=torch.float16)
            st = _lib.status_word(a.device)
            _lib.check(lib.bt_gemm(a.data_ptr(), b.data_ptr(), d.data_ptr(), 515, 264, 200, 200, 200, 264, 1, 1, 1, 1,
                                   None, 0, None, st.data_ptr(), _lib.stream_ptr(a.device)), "gemm")
            out.append(d)
            _lib.check_status(a.device, f"tile stores {mode}")
            results[mode] = out
    finally:
        lib.bt_set_gemm_tile_stores(prev)
        lib.bt_set_gemm_cta_pairs(prev_pairs)
    for i, (u, v) in enumerate(zip(results[1], results[0])):
        assert torch.equal(u, v), f"result {i} differs between tile stores and register stores"
    ref = (a.float() @ b.float().T)
    assert_close(results[1][-1], ref, what="plain product", rtol=2e-2, atol=2e-2 * float(ref.abs().max()))


def test_wait_limit_can_be_raised_and_is_validated():
    """bt_set_wait_limit_ms: out-of-range values are refused, a raised limit leaves results alone."""
    from bastile_b200 import _lib
    from bastile_b200.ops.swiglu import SwiGLUMLPFunction

    lib = _lib.get_lib()
    assert lib.bt_set_wait_limit_ms(0) != 0 and b"limit" in lib.bt_last_error()
    assert lib.bt_set_wait_limit_ms(10 ** 7) != 0
    x, wg, wu, wd, dy = _mlp_case(130, 128, 256, torch.bfloat16, seed=9)
    y0 = SwiGLUMLPFunction.apply(x, wg, wu, wd)
    try:
        _lib.check(lib.bt_set_wait_limit_ms(5000), "bt_set_wait_limit_ms")
        y1 = SwiGLUMLPFunction.apply(x, wg, wu, wd)
        _lib.check_status(x.device, "raised wait limit")
        assert torch.equal(y0, y1)
    finally:
        _lib.check(lib.bt_set_wait_limit_ms(1000), "bt_set_wait_limit_ms")
