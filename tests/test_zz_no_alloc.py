"""bt_rmsnorm_bwd_noalloc: the RMSNorm backward whose scratch is built into the library, for
callers that may not allocate device memory themselves (FFI hosts living inside a framework's
memory pool, latency-critical loops that cannot afford cudaMalloc's device-wide sync).

It must give what bt_rmsnorm_bwd gives with a caller-owned scratch buffer - checked here through
the C ABI, on two calls in a row (the built-in array is shared by all calls and keeps the last
call's contents, so the second call is the one that shows whether it is cleared properly).
This file is collected last on purpose."""

import pytest
import torch

from conftest import BF16_TOL, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _both(lib, _lib, m, n, dtype, seed):
    torch.manual_seed(seed)
    dev = torch.device(DEV, torch.cuda.current_device())
    x = torch.randn(m, n, device=dev).to(dtype)
    w = (1 + 0.02 * torch.randn(n, device=dev)).to(dtype)
    dy = torch.randn(m, n, device=dev).to(dtype)
    y = torch.empty_like(x)
    rstd = torch.empty(m, device=dev, dtype=torch.float32)
    code = _lib.dtype_code(dtype)
    stream = _lib.stream_ptr(dev)
    _lib.check(lib.bt_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), m, n, n, n, 1e-6, code,
                                  stream), "bt_rmsnorm_fwd")
    ws = torch.zeros(int(lib.bt_rmsnorm_bwd_ws_bytes(n)), dtype=torch.uint8, device=dev)
    dx_a, dw_a = torch.empty_like(x), torch.empty_like(w)
    _lib.check(lib.bt_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx_a.data_ptr(),
                                  dw_a.data_ptr(), ws.data_ptr(), m, n, n, n, n, code, stream), "bt_rmsnorm_bwd")
    dx_b, dw_b = torch.full_like(x, float("nan")), torch.full_like(w, float("nan"))
    before = torch.cuda.memory_allocated(dev)
    _lib.check(lib.bt_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx_b.data_ptr(),
                                          dw_b.data_ptr(), m, n, n, n, n, code, stream), "bt_rmsnorm_bwd_noalloc")
    assert torch.cuda.memory_allocated(dev) == before
    torch.cuda.synchronize()
    return (dx_a, dw_a), (dx_b, dw_b), m


def test_noalloc_matches_caller_scratch_twice_in_a_row():
    from bastile_b200 import _lib

    lib = _lib.get_lib()
    # two different shapes back to back: wide rows (block kernel), then short rows (rows kernel);
    # then the first shape again so that leftovers of a larger N would show
    for seed, (m, n, dtype) in enumerate([(513, 4096, torch.bfloat16), (4100, 128, torch.bfloat16),
                                          (513, 4096, torch.bfloat16), (77, 1000, torch.float32)]):
        (dx_a, dw_a), (dx_b, dw_b), rows = _both(lib, _lib, m, n, dtype, seed)
        assert torch.equal(dx_a, dx_b), "dx must be bit-identical: same kernel, same inputs"
        # dw is a sum of fp32 atomics whose order differs from launch to launch
        tol = dict(rtol=BF16_TOL["rtol"], atol=BF16_TOL["atol"] * max(1.0, rows ** 0.5 / 4))
        assert_close(dw_b, dw_a, what=f"dw ({m}x{n})", **tol)


def test_noalloc_rejects_rows_wider_than_its_scratch():
    from bastile_b200 import _lib

    lib = _lib.get_lib()
    dev = torch.device(DEV, torch.cuda.current_device())
    t = torch.zeros(8, device=dev)
    rc = lib.bt_rmsnorm_bwd_noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                    t.data_ptr(), 1, 16385, 16385, 16385, 16385, 0, _lib.stream_ptr(dev))
    assert rc == -5
    assert b"exceeds the built-in scratch" in lib.bt_last_error()
