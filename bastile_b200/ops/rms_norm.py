"""RMSNorm on the sm_100a kernels (replaces src/bastile/ops/rms_norm.py).

``y = x * rsqrt(mean(x^2) + eps) * weight`` computed in fp32 and rounded once
to the input dtype, as the reference kernel does (rms_norm.py:15-34).  The
backward returns ``dx`` and ``dw`` from one kernel launch; the column sums for
``dw`` are finished on the device (no torch reduction kernels, no partials
tensor - rms_norm.py:128-153 needed both).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import _lib
from ..registry import register_patch


def _as_rows(t: torch.Tensor, n: int) -> torch.Tensor:
    """[..., n] -> 2-D [rows, n] with unit inner stride (a view when possible)."""
    t2 = t.reshape(-1, n)
    if t2.stride(-1) != 1 or (t2.shape[0] > 1 and t2.stride(0) < n):
        t2 = t2.contiguous()
    return t2


class RMSNormFunction(torch.autograd.Function):
    """autograd wrapper of bt_rmsnorm_fwd / bt_rmsnorm_bwd."""

    @staticmethod
    def forward(ctx, x, weight, eps):
        dev = _lib.require_cuda(x, weight)
        lib = _lib.get_lib()
        code = _lib.dtype_code(x.dtype)
        shape = x.shape
        n = shape[-1]
        if weight.numel() != n:
            raise ValueError(f"rms_norm: weight has {weight.numel()} elements, rows have {n}")
        x2 = _as_rows(x, n)
        m = x2.shape[0]
        w = weight.detach()
        if w.dtype != x.dtype:
            w = w.to(x.dtype)
        w = w.contiguous()
        y = torch.empty((m, n), dtype=x.dtype, device=dev)
        rstd = torch.empty((m,), dtype=torch.float32, device=dev)
        with _lib.device_of(dev), _lib.timed("rmsnorm_fwd", 1, dev):
            rc = lib.bt_rmsnorm_fwd(x2.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), m, n,
                                    x2.stride(0) if m > 1 else n, n, float(eps), code, _lib.stream_ptr(dev))
        _lib.check(rc, "bt_rmsnorm_fwd")
        ctx.save_for_backward(x2, w, rstd)
        ctx.shape = shape
        ctx.weight_dtype = weight.dtype
        ctx.eps = eps
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        dev = x2.device
        lib = _lib.get_lib()
        m, n = x2.shape
        code = _lib.dtype_code(x2.dtype)
        if dy.dtype != x2.dtype:
            dy = dy.to(x2.dtype)
        dy2 = _as_rows(dy, n)
        dx = torch.empty((m, n), dtype=x2.dtype, device=dev)
        dw = torch.empty((n,), dtype=x2.dtype, device=dev)
        ws = _lib.zero_workspace(dev, int(lib.bt_rmsnorm_bwd_ws_bytes(n)))
        with _lib.device_of(dev), _lib.timed("rmsnorm_bwd", 1, dev):
            rc = lib.bt_rmsnorm_bwd(dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                    dw.data_ptr(), ws.data_ptr(), m, n, dy2.stride(0) if m > 1 else n,
                                    x2.stride(0) if m > 1 else n, n, code, _lib.stream_ptr(dev))
        _lib.check(rc, "bt_rmsnorm_bwd")
        if dw.dtype != ctx.weight_dtype:
            dw = dw.to(ctx.weight_dtype)
        return dx.view(ctx.shape), dw, None


class B200RMSNorm(nn.Module):
    """Drop-in for ``Qwen3RMSNorm``: same constructor, ``weight`` parameter and
    ``variance_epsilon`` attribute (rms_norm.py:156-168), so checkpoints load."""

    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return RMSNormFunction.apply(x, self.weight, self.variance_epsilon)

    def extra_repr(self) -> str:
        return f"{self.weight.shape[0]}, eps={self.variance_epsilon}"


# Names under which the reference exposes the same things.
CuTileRMSNormFunction = RMSNormFunction
CuTileRMSNorm = B200RMSNorm


def rms_norm(x, weight, eps=1e-6, **_kw):
    """Stand-alone RMSNorm (rms_norm.py:171-173)."""
    return RMSNormFunction.apply(x, weight, eps)


def warmup_rms_norm(hidden_size: int, dtype=torch.bfloat16, device="cuda"):
    """One forward+backward at ``hidden_size`` (rms_norm.py:176-181)."""
    x = torch.randn(2, hidden_size, dtype=dtype, device=device, requires_grad=True)
    w = torch.ones(hidden_size, dtype=dtype, device=device, requires_grad=True)
    rms_norm(x, w, 1e-6).sum().backward()
    torch.cuda.synchronize()


register_patch(
    name="rms_norm_qwen3",
    description="sm_100a RMSNorm for Qwen3 (row-in-registers fwd, single-launch bwd)",
    target_module="transformers.models.qwen3.modeling_qwen3",
    target_attr="Qwen3RMSNorm",
    replacement=B200RMSNorm,
    has_backward=True,
    priority=10,
    models=["qwen3"],
)
