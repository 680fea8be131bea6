"""SwiGLU on sm_100a: the stand-alone ``silu(gate) * up`` op and the fused MLP block
(replaces src/bastile/ops/swiglu.py).

``SwiGLUFunction`` / ``swiglu`` are the elementwise op of the reference
(swiglu.py:149-167) as streaming kernels.  ``B200SwiGLUMLP`` replaces
``Qwen3MLP``: where the reference runs three cuBLAS GEMMs around the elementwise
kernel (swiglu.py:170-187), the gate and up projections here are ONE tcgen05
kernel with two accumulators in tensor memory whose epilogue applies
``silu(gate) * up`` before anything is written, and the backward fuses the
``dgate`` / ``dup`` arithmetic into the epilogue of the ``dy @ W_down`` product.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import _lib
from ..registry import register_patch


def _rows(t: torch.Tensor) -> torch.Tensor:
    n = t.shape[-1]
    t2 = t.reshape(-1, n)
    if t2.stride(-1) != 1 or (t2.shape[0] > 1 and t2.stride(0) < n):
        t2 = t2.contiguous()
    return t2


def _ld(t2: torch.Tensor) -> int:
    return t2.stride(0) if t2.shape[0] > 1 else t2.shape[1]


class SwiGLUFunction(torch.autograd.Function):
    """``silu(gate) * up`` with the backward recomputed from (gate, up)."""

    @staticmethod
    def forward(ctx, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        dev = _lib.require_cuda(gate, up)
        if gate.shape != up.shape or gate.dtype != up.dtype:
            raise ValueError("swiglu: gate and up must share shape and dtype")
        lib = _lib.get_lib()
        g2, u2 = _rows(gate), _rows(up)
        rows, cols = g2.shape
        out = torch.empty((rows, cols), dtype=gate.dtype, device=dev)
        with _lib.device_of(dev), _lib.timed("swiglu_fwd", 1, dev):
            rc = lib.bt_swiglu_fwd(g2.data_ptr(), u2.data_ptr(), out.data_ptr(), rows, cols, _ld(g2), _ld(u2), cols,
                                   _lib.dtype_code(gate.dtype), _lib.stream_ptr(dev))
        _lib.check(rc, "bt_swiglu_fwd")
        ctx.save_for_backward(g2, u2)
        ctx.shape = gate.shape
        return out.view(gate.shape)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        g2, u2 = ctx.saved_tensors
        dev = g2.device
        lib = _lib.get_lib()
        rows, cols = g2.shape
        if grad_output.dtype != g2.dtype:
            grad_output = grad_output.to(g2.dtype)
        d2 = _rows(grad_output)
        dg = torch.empty((rows, cols), dtype=g2.dtype, device=dev)
        du = torch.empty((rows, cols), dtype=g2.dtype, device=dev)
        with _lib.device_of(dev), _lib.timed("swiglu_bwd", 1, dev):
            rc = lib.bt_swiglu_bwd(d2.data_ptr(), g2.data_ptr(), u2.data_ptr(), dg.data_ptr(), du.data_ptr(), rows,
                                   cols, _ld(d2), _ld(g2), _ld(u2), cols, cols, _lib.dtype_code(g2.dtype),
                                   _lib.stream_ptr(dev))
        _lib.check(rc, "bt_swiglu_bwd")
        return dg.view(ctx.shape), du.view(ctx.shape)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` (swiglu.py:165-167)."""
    return SwiGLUFunction.apply(gate, up)


# fp32 tensors are fed to the tensor cores as tf32 (10-bit mantissa products, fp32 accumulation)
_GEMM_DTYPES = (torch.bfloat16, torch.float16, torch.float32)


class SwiGLUMLPFunction(torch.autograd.Function):
    """down(silu(gate(x)) * up(x)) as fused tcgen05 kernels (bt_mlp_fwd / bt_mlp_bwd).

    With ``residual`` the result is ``residual + down(...)``, added in the down projection's
    epilogue; its gradient is the incoming gradient itself."""

    @staticmethod
    def forward(ctx, x, wg, wu, wd, residual=None):
        dev = _lib.require_cuda(x, wg, wu, wd)
        lib = _lib.get_lib()
        if x.dtype not in _GEMM_DTYPES:
            raise TypeError(f"bastile_b200 MLP: unsupported activation dtype {x.dtype}")
        inter, hidden = wg.shape
        if wu.shape != (inter, hidden) or wd.shape != (hidden, inter) or x.shape[-1] != hidden:
            raise ValueError("bastile_b200 MLP: weight shapes do not match a SwiGLU block")
        code = _lib.dtype_code(x.dtype)
        x2 = _rows(x)
        t = x2.shape[0]
        wgc, wuc, wdc = (w.detach().to(x.dtype).contiguous() for w in (wg, wu, wd))
        gate = torch.empty((t, inter), dtype=x.dtype, device=dev)
        up = torch.empty((t, inter), dtype=x.dtype, device=dev)
        h = torch.empty((t, inter), dtype=x.dtype, device=dev)
        y = torch.empty((t, hidden), dtype=x.dtype, device=dev)
        res2 = None
        if residual is not None:
            if residual.shape != x.shape or residual.dtype != x.dtype:
                raise ValueError("bastile_b200 MLP: residual must match the input's shape and dtype")
            res2 = _rows(residual)
        st = _lib.status_word(dev)
        with _lib.device_of(dev), _lib.timed("mlp_fwd", 2, dev):
            rc = lib.bt_mlp_fwd(x2.data_ptr(), wgc.data_ptr(), wuc.data_ptr(), wdc.data_ptr(), gate.data_ptr(),
                                up.data_ptr(), h.data_ptr(), y.data_ptr(), t, hidden, inter, _ld(x2),
                                res2.data_ptr() if res2 is not None else None,
                                _ld(res2) if res2 is not None else 0, code, st.data_ptr(),
                                _lib.stream_ptr(dev))
        _lib.check(rc, "bt_mlp_fwd")
        ctx.save_for_backward(x2, wgc, wuc, wdc, gate, up, h)
        ctx.x_shape = x.shape
        ctx.w_dtypes = (wg.dtype, wu.dtype, wd.dtype)
        return y.view(*x.shape[:-1], hidden)

    @staticmethod
    def backward(ctx, dy):
        x2, wg, wu, wd, gate, up, h = ctx.saved_tensors
        dev = x2.device
        lib = _lib.get_lib()
        t, hidden = x2.shape
        inter = wg.shape[0]
        if dy.dtype != x2.dtype:
            dy = dy.to(x2.dtype)
        dy2 = _rows(dy)
        need_x, need_g, need_u, need_d = ctx.needs_input_grad[:4]
        need_res = len(ctx.needs_input_grad) > 4 and ctx.needs_input_grad[4]
        # dgate | dup share one [T, 2I] buffer and dWg | dWu one [2I, H] buffer, so that the
        # library can compute both weight gradients as a single product
        dgu = torch.empty((t, 2 * inter), dtype=gate.dtype, device=dev)
        dgate, dup = dgu[:, :inter], dgu[:, inter:]
        dx = torch.empty_like(x2, memory_format=torch.contiguous_format) if need_x else None
        dwg = dwu = None
        # a gradient destination registered for a weight (a flat bucket of a data-parallel optimizer)
        # is written directly; dWg | dWu only when the two destinations are stacked like the result
        sink_g, sink_u, sink_d = (_lib.grad_sink(w, dt) if w.dtype == dt else None
                                  for w, dt in zip((wg, wu, wd), ctx.w_dtypes))
        if need_g and need_u:
            if (sink_g is not None and sink_u is not None
                    and sink_u.data_ptr() == sink_g.data_ptr() + sink_g.numel() * sink_g.element_size()):
                dwg, dwu = sink_g, sink_u
            else:
                dwgu = torch.empty((2 * inter, hidden), dtype=wg.dtype, device=dev)
                dwg, dwu = dwgu[:inter], dwgu[inter:]
        elif need_g:
            dwg = sink_g if sink_g is not None else torch.empty_like(wg)
        elif need_u:
            dwu = sink_u if sink_u is not None else torch.empty_like(wu)
        dwd = (sink_d if sink_d is not None else torch.empty_like(wd)) if need_d else None
        st = _lib.status_word(dev)

        def p(tensor):
            return tensor.data_ptr() if tensor is not None else None

        n_k = 1 + sum(t is not None for t in (dx, dwd)) + (1 if (dwg is not None and dwu is not None) else
                                                           int(dwg is not None) + int(dwu is not None))
        with _lib.device_of(dev), _lib.timed("mlp_bwd", n_k, dev):
            rc = lib.bt_mlp_bwd(dy2.data_ptr(), x2.data_ptr(), wg.data_ptr(), wu.data_ptr(), wd.data_ptr(),
                                gate.data_ptr(), up.data_ptr(), h.data_ptr(), dgate.data_ptr(), dup.data_ptr(),
                                p(dx), p(dwg), p(dwu), p(dwd), t, hidden, inter, _ld(x2), _ld(dy2), 2 * inter,
                                _lib.dtype_code(x2.dtype), st.data_ptr(), _lib.stream_ptr(dev))
        _lib.check(rc, "bt_mlp_bwd")
        dts = ctx.w_dtypes
        return (
            dx.view(ctx.x_shape) if dx is not None else None,
            dwg.to(dts[0]) if dwg is not None else None,
            dwu.to(dts[1]) if dwu is not None else None,
            dwd.to(dts[2]) if dwd is not None else None,
            dy if need_res else None,
        )


class B200SwiGLUMLP(nn.Module):
    """Drop-in for ``Qwen3MLP`` (swiglu.py:170-187): same constructor argument,
    same three bias-free ``nn.Linear`` parameters ``gate_proj / up_proj /
    down_proj``, ``ValueError`` for an activation other than silu/swish."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.hidden_size = config.hidden_size
        self.intermediate_size = config.intermediate_size
        self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.down_proj = nn.Linear(self.intermediate_size, self.hidden_size, bias=False)
        if hasattr(config, "hidden_act") and config.hidden_act not in ["silu", "swish"]:
            raise ValueError(f"Activation function {config.hidden_act} not supported.")

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``residual`` (not part of the reference's module): returns ``residual + mlp(x)``
        with the add folded into the down projection."""
        if torch.is_autocast_enabled() and x.is_cuda:
            x = x.to(torch.get_autocast_dtype("cuda"))
            if residual is not None:
                residual = residual.to(x.dtype)
        return SwiGLUMLPFunction.apply(x, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight,
                                       residual)


CuTileSwiGLUMLP = B200SwiGLUMLP


register_patch(
    name="swiglu_qwen3",
    description="sm_100a SwiGLU MLP for Qwen3 (gate+up tcgen05 GEMM with silu*mul epilogue, fused backward)",
    target_module="transformers.models.qwen3.modeling_qwen3",
    target_attr="Qwen3MLP",
    replacement=B200SwiGLUMLP,
    has_backward=True,
    priority=10,
    models=["qwen3"],
)
