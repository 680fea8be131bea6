"""Fusions across the op boundaries of a Qwen3 decoder layer (opt-in: ``apply(fused_layers=True)``).

The reference patches four ops and leaves what sits between them to torch: the two
``residual + hidden_states`` adds of ``Qwen3DecoderLayer.forward`` (transformers
modeling_qwen3.py:316-336), the gradient accumulation autograd runs where a residual branch and
a norm branch meet, and the q_norm / k_norm -> apply_rotary_pos_emb sequence of
``Qwen3Attention.forward`` (modeling_qwen3.py:256-261), where every head row makes three round
trips through HBM.  This module replaces those two ``forward`` methods so that

* ``residual + attention_output`` is computed inside the post-attention RMSNorm kernel
  (``bt_add_rmsnorm_fwd``), ``residual + mlp_output`` inside the down projection's epilogue
  (``bt_mlp_fwd`` with a residual), and both gradient merges inside the RMSNorm backward
  (``bt_add_rmsnorm_bwd``) - no stand-alone elementwise add is left in a layer;
* q_norm + RoPE and k_norm + RoPE are one kernel for both tensors (``bt_qk_norm_rope_fwd/_bwd``).

Parameters, module names and results are those of the unfused patched model: the fused kernels
round where the separate ones round (bit-identical for the norm + RoPE pair; the residual folded
into the down projection is added before the single rounding instead of after it).
"""

from __future__ import annotations

import ctypes
import inspect
import logging

import torch

from .. import _lib
from .rms_norm import B200RMSNorm, _as_rows
from .rope import _dense
from .swiglu import B200SwiGLUMLP

log = logging.getLogger(__name__)


def _ld(t2: torch.Tensor) -> int:
    return t2.stride(0) if t2.shape[0] > 1 else t2.shape[1]


class AddRMSNormFunction(torch.autograd.Function):
    """``stream = x + residual``; returns ``(rms_norm(stream) * weight, stream)``.

    With ``residual=None`` the stream is ``x`` itself (returned as a second output so that the
    gradient of whatever consumes it later comes back through this node).  Either way the
    backward adds the stream's gradient to the norm's input gradient inside the kernel."""

    @staticmethod
    def forward(ctx, x, residual, weight, eps):
        dev = _lib.require_cuda(x, weight)
        lib = _lib.get_lib()
        code = _lib.dtype_code(x.dtype)
        shape = x.shape
        n = shape[-1]
        if weight.numel() != n:
            raise ValueError(f"add_rms_norm: weight has {weight.numel()} elements, rows have {n}")
        x2 = _as_rows(x, n)
        m = x2.shape[0]
        w = weight.detach()
        if w.dtype != x.dtype:
            w = w.to(x.dtype)
        w = w.contiguous()
        y = torch.empty((m, n), dtype=x.dtype, device=dev)
        rstd = torch.empty((m,), dtype=torch.float32, device=dev)
        if residual is None:
            with _lib.device_of(dev), _lib.timed("rmsnorm_fwd", 1, dev):
                rc = lib.bt_rmsnorm_fwd(x2.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), m, n, _ld(x2), n,
                                        float(eps), code, _lib.stream_ptr(dev))
            _lib.check(rc, "bt_rmsnorm_fwd")
            stream2, stream = x2, x.view_as(x)
        else:
            if residual.shape != shape or residual.dtype != x.dtype:
                raise ValueError("add_rms_norm: residual must match x in shape and dtype")
            r2 = _as_rows(residual, n)
            stream2 = torch.empty((m, n), dtype=x.dtype, device=dev)
            with _lib.device_of(dev), _lib.timed("rmsnorm_fwd", 1, dev):
                rc = lib.bt_add_rmsnorm_fwd(x2.data_ptr(), r2.data_ptr(), w.data_ptr(), stream2.data_ptr(),
                                            y.data_ptr(), rstd.data_ptr(), m, n, _ld(x2), _ld(r2), n, n, float(eps),
                                            code, _lib.stream_ptr(dev))
            _lib.check(rc, "bt_add_rmsnorm_fwd")
            stream = stream2.view(shape)
        ctx.save_for_backward(stream2, w, rstd)
        ctx.set_materialize_grads(False)  # an unused output arrives as None, not as zeros
        ctx.shape = shape
        ctx.weight_dtype = weight.dtype
        ctx.has_residual = residual is not None
        return y.view(shape), stream

    @staticmethod
    def backward(ctx, dy, dstream):
        s2, w, rstd = ctx.saved_tensors
        dev = s2.device
        lib = _lib.get_lib()
        m, n = s2.shape
        code = _lib.dtype_code(s2.dtype)
        if dy is None:  # only the stream was used downstream
            return dstream, (dstream if ctx.has_residual else None), None, None
        if dy.dtype != s2.dtype:
            dy = dy.to(s2.dtype)
        dy2 = _as_rows(dy, n)
        dx = torch.empty((m, n), dtype=s2.dtype, device=dev)
        dw = torch.empty((n,), dtype=s2.dtype, device=dev)
        ws = _lib.zero_workspace(dev, int(lib.bt_rmsnorm_bwd_ws_bytes(n)))
        with _lib.device_of(dev), _lib.timed("rmsnorm_bwd", 1, dev):
            if dstream is None:
                rc = lib.bt_rmsnorm_bwd(dy2.data_ptr(), s2.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                        dw.data_ptr(), ws.data_ptr(), m, n, _ld(dy2), _ld(s2), n, code,
                                        _lib.stream_ptr(dev))
            else:
                if dstream.dtype != s2.dtype:
                    dstream = dstream.to(s2.dtype)
                ds2 = _as_rows(dstream, n)
                rc = lib.bt_add_rmsnorm_bwd(dy2.data_ptr(), s2.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                            ds2.data_ptr(), dx.data_ptr(), dw.data_ptr(), ws.data_ptr(), m, n,
                                            _ld(dy2), _ld(s2), _ld(ds2), n, code, _lib.stream_ptr(dev))
        _lib.check(rc, "bt_add_rmsnorm_bwd")
        if dw.dtype != ctx.weight_dtype:
            dw = dw.to(ctx.weight_dtype)
        dx = dx.view(ctx.shape)
        return dx, (dx if ctx.has_residual else None), dw, None


def add_rms_norm(x, residual, weight, eps=1e-6):
    """``(rms_norm(x + residual) * weight, x + residual)``; ``residual`` may be None."""
    return AddRMSNormFunction.apply(x, residual, weight, eps)


def _head_rows_supported(head_dim: int, dtype: torch.dtype) -> bool:
    return dtype in (torch.bfloat16, torch.float16, torch.float32) and head_dim * dtype.itemsize in (128, 256, 512)


def _cos_sin(cos, sin, dtype):
    if cos.shape != sin.shape or cos.stride() != sin.stride():
        sin = sin.expand_as(cos).contiguous()
        cos = cos.contiguous()
    if cos.dtype != dtype:
        cos, sin = cos.to(dtype), sin.to(dtype)
    if cos.stride(-1) != 1:
        cos, sin = cos.contiguous(), sin.contiguous()
    return cos, sin


class QKNormRoPEFunction(torch.autograd.Function):
    """Per-head RMSNorm then RoPE of ``q`` [B, T, Hq, D] and ``k`` [B, T, Hk, D] (the q / k
    projections viewed per head), one kernel launch for both; returns tensors of the same
    shapes (the caller transposes to [B, H, T, D] as HF attention does)."""

    @staticmethod
    def forward(ctx, q, k, wq, wk, cos, sin, eps_q, eps_k):
        dev = _lib.require_cuda(q, k, wq, wk, cos, sin)
        lib = _lib.get_lib()
        if q.dim() != 4 or k.dim() != 4:
            raise ValueError("qk_norm_rope: q and k must be [batch, seq, heads, head_dim]")
        b, t, hq, d = q.shape
        hk = k.shape[2]
        if k.shape[0] != b or k.shape[1] != t or k.shape[3] != d or k.dtype != q.dtype:
            raise ValueError(f"qk_norm_rope: q {tuple(q.shape)} and k {tuple(k.shape)} disagree")
        if wq.numel() != d or wk.numel() != d:
            raise ValueError(f"qk_norm_rope: norm weights must have head_dim = {d} elements")
        if cos.dim() != 3 or cos.shape[1] != t or cos.shape[-1] not in (d, d // 2) or cos.shape[0] not in (1, b):
            raise ValueError(f"qk_norm_rope: cos of shape {tuple(cos.shape)} does not fit q {tuple(q.shape)}")
        if q.stride(-1) != 1:
            q = q.contiguous()
        if k.stride(-1) != 1:
            k = k.contiguous()
        ws = [_weight(w, q.dtype) for w in (wq, wk)]
        cos, sin = _cos_sin(cos, sin, q.dtype)
        q_out = torch.empty((b, t, hq, d), dtype=q.dtype, device=dev)
        k_out = torch.empty((b, t, hk, d), dtype=q.dtype, device=dev)
        rstd_q = torch.empty((b * t * hq,), dtype=torch.float32, device=dev)
        rstd_k = torch.empty((b * t * hk,), dtype=torch.float32, device=dev)
        if q.numel() > 0 and k.numel() > 0:
            with _lib.device_of(dev), _lib.timed("rope_fwd", 1, dev):
                rc = lib.bt_qk_norm_rope_fwd(q.data_ptr(), k.data_ptr(), ws[0].data_ptr(), ws[1].data_ptr(),
                                             cos.data_ptr(), sin.data_ptr(), q_out.data_ptr(), k_out.data_ptr(),
                                             rstd_q.data_ptr(), rstd_k.data_ptr(), b, t, hq, hk, d,
                                             _lib.I64x3(*q.stride()[:3]), _lib.I64x3(*k.stride()[:3]),
                                             _lib.I64x3(*q_out.stride()[:3]), _lib.I64x3(*k_out.stride()[:3]),
                                             _lib.I64x2(cos.stride(0), cos.stride(1)), cos.shape[0], float(eps_q),
                                             float(eps_k), _lib.dtype_code(q.dtype), _lib.stream_ptr(dev))
            _lib.check(rc, "bt_qk_norm_rope_fwd")
        ctx.save_for_backward(q, k, ws[0], ws[1], rstd_q, rstd_k, cos, sin)
        ctx.w_dtypes = (wq.dtype, wk.dtype)
        ctx.layouts = ((tuple(q.shape), tuple(q.stride())), (tuple(k.shape), tuple(k.stride())))
        return q_out, k_out

    @staticmethod
    def backward(ctx, dq_out, dk_out):
        q, k, wq, wk, rstd_q, rstd_k, cos, sin = ctx.saved_tensors
        dev = q.device
        lib = _lib.get_lib()
        b, t, hq, d = q.shape
        hk = k.shape[2]

        def grad_in(g, like):
            if g is None:
                return torch.zeros_like(like, memory_format=torch.contiguous_format)
            if g.dtype != like.dtype:
                g = g.to(like.dtype)
            return g if g.stride(-1) == 1 else g.contiguous()

        def grad_out(layout, like):
            # in the memory layout of the input, so that the projection's backward can flatten it for free
            if _dense(layout):
                return torch.empty_strided(layout[0], layout[1], dtype=like.dtype, device=dev)
            return torch.empty(like.shape, dtype=like.dtype, device=dev)

        dq_out, dk_out = grad_in(dq_out, q), grad_in(dk_out, k)
        dq, dk = grad_out(ctx.layouts[0], q), grad_out(ctx.layouts[1], k)
        dwq = torch.empty((d,), dtype=q.dtype, device=dev)
        dwk = torch.empty((d,), dtype=q.dtype, device=dev)
        nbytes = (int(lib.bt_rmsnorm_bwd_ws_bytes(d)) + 255) // 256 * 256
        ws = _lib.zero_workspace(dev, 2 * nbytes)
        if q.numel() > 0 and k.numel() > 0:
            with _lib.device_of(dev), _lib.timed("rope_bwd", 1, dev):
                rc = lib.bt_qk_norm_rope_bwd(dq_out.data_ptr(), dk_out.data_ptr(), q.data_ptr(), k.data_ptr(),
                                             wq.data_ptr(), wk.data_ptr(), rstd_q.data_ptr(), rstd_k.data_ptr(),
                                             cos.data_ptr(), sin.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                             dwq.data_ptr(), dwk.data_ptr(), ws.data_ptr(), ws.data_ptr() + nbytes,
                                             b, t, hq, hk, d, _lib.I64x3(*dq_out.stride()[:3]),
                                             _lib.I64x3(*dk_out.stride()[:3]), _lib.I64x3(*q.stride()[:3]),
                                             _lib.I64x3(*k.stride()[:3]), _lib.I64x3(*dq.stride()[:3]),
                                             _lib.I64x3(*dk.stride()[:3]), _lib.I64x2(cos.stride(0), cos.stride(1)),
                                             cos.shape[0], _lib.dtype_code(q.dtype), _lib.stream_ptr(dev))
            _lib.check(rc, "bt_qk_norm_rope_bwd")
        else:
            dwq.zero_()
            dwk.zero_()
        return dq, dk, dwq.to(ctx.w_dtypes[0]), dwk.to(ctx.w_dtypes[1]), None, None, None, None


def qk_norm_rope(q, k, wq, wk, cos, sin, eps_q=1e-6, eps_k=1e-6):
    """(RoPE(rms_norm(q) * wq), RoPE(rms_norm(k) * wk)) for q [B, T, Hq, D], k [B, T, Hk, D] and
    cos/sin [1 or B, T, D]."""
    return QKNormRoPEFunction.apply(q, k, wq, wk, cos, sin, eps_q, eps_k)


# ------------------------------------------------------------------ projections on the tcgen05 GEMM
_GEMM_DTYPES = (torch.bfloat16, torch.float16, torch.float32)
# How the patched attention forward runs the q/k/v/o projections (install(projections=...)):
#   "off": nn.Linear;  "dx": nn.Linear's GEMMs for the outputs and the weight gradients, but the
#   shared input gradient dX = dQ Wq + dK Wk + dV Wv from two bt_gemm_ex launches (no accumulation
#   passes);  "all": every product of q/k/v/o_proj on bt_gemm_ex;  "qkv": the q, k and v
#   projections as ONE product each way (forward, input gradient, weight gradients: three launches
#   instead of nine GEMMs and two accumulation passes) wherever the three weights lie one after the
#   other in memory (stack_qkv_weights), o_proj on nn.Linear; layers whose weights are not stacked
#   run as in "off".
PROJECTION_MODES = ("off", "acc", "dx", "all", "qkv")
_projection_mode = "off"


def _gemm(a, b, out, m, n, k, a_kmajor, b_kmajor, *, a1=None, b1=None, k1=0, addend_t=None, label, dev):
    """out[m,n] = op(a) op(b) (+ op(a1) op(b1)) (+ addend_t) through bt_gemm_ex; 2-D row-major tensors."""
    lib = _lib.get_lib()
    d = _lib.GemmDesc()
    d.A, d.B, d.lda, d.ldb, d.K = a.data_ptr(), b.data_ptr(), _ld(a), _ld(b), k
    if a1 is not None:
        d.A1, d.B1, d.lda1, d.ldb1, d.K1 = a1.data_ptr(), b1.data_ptr(), _ld(a1), _ld(b1), k1
    d.D, d.ldd, d.M, d.N = out.data_ptr(), _ld(out), m, n
    d.a_kmajor, d.b_kmajor = int(a_kmajor), int(b_kmajor)
    d.in_dtype = _lib.dtype_code(a.dtype)
    d.out_dtype = _lib.dtype_code(out.dtype)
    if addend_t is not None:
        d.addend_t, d.ld_addend_t = addend_t.data_ptr(), _ld(addend_t)
    st = _lib.status_word(dev)
    with _lib.device_of(dev), _lib.timed(label, 1, dev):
        rc = lib.bt_gemm_ex(ctypes.byref(d), st.data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "bt_gemm_ex")


def _rows2d(t: torch.Tensor) -> torch.Tensor:
    """[..., n] -> [rows, n], unit inner stride, row stride a multiple of 8 elements (16-byte rows)."""
    n = t.shape[-1]
    t2 = t.reshape(-1, n)
    if t2.stride(-1) != 1 or (t2.shape[0] > 1 and (t2.stride(0) < n or t2.stride(0) % 8 != 0)):
        t2 = t2.contiguous()
    return t2


def _weight(w: torch.Tensor, dtype) -> torch.Tensor:
    w = w.detach()
    if w.dtype != dtype:
        w = w.to(dtype)
    return w.contiguous()


class SharedInputLinearFunction(torch.autograd.Function):
    """``tuple(x @ w.T for w in weights)`` for bias-free linear layers that share their input
    (the q / k / v projections; with one weight, a plain linear such as o_proj) on the tcgen05
    GEMM.  The backward forms ``dx = sum_i dy_i @ w_i`` inside the GEMMs - two products per
    launch accumulate in tensor memory, a third takes the running sum in as an addend - instead
    of one GEMM per layer plus the accumulation passes autograd would add."""

    @staticmethod
    def forward(ctx, dx_only, x, *weights):
        dev = _lib.require_cuda(x, *weights)
        if x.dtype not in _GEMM_DTYPES:
            raise TypeError(f"bastile_b200 linear: unsupported dtype {x.dtype}")
        k = x.shape[-1]
        x2 = _rows2d(x)
        m = x2.shape[0]
        ws = [_weight(w, x.dtype) for w in weights]
        outs = []
        for w in ws:
            if w.dim() != 2 or w.shape[1] != k:
                raise ValueError(f"bastile_b200 linear: weight {tuple(w.shape)} does not fit input [..., {k}]")
            if dx_only:
                y = torch.mm(x2, w.t())
            else:
                y = torch.empty((m, w.shape[0]), dtype=x.dtype, device=dev)
                if m > 0:
                    _gemm(x2, w, y, m, w.shape[0], k, True, True, label="proj_fwd", dev=dev)
            outs.append(y.view(*x.shape[:-1], w.shape[0]))
        ctx.dx_only = bool(dx_only)
        ctx.save_for_backward(x2, *ws)
        ctx.x_shape = x.shape
        ctx.w_dtypes = [w.dtype for w in weights]
        ctx.set_materialize_grads(False)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *dys):
        x2, *ws = ctx.saved_tensors
        dev = x2.device
        m, k = x2.shape
        live = [(i, _rows2d(dy.to(x2.dtype))) for i, dy in enumerate(dys) if dy is not None]
        dx = None
        if ctx.needs_input_grad[1] and live and m > 0:
            dx = torch.empty((m, k), dtype=x2.dtype, device=dev)
            todo = list(live)
            first = True
            while todo:
                # with an odd count, the first launch takes one product so that every later one
                # carries two and the running sum
                take = 1 if (first and len(todo) % 2 == 1) else 2
                pairs, todo = todo[:take], todo[take:]
                (i0, g0) = pairs[0]
                kw = {}
                if len(pairs) == 2:
                    i1, g1 = pairs[1]
                    kw = dict(a1=g1, b1=ws[i1], k1=ws[i1].shape[0])
                # dy_i [m, n_i] is K-major; w_i [n_i, k] is stored [K, N]: N-major
                _gemm(g0, ws[i0], dx, m, k, ws[i0].shape[0], True, False, addend_t=None if first else dx,
                      label="proj_bwd", dev=dev, **kw)
                first = False
            dx = dx.view(ctx.x_shape)
        elif ctx.needs_input_grad[1]:
            dx = torch.zeros(ctx.x_shape, dtype=x2.dtype, device=dev)
        dws = [None] * len(ws)
        for i, g in live:
            if ctx.needs_input_grad[2 + i]:
                n = ws[i].shape[0]
                if ctx.dx_only:
                    dws[i] = torch.mm(g.t(), x2).to(ctx.w_dtypes[i])
                    continue
                dw = torch.empty((n, k), dtype=x2.dtype, device=dev)
                if m > 0:
                    # dw = dy^T x: both operands stored [K = rows, ...]: M-major and N-major
                    _gemm(g, x2, dw, n, k, m, False, False, label="proj_bwd", dev=dev)
                else:
                    dw.zero_()
                dws[i] = dw.to(ctx.w_dtypes[i])
        return (None, dx, *dws)


class AccumulatedInputGradFunction(torch.autograd.Function):
    """``tuple(x @ w.T for w in weights)`` for bias-free linear layers that share their input,
    on the LIBRARY GEMMs exactly as ``nn.Linear`` runs them, with one difference in the backward:
    ``dx = sum_i dy_i @ w_i`` is accumulated by the GEMMs themselves (``addmm_``, beta = 1) instead
    of one result per layer plus the elementwise additions autograd would append - for q / k / v
    that is two passes over a [tokens, hidden] tensor less per layer.  Weight gradients go
    straight into a registered gradient destination when there is one."""

    @staticmethod
    def forward(ctx, x, *weights):
        _lib.require_cuda(x, *weights)
        x2 = _rows2d(x)
        ws = [_weight(w, x.dtype) for w in weights]
        outs = tuple(torch.mm(x2, w.t()).view(*x.shape[:-1], w.shape[0]) for w in ws)
        ctx.save_for_backward(x2, *ws)
        ctx.x_shape = x.shape
        ctx.w_dtypes = [w.dtype for w in weights]
        ctx.sinks = [w if w.dtype == x.dtype else None for w in weights]
        ctx.set_materialize_grads(False)
        return outs

    @staticmethod
    def backward(ctx, *dys):
        x2, *ws = ctx.saved_tensors
        live = [(i, _rows2d(dy.to(x2.dtype))) for i, dy in enumerate(dys) if dy is not None]
        dx = None
        if ctx.needs_input_grad[0]:
            for i, g in live:
                if dx is None:
                    dx = torch.mm(g, ws[i])
                else:
                    dx.addmm_(g, ws[i])
            dx = dx.view(ctx.x_shape) if dx is not None else torch.zeros(ctx.x_shape, dtype=x2.dtype, device=x2.device)
        dws = [None] * len(ws)
        for i, g in live:
            if ctx.needs_input_grad[1 + i]:
                sink = _lib.grad_sink(ctx.sinks[i], x2.dtype) if ctx.sinks[i] is not None else None
                if sink is not None:
                    dws[i] = torch.mm(g.t(), x2, out=sink)
                else:
                    dws[i] = torch.mm(g.t(), x2).to(ctx.w_dtypes[i])
        ctx.sinks = None
        return (dx, *dws)


def _stacked(wq, wk, wv) -> bool:
    """True when the three [n_i, k] weights lie one after the other in memory, in this order."""
    es = wq.element_size()
    return (wq.dtype == wk.dtype == wv.dtype and wq.is_contiguous() and wk.is_contiguous() and wv.is_contiguous()
            and wq.shape[1] == wk.shape[1] == wv.shape[1]
            and wk.data_ptr() == wq.data_ptr() + wq.numel() * es and wv.data_ptr() == wk.data_ptr() + wk.numel() * es)


@torch.no_grad()
def stack_qkv_weights(model) -> int:
    """Move ``q_proj.weight``, ``k_proj.weight`` and ``v_proj.weight`` of every attention block of
    ``model`` into one ``[nq + nk + nv, hidden]`` buffer per block (the parameters stay three
    separate ``nn.Parameter`` objects with unchanged names, shapes and values: only their storage
    moves).  ``apply(fused_layers=True, gemm_projections="qkv")`` then runs the three projections
    as one product each way.  Call it after the model is on its device and before the optimizer
    and any data-parallel wrapper are created; anything that re-allocates the parameters later
    (``model.to(...)``) undoes it, and the layers fall back to separate projections by themselves.
    Returns the number of blocks stacked."""
    done = 0
    for mod in model.modules():
        q, k, v = (getattr(mod, n, None) for n in ("q_proj", "k_proj", "v_proj"))
        if not all(_plain_linear(m) if m is not None else False for m in (q, k, v)):
            continue
        wq, wk, wv = q.weight, k.weight, v.weight
        if wq.dtype != wk.dtype or wq.dtype != wv.dtype or wq.shape[1] != wk.shape[1] or wq.shape[1] != wv.shape[1]:
            continue
        if not _stacked(wq.data, wk.data, wv.data):
            buf = torch.empty((wq.shape[0] + wk.shape[0] + wv.shape[0], wq.shape[1]), dtype=wq.dtype, device=wq.device)
            row = 0
            for w in (wq, wk, wv):
                view = buf[row:row + w.shape[0]]
                view.copy_(w.data)
                w.data = view
                row += w.shape[0]
        done += 1
    return done


class QKVProjectionFunction(torch.autograd.Function):
    """``(x @ wq.T, x @ wk.T, x @ wv.T)`` for three weights that are stacked in memory:
    forward = one product ``x [Wq; Wk; Wv]^T`` whose epilogue writes three dense results;
    ``dx = [dq | dk | dv] [Wq; Wk; Wv]`` = one product whose A operand is read from the three
    gradient tensors where they lie; ``[dWq; dWk; dWv] = [dq | dk | dv]^T x`` = one product into a
    stacked buffer of which the three weight gradients are views."""

    @staticmethod
    def forward(ctx, x, wq, wk, wv):
        dev = _lib.require_cuda(x, wq, wk, wv)
        lib = _lib.get_lib()
        k = x.shape[-1]
        x2 = _rows2d(x)
        m = x2.shape[0]
        ns = (wq.shape[0], wk.shape[0], wv.shape[0])
        w_all = torch.as_strided(wq.detach(), (sum(ns), k), (k, 1))  # the three weights as one matrix
        outs = [torch.empty((m, n), dtype=x.dtype, device=dev) for n in ns]
        if m > 0:
            d = _lib.GemmDesc()
            d.A, d.B, d.lda, d.ldb, d.K = x2.data_ptr(), w_all.data_ptr(), _ld(x2), k, k
            d.D, d.ldd, d.M, d.N = outs[0].data_ptr(), ns[0], m, sum(ns)
            d.a_kmajor, d.b_kmajor = 1, 1
            d.in_dtype = d.out_dtype = _lib.dtype_code(x.dtype)
            d.d_split, d.D1, d.D2, d.ldd1, d.ldd2, d.N0, d.N1 = 1, outs[1].data_ptr(), outs[2].data_ptr(), ns[1], ns[2], ns[0], ns[1]
            st = _lib.status_word(dev)
            with _lib.device_of(dev), _lib.timed("proj_fwd", 1, dev):
                rc = lib.bt_gemm_ex(ctypes.byref(d), st.data_ptr(), _lib.stream_ptr(dev))
            _lib.check(rc, "bt_gemm_ex(qkv)")
        ctx.save_for_backward(x2, w_all)
        ctx.ns = ns
        ctx.x_shape = x.shape
        ctx.set_materialize_grads(False)
        return tuple(o.view(*x.shape[:-1], n) for o, n in zip(outs, ns))

    @staticmethod
    def backward(ctx, dq, dk, dv):
        x2, w_all = ctx.saved_tensors
        dev = x2.device
        lib = _lib.get_lib()
        m, k = x2.shape
        ns = ctx.ns
        gs = []
        for g, n in zip((dq, dk, dv), ns):
            if g is None:
                g = torch.zeros((m, n), dtype=x2.dtype, device=dev)
            gs.append(_rows2d(g.to(x2.dtype)))
        code = _lib.dtype_code(x2.dtype)
        st = _lib.status_word(dev)
        dx = dw = None
        if m == 0:
            dx = torch.zeros(ctx.x_shape, dtype=x2.dtype, device=dev) if ctx.needs_input_grad[0] else None
            dws = [torch.zeros((n, k), dtype=x2.dtype, device=dev) for n in ns]
            return (dx, *dws)
        if ctx.needs_input_grad[0]:
            # dx[m, k] = [dq | dk | dv][m, sum ns] @ W_all[sum ns, k]: A in three pieces along the contraction
            dx = torch.empty((m, k), dtype=x2.dtype, device=dev)
            d = _lib.GemmDesc()
            d.A, d.lda, d.K = gs[0].data_ptr(), _ld(gs[0]), ns[0]
            d.A1, d.lda1, d.K1 = gs[1].data_ptr(), _ld(gs[1]), ns[1]
            d.A2, d.lda2, d.K2 = gs[2].data_ptr(), _ld(gs[2]), ns[2]
            d.a_split = 1
            d.B, d.ldb = w_all.data_ptr(), k
            d.D, d.ldd, d.M, d.N = dx.data_ptr(), k, m, k
            d.a_kmajor, d.b_kmajor = 1, 0
            d.in_dtype = d.out_dtype = code
            with _lib.device_of(dev), _lib.timed("proj_bwd", 1, dev):
                rc = lib.bt_gemm_ex(ctypes.byref(d), st.data_ptr(), _lib.stream_ptr(dev))
            _lib.check(rc, "bt_gemm_ex(qkv dx)")
            dx = dx.view(ctx.x_shape)
        if any(ctx.needs_input_grad[1:]):
            # [dWq; dWk; dWv][sum ns, k] = [dq | dk | dv]^T @ x: A in three pieces along M
            dw = torch.empty((sum(ns), k), dtype=x2.dtype, device=dev)
            d = _lib.GemmDesc()
            d.A, d.lda, d.K = gs[0].data_ptr(), _ld(gs[0]), m
            d.A1, d.lda1 = gs[1].data_ptr(), _ld(gs[1])
            d.A2, d.lda2 = gs[2].data_ptr(), _ld(gs[2])
            d.a_split, d.M0, d.M1 = 2, ns[0], ns[1]
            d.B, d.ldb = x2.data_ptr(), _ld(x2)
            d.D, d.ldd, d.M, d.N = dw.data_ptr(), k, sum(ns), k
            d.a_kmajor, d.b_kmajor = 0, 0
            d.in_dtype = d.out_dtype = code
            with _lib.device_of(dev), _lib.timed("proj_bwd", 1, dev):
                rc = lib.bt_gemm_ex(ctypes.byref(d), st.data_ptr(), _lib.stream_ptr(dev))
            _lib.check(rc, "bt_gemm_ex(qkv dW)")
        dws, row = [], 0
        for i, n in enumerate(ns):
            dws.append(dw[row:row + n] if (dw is not None and ctx.needs_input_grad[1 + i]) else None)
            row += n
        return (dx, *dws)


def _qkv_fusable(x, wq, wk, wv) -> bool:
    """One product for the three projections: stacked weights of the input's dtype, and segment
    sizes the kernel's tiles divide (256 result columns / rows, 64-element contraction blocks)."""
    return (x.is_cuda and x.dtype in _GEMM_DTYPES and wq.dtype == x.dtype and x.shape[-1] % 8 == 0
            and wq.shape[0] % 256 == 0 and wk.shape[0] % 256 == 0 and wv.shape[0] % 8 == 0
            and _stacked(wq, wk, wv))


def shared_input_linear(x, *weights, dx_only: bool = False):
    """``dx_only``: outputs and weight gradients from torch.mm, only the input gradient fused."""
    return SharedInputLinearFunction.apply(dx_only, x, *weights)


def _plain_linear(mod) -> bool:
    return type(mod) is torch.nn.Linear and mod.bias is None


# ------------------------------------------------------------------ the two patched forwards
def decoder_layer_forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_values=None,
                          use_cache=False, position_embeddings=None, **kwargs):
    """``Qwen3DecoderLayer.forward`` (modeling_qwen3.py:316-336) with the residual adds folded
    into the neighbouring kernels.  Falls back to separate adds around modules that are not the
    B200 ones (a model built before ``apply()``)."""
    norm_in, norm_post, mlp = self.input_layernorm, self.post_attention_layernorm, self.mlp
    fused_norms = isinstance(norm_in, B200RMSNorm) and isinstance(norm_post, B200RMSNorm)
    if fused_norms:
        normed, stream = add_rms_norm(hidden_states, None, norm_in.weight, norm_in.variance_epsilon)
    else:
        stream, normed = hidden_states, norm_in(hidden_states)
    attn_out, _ = self.self_attn(hidden_states=normed, attention_mask=attention_mask, position_ids=position_ids,
                                 past_key_values=past_key_values, use_cache=use_cache,
                                 position_embeddings=position_embeddings, **kwargs)
    if fused_norms:
        normed, stream = add_rms_norm(attn_out, stream, norm_post.weight, norm_post.variance_epsilon)
    else:
        stream = stream + attn_out
        normed = norm_post(stream)
    if isinstance(mlp, B200SwiGLUMLP):
        return mlp(normed, residual=stream)
    return stream + mlp(normed)


def attention_forward(self, hidden_states, position_embeddings, attention_mask, past_key_values=None, **kwargs):
    """``Qwen3Attention.forward`` (modeling_qwen3.py:243-288) with q_norm + RoPE and
    k_norm + RoPE as one kernel; everything from the cache update on is unchanged."""
    from transformers.models.qwen3 import modeling_qwen3 as hf

    lead = hidden_states.shape[:-1]
    cos, sin = position_embeddings
    plain = all(_plain_linear(m) for m in (self.q_proj, self.k_proj, self.v_proj, self.o_proj))
    on_gemm = (_projection_mode in ("dx", "all") and hidden_states.is_cuda and hidden_states.dtype in _GEMM_DTYPES
               and hidden_states.shape[-1] % 8 == 0 and self.head_dim % 8 == 0 and plain)
    if (_projection_mode == "qkv" and plain
            and _qkv_fusable(hidden_states, self.q_proj.weight, self.k_proj.weight, self.v_proj.weight)):
        q_lin, k_lin, v_lin = QKVProjectionFunction.apply(hidden_states, self.q_proj.weight, self.k_proj.weight,
                                                          self.v_proj.weight)
    elif (_projection_mode == "acc" and plain and hidden_states.is_cuda and torch.is_grad_enabled()
          and not torch.is_autocast_enabled()):
        q_lin, k_lin, v_lin = AccumulatedInputGradFunction.apply(hidden_states, self.q_proj.weight,
                                                                 self.k_proj.weight, self.v_proj.weight)
    elif on_gemm:
        q_lin, k_lin, v_lin = shared_input_linear(hidden_states, self.q_proj.weight, self.k_proj.weight,
                                                  self.v_proj.weight, dx_only=_projection_mode == "dx")
    else:
        q_lin, k_lin, v_lin = self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)
    q_lin = q_lin.view(*lead, -1, self.head_dim)
    k_lin = k_lin.view(*lead, -1, self.head_dim)
    value = v_lin.view(*lead, -1, self.head_dim).transpose(1, 2)
    fusable = (q_lin.dim() == 4 and q_lin.is_cuda and isinstance(self.q_norm, B200RMSNorm)
               and isinstance(self.k_norm, B200RMSNorm) and _head_rows_supported(self.head_dim, q_lin.dtype)
               and cos.dim() == 3)
    if fusable:
        query, key = qk_norm_rope(q_lin, k_lin, self.q_norm.weight, self.k_norm.weight, cos, sin,
                                  self.q_norm.variance_epsilon, self.k_norm.variance_epsilon)
        query, key = query.transpose(1, 2), key.transpose(1, 2)
    else:
        query, key = hf.apply_rotary_pos_emb(self.q_norm(q_lin).transpose(1, 2), self.k_norm(k_lin).transpose(1, 2),
                                             cos, sin)
    if past_key_values is not None:
        key, value = past_key_values.update(key, value, self.layer_idx)
    attend = hf.ALL_ATTENTION_FUNCTIONS.get_interface(self.config._attn_implementation, hf.eager_attention_forward)
    out, weights = attend(self, query, key, value, attention_mask,
                          dropout=0.0 if not self.training else self.attention_dropout, scaling=self.scaling,
                          sliding_window=self.sliding_window, **kwargs)
    out = out.reshape(*lead, -1).contiguous()
    if on_gemm and _projection_mode == "all":
        return shared_input_linear(out, self.o_proj.weight)[0], weights
    if (_projection_mode == "acc" and plain and out.is_cuda and torch.is_grad_enabled()
            and not torch.is_autocast_enabled() and _lib.grad_sink(self.o_proj.weight, out.dtype) is not None):
        # same library products; the weight gradient lands in its registered destination uncopied
        return AccumulatedInputGradFunction.apply(out, self.o_proj.weight)[0], weights
    return self.o_proj(out), weights


# Parameters the installed transformers must give the two methods for the replacements to be
# drop-in; anything else and the fused forwards are not installed.
_EXPECTED_PARAMS = {
    "Qwen3DecoderLayer": ("self", "hidden_states", "attention_mask", "position_ids", "past_key_values", "use_cache",
                          "position_embeddings", "kwargs"),
    "Qwen3Attention": ("self", "hidden_states", "position_embeddings", "attention_mask", "past_key_values", "kwargs"),
}
_REPLACEMENTS = {"Qwen3DecoderLayer": decoder_layer_forward, "Qwen3Attention": attention_forward}
PATCH_NAMES = {"Qwen3DecoderLayer": "decoder_layer_qwen3", "Qwen3Attention": "attention_qwen3"}
_originals: dict[str, object] = {}


def install(hf_module, decoder_layer: bool = True, attention: bool = True, projections: str = "off") -> list[str]:
    """Replace the two ``forward`` methods on the classes of ``hf_module``; returns the names installed.
    ``projections`` is one of PROJECTION_MODES."""
    global _projection_mode
    if projections not in PROJECTION_MODES:
        raise ValueError(f"projections must be one of {PROJECTION_MODES}, got {projections!r}")
    _projection_mode = projections
    done = []
    for cls_name, wanted in (("Qwen3DecoderLayer", decoder_layer), ("Qwen3Attention", attention)):
        if not wanted:
            continue
        cls = getattr(hf_module, cls_name, None)
        if cls is None:
            log.warning("fused layers: %s not found", cls_name)
            continue
        current = cls.forward
        if current is _REPLACEMENTS[cls_name]:
            done.append(PATCH_NAMES[cls_name])
            continue
        params = tuple(inspect.signature(inspect.unwrap(current)).parameters)
        if params != _EXPECTED_PARAMS[cls_name]:
            log.warning("fused layers: %s.forward has parameters %s, expected %s - left alone", cls_name, params,
                        _EXPECTED_PARAMS[cls_name])
            continue
        _originals[cls_name] = current
        cls.forward = _REPLACEMENTS[cls_name]
        done.append(PATCH_NAMES[cls_name])
    return done


def uninstall(hf_module, names=None) -> list[str]:
    """Put the original ``forward`` methods back (all, or those whose patch name is in ``names``)."""
    done = []
    for cls_name, original in list(_originals.items()):
        if names is not None and PATCH_NAMES[cls_name] not in names:
            continue
        cls = getattr(hf_module, cls_name, None)
        if cls is not None:
            cls.forward = original
            done.append(PATCH_NAMES[cls_name])
        del _originals[cls_name]
    return done


def installed() -> list[str]:
    return [PATCH_NAMES[c] for c in _originals]
