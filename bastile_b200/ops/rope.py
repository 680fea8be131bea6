"""Rotary position embedding on the sm_100a kernel (replaces src/bastile/ops/rope.py).

Forward rotates ``q`` and ``k`` in place and returns them, like the reference
(rope.py:93-130); strides are passed to the kernel, so the transposed
``[B, H, T, D]`` views that ``Qwen3Attention`` hands over need no copy.  The
backward is the same kernel with ``sin`` negated inside the kernel, reading the
incoming gradients with their own strides and writing fresh tensors - no
``-sin`` tensor and no ``.contiguous()`` copies (rope.py:132-136 made both).
Only the first ``D/2`` columns of ``cos``/``sin`` are read (rope.py:100-105).

Like the reference, the forward does NOT call ``ctx.mark_dirty(q, k)``.  It cannot: HF hands
over transposed VIEWS (``q_norm(...).transpose(1, 2)``), and torch refuses a Function that
modifies a view input in place and returns more than one tensor ("your Function cannot return
more than one Tensor"; tests/test_patch_engine.py keeps a stand-in of that shape to notice if
torch ever lifts the rule).  The consequence is the reference's: whatever produced ``q`` / ``k``
must not need its own OUTPUT in its backward - true for ``Qwen3RMSNorm`` here and there, which
saves its input.  ``apply(fused_layers=True)`` replaces the pair q/k-norm + RoPE by one
out-of-place kernel and has no such caveat.
"""

from __future__ import annotations

import torch

from .. import _lib
from ..registry import register_patch


def _strides3(t: torch.Tensor):
    return _lib.I64x3(t.stride(0), t.stride(1), t.stride(2))


def _launch(q_in, k_in, q_out, k_out, cos, sin, negate: bool) -> None:
    dev = _lib.require_cuda(q_in, k_in, q_out, k_out, cos, sin)
    lib = _lib.get_lib()
    b, hq, t, d = q_in.shape
    hk = k_in.shape[1]
    if k_in.shape[0] != b or k_in.shape[2] != t or k_in.shape[3] != d:
        raise ValueError(f"rope: q {tuple(q_in.shape)} and k {tuple(k_in.shape)} disagree")
    if cos.dim() != 3 or cos.shape[1] != t or cos.shape[-1] not in (d, d // 2):
        raise ValueError(f"rope: cos of shape {tuple(cos.shape)} does not fit q {tuple(q_in.shape)}")
    if cos.shape != sin.shape or cos.stride() != sin.stride():
        sin = sin.expand_as(cos).contiguous()
        cos = cos.contiguous()
    if cos.dtype != q_in.dtype:
        cos, sin = cos.to(q_in.dtype), sin.to(q_in.dtype)
    if cos.stride(-1) != 1:
        cos, sin = cos.contiguous(), sin.contiguous()
    code = _lib.dtype_code(q_in.dtype)
    with _lib.device_of(dev), _lib.timed("rope_bwd" if negate else "rope_fwd", 1, dev):
        rc = lib.bt_rope(q_in.data_ptr(), k_in.data_ptr(), q_out.data_ptr(), k_out.data_ptr(), cos.data_ptr(),
                         sin.data_ptr(), b, hq, hk, t, d, _strides3(q_in), _strides3(k_in), _strides3(q_out),
                         _strides3(k_out), _lib.I64x2(cos.stride(0), cos.stride(1)), cos.shape[0],
                         1 if negate else 0, code, _lib.stream_ptr(dev))
    _lib.check(rc, "bt_rope")


def _dense(layout) -> bool:
    """True when (shape, strides) is a permutation of a contiguous tensor (no gaps, no overlap)."""
    shape, strides = layout
    expect = 1
    for size, stride in sorted(zip(shape, strides), key=lambda p: p[1]):
        if size == 1:
            continue
        if stride != expect:
            return False
        expect *= size
    return True


class RoPEFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
        if q.dim() != 4 or k.dim() != 4:
            raise ValueError("rope: q and k must be [batch, heads, seq, head_dim]")
        if k.dtype != q.dtype:
            raise TypeError("rope: q and k must share a dtype")
        # The kernel needs unit stride along head_dim; anything else is rotated
        # into a fresh contiguous tensor instead of in place.
        q_dst = q if q.stride(-1) == 1 else torch.empty_like(q, memory_format=torch.contiguous_format)
        k_dst = k if k.stride(-1) == 1 else torch.empty_like(k, memory_format=torch.contiguous_format)
        q_src = q if q.stride(-1) == 1 else q.contiguous()
        k_src = k if k.stride(-1) == 1 else k.contiguous()
        _launch(q_src, k_src, q_dst, k_dst, cos, sin, negate=False)
        ctx.save_for_backward(cos, sin)
        # the gradients are handed back in the memory layout of the inputs, so that whatever
        # produced q / k (a transposed view of [B, T, H, D] storage in HF attention) gets a
        # gradient it can flatten without a copy
        ctx.q_layout = (tuple(q.shape), tuple(q.stride())) if q.stride(-1) == 1 else None
        ctx.k_layout = (tuple(k.shape), tuple(k.stride())) if k.stride(-1) == 1 else None
        return q_dst.view(q_dst.shape), k_dst.view(k_dst.shape)

    @staticmethod
    def backward(ctx, dq, dk):
        cos, sin = ctx.saved_tensors
        if dq.stride(-1) != 1:
            dq = dq.contiguous()
        if dk.stride(-1) != 1:
            dk = dk.contiguous()
        def like_input(grad, layout):
            if layout is not None and _dense(layout):
                return torch.empty_strided(layout[0], layout[1], dtype=grad.dtype, device=grad.device)
            return torch.empty(grad.shape, dtype=grad.dtype, device=grad.device)

        dq_out = like_input(dq, ctx.q_layout)
        dk_out = like_input(dk, ctx.k_layout)
        _launch(dq, dk, dq_out, dk_out, cos, sin, negate=True)
        return dq_out, dk_out, None, None, None, None


def apply_rotary_pos_emb(q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
    """HF-compatible signature; ``position_ids`` / ``unsqueeze_dim`` are accepted
    and ignored, the layout is ``[B, H, T, D]`` (rope.py:139-141)."""
    return RoPEFunction.apply(q, k, cos, sin, position_ids, unsqueeze_dim)


register_patch(
    name="rope_qwen3",
    description="sm_100a in-place RoPE for Qwen3 (strided q/k, sin negated in-kernel for backward)",
    target_module="transformers.models.qwen3.modeling_qwen3",
    target_attr="apply_rotary_pos_emb",
    replacement=apply_rotary_pos_emb,
    has_backward=True,
    priority=10,
    models=["qwen3"],
)
