"""Fused lm_head + cross-entropy on sm_100a
(replaces src/bastile/ops/fused_linear_cross_entropy.py).

Per chunk of ``chunk_size`` rows the work is the reference's (``_chunked_fwd``,
:136-187): logits GEMM, softmax statistics, ``dlogits``, the ``dx`` GEMM and the
``dW`` GEMM, with the gradients produced during the forward and only scaled by
the incoming ``dloss`` in the backward (:371-399).  What changes is where the
arithmetic runs:

* the logits GEMM is a tcgen05 kernel whose epilogue produces the per-row
  (max, sum-exp) of each 256-column tile and picks up the target logit while the
  accumulator is still in tensor memory, and writes the chunk of logits once;
* one streaming pass turns that chunk into scaled ``dlogits`` in place (loss,
  ``-1`` at the label, zeroed ignored rows, ``1/n_valid``) - the reference needs
  two reads and a write plus torch indexing kernels with host syncs (:103-130);
* ``n_valid`` is counted on the device, so nothing in the forward or backward
  waits for the host (the reference calls ``.item()`` at :338 and :394);
* the ``dW`` accumulation across chunks happens in the fp32 epilogue of the
  GEMM, and the last chunk's GEMM in the backward applies ``dloss`` and writes
  the weight dtype directly.

With ``vocab_parallel_group`` every rank holds a slice ``[vocab_start,
vocab_start + V_local)`` of the lm_head rows and sees all rows of ``hidden``;
the only exchanges are one all-gather of the packed per-row statistics per
chunk and one all-reduce of ``d hidden``; ``dW`` stays local.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import Tensor

from .. import _lib

# fp32 tensors are fed to the tensor cores as tf32 (10-bit mantissa products, fp32 accumulation)
_GEMM_DTYPES = (torch.bfloat16, torch.float16, torch.float32)

# With the default chunk_size the op may work on up to this many rows at a time as long as
# the 16-bit logits chunk stays under AUTO_CHUNK_BYTES: 8192 rows x 4096 hidden is a whole
# number of waves of tiles for the dx GEMM, and fewer chunks mean fewer read-modify-write
# passes over the fp32 dW accumulator.  Larger is not better: with 16384 rows per chunk (no
# accumulator at all at 16384 x 151936) the call measured 50.8-51.5 ms against 49.8-50.0 ms on
# one B200 (4096 rows: 50.1-50.9 ms) - the operand panel that a group of row tiles shares in the
# dW product grows with the chunk and stops fitting the 126 MB L2.  An explicit chunk_size is
# obeyed.
DEFAULT_CHUNK = 4096
AUTO_CHUNK_ROWS = 8192
AUTO_CHUNK_BYTES = 3 << 30
# a [B, T', H] input that cannot be flattened without a copy is processed batch entry by batch entry
# when T' is at least this (shorter entries are copied once instead: many small launches cost more)
_SEGMENT_MIN_ROWS = 1024


def merge_shard_stats(gathered: Tensor) -> Tensor:
    """[n_shards, rows, 3] (max, sum-exp, target logit) -> [rows, 3] for the full vocabulary.
    The op itself runs this merge as one kernel (``bt_lce_stats_combine``); this torch form is the
    same arithmetic for CPU ranks and tests."""
    mx = gathered[..., 0]
    gmax = mx.max(dim=0).values
    gsum = (gathered[..., 1] * torch.exp(mx - gmax)).sum(dim=0)
    tgt = gathered[..., 2].sum(dim=0)
    return torch.stack((gmax, gsum, tgt), dim=-1).contiguous()


class LinearCrossEntropyFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, target, ignore_index, reduction, chunk_size, v_chunk_size,
                group=None, vocab_start=0, shard_tokens=False, grad_hidden_scale=1.0, vocab_size=None):
        dev = _lib.require_cuda(x, weight, target)
        lib = _lib.get_lib()
        if x.dtype not in _GEMM_DTYPES:
            raise TypeError(
                f"bastile_b200 fused_linear_cross_entropy: unsupported hidden-state dtype {x.dtype}"
            )
        if reduction not in ("mean", "sum"):
            raise ValueError(f"reduction must be 'mean' or 'sum', got {reduction!r}")
        code = _lib.dtype_code(x.dtype)
        batch_shape = x.shape[:-1]
        hdim = x.shape[-1]
        # The rows as a list of 2-D views with a uniform row stride.  A [B, T', H] slice of a larger
        # [B, T, H] tensor (hidden_states[:, :-1]) cannot be flattened without a copy, but each
        # batch entry by itself can be handed to the GEMMs with its row stride: no copy when the
        # entries are long enough to make chunks of their own.
        if (x.dim() == 3 and x.shape[0] > 1 and x.shape[1] >= _SEGMENT_MIN_ROWS and x.stride(-1) == 1
                and x.stride(1) % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(0) != x.shape[1] * x.stride(1)
                and not (group is not None and shard_tokens)):
            segments = [x[b] for b in range(x.shape[0])]
        else:
            xf = x.reshape(-1, hdim)
            if xf.stride(-1) != 1 or (xf.shape[0] > 1 and xf.stride(0) % 8 != 0):
                xf = xf.contiguous()
            segments = [xf]
        bt_local = sum(seg.shape[0] for seg in segments)
        if group is not None and shard_tokens:
            # every rank brought its own rows: assemble all rows of all ranks (same count each)
            xf = segments[0]
            world_sz = dist.get_world_size(group)
            x_all = torch.empty((world_sz * bt_local, hdim), dtype=x.dtype, device=dev)
            dist.all_gather_into_tensor(x_all, xf.contiguous(), group=group)
            t_local = target.reshape(-1).to(torch.int64).contiguous()
            t_all = torch.empty(world_sz * bt_local, dtype=torch.int64, device=dev)
            dist.all_gather_into_tensor(t_all, t_local, group=group)
            segments, target = [x_all], t_all
        bt = sum(seg.shape[0] for seg in segments)
        w = weight.detach()
        if w.dtype != x.dtype:
            w = w.to(x.dtype)
        w = w.contiguous()
        vloc = w.shape[0]
        if w.shape[1] != hdim:
            raise ValueError("fused_linear_cross_entropy: weight must be [vocab, hidden]")
        labels = target.reshape(-1)
        if labels.dtype != torch.int64:
            labels = labels.to(torch.int64)
        labels = labels.contiguous()
        if labels.numel() != bt:
            raise ValueError("fused_linear_cross_entropy: target does not match hidden_states")

        ld_logits = (vloc + 7) // 8 * 8
        rows_wanted = int(chunk_size)
        if rows_wanted == DEFAULT_CHUNK and AUTO_CHUNK_ROWS * ld_logits * 2 <= AUTO_CHUNK_BYTES:
            rows_wanted = AUTO_CHUNK_ROWS
        chunk = max(1, min(rows_wanted, max(seg.shape[0] for seg in segments))) if bt > 0 else 1
        # (view of the rows, first global row) per chunk; chunks never straddle two segments
        chunks, first = [], 0
        for seg in segments:
            for s0 in range(0, seg.shape[0], chunk):
                chunks.append((seg[s0:s0 + chunk], first + s0))
            first += seg.shape[0]
        n_chunks = len(chunks) if bt > 0 else 0
        n_vt = int(lib.bt_lce_num_vtiles(vloc))
        stream = _lib.stream_ptr(dev)
        st = _lib.status_word(dev)
        f32 = dict(dtype=torch.float32, device=dev)

        scal = torch.empty(3, **f32)  # n_valid, grad_scale, loss
        loss_row = torch.empty(max(bt, 1), **f32)
        logits_buf = torch.empty((chunk, ld_logits), dtype=x.dtype, device=dev)
        tile_stats = torch.empty((chunk, n_vt, 2), **f32)
        tgt_logit = torch.empty(chunk, **f32)
        row_stats = torch.empty((chunk, 3), **f32)
        dx_dtype = torch.float32 if group is not None else x.dtype
        dx = torch.empty((bt, hdim), dtype=dx_dtype, device=dev)
        dw_acc = torch.empty((vloc, hdim), **f32) if n_chunks > 1 else None
        world = 1
        if group is not None:
            world = dist.get_world_size(group)
            gathered = torch.empty((world, chunk, 3), **f32)
            merged = torch.empty((chunk, 3), **f32)

        # d(hidden) is a sum over the vocabulary shards.  Each chunk's rows are reduced as soon as its dx
        # GEMM is queued - NCCL runs that on its own stream underneath the next chunk's GEMMs - so only
        # the last chunk's reduction is exposed: an all-reduce per chunk when every rank needs all rows,
        # a reduce to the owning rank when the ranks brought their own rows and the chunk lies inside one
        # rank's block (otherwise one reduce-scatter at the end).
        reductions = []
        per_chunk_reduce = group is not None and bt > 0 and (
            not shard_tokens or all(s0 // bt_local == (s0 + xc0.shape[0] - 1) // bt_local for xc0, s0 in chunks))
        n_k = 2 + 5 * n_chunks - (1 if n_chunks else 0)
        with _lib.device_of(dev), _lib.timed("lce_fwd", n_k, dev):
            v_total = vloc if group is None else int(vocab_size or 0)  # 0: bound unknown, labels unchecked
            _lib.check(lib.bt_lce_count_valid(labels.data_ptr(), bt, ignore_index, 1 if reduction == "mean" else 0,
                                              scal[0:].data_ptr(), scal[1:].data_ptr(), v_total, st.data_ptr(),
                                              stream), "bt_lce_count_valid")
            last_rows = 0
            x_last = None
            ld_last = hdim
            for i in range(n_chunks):
                xc, s = chunks[i]
                rows = xc.shape[0]
                ld_xc = xc.stride(0) if rows > 1 else hdim
                lc = labels[s:s + rows]
                _lib.check(lib.bt_lce_logits_stats(xc.data_ptr(), w.data_ptr(), lc.data_ptr(), logits_buf.data_ptr(),
                                                   tile_stats.data_ptr(), tgt_logit.data_ptr(), rows, hdim, vloc,
                                                   ld_xc, ld_logits, int(vocab_start),
                                                   ignore_index, code, st.data_ptr(), stream),
                           "bt_lce_logits_stats")
                _lib.check(lib.bt_lce_row_stats(tile_stats.data_ptr(), tgt_logit.data_ptr(), row_stats.data_ptr(),
                                                rows, n_vt, stream), "bt_lce_row_stats")
                stats = row_stats
                if group is not None:
                    dist.all_gather_into_tensor(gathered.view(-1), row_stats.view(-1), group=group)
                    stats = merged
                    _lib.check(lib.bt_lce_stats_combine(gathered.data_ptr(), merged.data_ptr(), rows, chunk * 3, world,
                                                        stream), "bt_lce_stats_combine")
                _lib.check(lib.bt_lce_dlogits(logits_buf.data_ptr(), stats.data_ptr(), lc.data_ptr(),
                                              loss_row[s:].data_ptr(), scal[1:].data_ptr(), rows, vloc, ld_logits,
                                              int(vocab_start), ignore_index, 1, code, stream), "bt_lce_dlogits")
                # dx_chunk = dlogits[rows, V] @ W[V, H]
                _lib.check(lib.bt_gemm(logits_buf.data_ptr(), w.data_ptr(), dx[s:].data_ptr(), rows, hdim, vloc,
                                       ld_logits, hdim, hdim, 1, 0, code, _lib.dtype_code(dx_dtype), None, 0, None,
                                       st.data_ptr(), stream), "bt_gemm(dx)")
                if per_chunk_reduce:
                    if shard_tokens:
                        owner = dist.get_global_rank(group, s // bt_local)
                        reductions.append(dist.reduce(dx[s:s + rows], dst=owner, group=group, async_op=True))
                    else:
                        reductions.append(dist.all_reduce(dx[s:s + rows], group=group, async_op=True))
                if i < n_chunks - 1:
                    # dW += dlogits^T[V, rows] @ x_chunk[rows, H], fp32 accumulation across chunks
                    _lib.check(lib.bt_gemm(logits_buf.data_ptr(), xc.data_ptr(), dw_acc.data_ptr(), vloc, hdim, rows,
                                           ld_logits, ld_xc, hdim, 0, 0, code,
                                           _lib.BT_FP32, dw_acc.data_ptr() if i > 0 else None, hdim, None,
                                           st.data_ptr(), stream), "bt_gemm(dW)")
                else:
                    last_rows, x_last, ld_last = rows, xc, ld_xc
            _lib.check(lib.bt_lce_reduce_loss(loss_row.data_ptr(), bt, scal[1:].data_ptr() if reduction == "mean"
                                              else None, scal[2:].data_ptr(), stream), "bt_lce_reduce_loss")
        if group is not None and bt > 0:
            for work in reductions:
                work.wait()  # the current stream waits; the host does not
            if shard_tokens:  # each rank only needs the gradient of its own rows
                if per_chunk_reduce:
                    me = dist.get_rank(group)
                    dx = dx[me * bt_local:(me + 1) * bt_local]
                else:
                    dx_local = torch.empty((bt_local, hdim), dtype=dx.dtype, device=dev)
                    dist.reduce_scatter_tensor(dx_local, dx, group=group)
                    dx = dx_local
                batch_shape = x.shape[:-1]
            elif not per_chunk_reduce:
                dist.all_reduce(dx, group=group)

        ctx.save_for_backward(dx, w, logits_buf, x_last if x_last is not None else segments[0][:0],
                              dw_acc if dw_acc is not None else scal[:0])
        ctx.meta = (batch_shape, hdim, vloc, last_rows, ld_logits, x.dtype, weight.dtype, n_chunks, ld_last)
        ctx.grad_hidden_scale = float(grad_hidden_scale)
        return scal[2].clone()

    @staticmethod
    def backward(ctx, dloss):
        dx, w, dlogits_last, x_last, dw_acc = ctx.saved_tensors
        batch_shape, hdim, vloc, last_rows, ld_logits, x_dtype, w_dtype, n_chunks, ld_x = ctx.meta
        dev = dx.device
        lib = _lib.get_lib()
        stream = _lib.stream_ptr(dev)
        st = _lib.status_word(dev)
        code = _lib.dtype_code(x_dtype)
        scale = dloss.detach().to(torch.float32).reshape(1).contiguous()
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dx_out = dw_out = None
        with _lib.device_of(dev), _lib.timed("lce_bwd", int(need_x) + int(need_w and n_chunks > 0), dev):
            if need_x:
                dx_out = torch.empty(dx.shape, dtype=x_dtype, device=dev)
                scale_x = scale if ctx.grad_hidden_scale == 1.0 else scale * ctx.grad_hidden_scale
                _lib.check(lib.bt_scale_cast(dx.data_ptr(), dx_out.data_ptr(), dx.numel(), scale_x.data_ptr(),
                                             _lib.dtype_code(dx.dtype), code, stream), "bt_scale_cast(dx)")
                dx_out = dx_out.view(*batch_shape, hdim)
            if need_w:
                out_dtype = w_dtype if w_dtype in _lib._DTYPES else x_dtype
                # straight into a registered gradient bucket of the weight, if there is one
                dw_out = _lib.grad_sink(w, out_dtype) if w.dtype == w_dtype else None
                if dw_out is None:
                    dw_out = torch.empty((vloc, hdim), dtype=out_dtype, device=dev)
                if n_chunks == 0:
                    dw_out.zero_()
                else:
                    _lib.check(lib.bt_gemm(dlogits_last.data_ptr(), x_last.data_ptr(), dw_out.data_ptr(), vloc, hdim,
                                           last_rows, ld_logits, ld_x, hdim, 0, 0, code, _lib.dtype_code(out_dtype),
                                           dw_acc.data_ptr() if n_chunks > 1 else None, hdim, scale.data_ptr(),
                                           st.data_ptr(), stream), "bt_gemm(dW last)")
                if dw_out.dtype != w_dtype:
                    dw_out = dw_out.to(w_dtype)
        return dx_out, dw_out, None, None, None, None, None, None, None, None, None, None


ChunkedLinearCrossEntropyFunction = LinearCrossEntropyFunction


def fused_linear_cross_entropy(hidden_states: Tensor, weight: Tensor, target: Tensor, bias=None,
                               ignore_index: int = -100, chunk_size: int = 4096, reduction: str = "mean",
                               v_chunk_size: int | None = None, vocab_parallel_group=None,
                               vocab_start: int = 0, shard_tokens: bool = False,
                               grad_hidden_scale: float = 1.0, vocab_size: int | None = None) -> Tensor:
    """Loss of ``cross_entropy(hidden_states @ weight.T, target)`` without ever holding
    ``[tokens, vocab]`` logits; same arguments as the reference (:405-438).

    ``v_chunk_size`` is accepted for compatibility: the kernels already tile the
    vocabulary, so it selects nothing.  ``vocab_parallel_group`` / ``vocab_start``
    are additions for the vocabulary-sharded form (``weight`` is then the local
    slice of rows starting at ``vocab_start``; ``target`` holds global ids).  By default
    every rank passes the SAME ``hidden_states``; with ``shard_tokens=True`` every rank passes
    its own rows (equal counts), the op all-gathers them, the loss is the mean over all ranks'
    tokens, and each rank gets the gradient of its own rows back (reduce-scatter), multiplied
    by ``grad_hidden_scale`` (set it to the world size under data-parallel wrappers that
    average gradients over ranks).

    A label that is neither ``ignore_index`` nor a vocabulary row (``F.cross_entropy``, which the
    reference calls at :127 and :427, asserts on it) does not stop the call - nothing here waits
    for the device - but sets ``BT_STATUS_BAD_LABEL`` in the stream's status word, which
    ``bastile_b200._lib.check_all_status()`` turns into an exception.  With a vocabulary-parallel
    group pass ``vocab_size`` (rows of the full ``lm_head``) to have labels checked.
    """
    if bias is not None:
        if hidden_states.ndim == 3:
            hidden_states = hidden_states.reshape(-1, hidden_states.shape[-1])
            target = target.reshape(-1)
        if vocab_parallel_group is not None:
            raise ValueError("fused_linear_cross_entropy: bias is not supported with a vocabulary-parallel group")
        logits = F.linear(hidden_states, weight, bias)
        return F.cross_entropy(logits, target, ignore_index=ignore_index, reduction=reduction)
    return LinearCrossEntropyFunction.apply(hidden_states, weight, target, ignore_index, reduction, chunk_size,
                                            v_chunk_size, vocab_parallel_group, vocab_start, shard_tokens,
                                            grad_hidden_scale, vocab_size)


# Set by set_vocab_parallel(): the model forward then treats ``lm_head.weight`` as this rank's
# slice of vocabulary rows and the ranks' tokens as shards of one batch.
_VOCAB_PARALLEL = {"group": None, "vocab_start": 0, "grad_hidden_scale": 1.0, "vocab_size": None}


def set_vocab_parallel(group, vocab_start: int = 0, grad_hidden_scale: float = 1.0,
                       vocab_size: int | None = None) -> None:
    """Switch ``bastile_lce_forward`` to the vocabulary-parallel loss (``group=None`` switches back)."""
    _VOCAB_PARALLEL.update(group=group, vocab_start=int(vocab_start), grad_hidden_scale=float(grad_hidden_scale),
                           vocab_size=vocab_size)


def bastile_lce_forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None,
                        inputs_embeds=None, labels=None, use_cache=None, output_attentions=None,
                        output_hidden_states=None, cache_position=None, logits_to_keep=0, return_dict=None,
                        **kwargs):
    """Replacement for ``Qwen3ForCausalLM.forward`` (:444-511): in training with labels the
    shifted hidden states go straight into the fused loss and ``logits`` is ``None``;
    otherwise the stock ``lm_head`` + ``loss_function`` path runs."""
    from transformers.modeling_outputs import CausalLMOutputWithPast

    cfg = self.config
    if output_attentions is None:
        output_attentions = cfg.output_attentions
    if output_hidden_states is None:
        output_hidden_states = cfg.output_hidden_states
    if return_dict is None:
        return_dict = getattr(cfg, "return_dict", True)

    outputs = self.model(
        input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
        past_key_values=past_key_values, inputs_embeds=inputs_embeds, use_cache=use_cache,
        output_attentions=output_attentions, output_hidden_states=output_hidden_states,
        cache_position=cache_position, **kwargs,
    )
    hidden_states = outputs[0]
    logits = loss = None
    if self.training and labels is not None:
        # Next-token labels for EVERY position: position t is scored against labels[t + 1] and the
        # last position of each sequence against ignore_index.  Those rows add nothing to the loss,
        # to n_valid or to any gradient, so the result is that of the reference's
        # hidden[..., :-1, :].contiguous() / labels[..., 1:].contiguous() (:483-492) - without either
        # copy at any batch size, and without the zero-padded gradient that autograd's backward of
        # the slice would allocate: d(hidden) comes back for all positions at once.
        shift_labels = F.pad(labels[..., 1:], (0, 1), value=-100)
        vp = _VOCAB_PARALLEL
        if vp["group"] is None:
            loss = fused_linear_cross_entropy(hidden_states, self.lm_head.weight, shift_labels,
                                              bias=getattr(self.lm_head, "bias", None), ignore_index=-100)
        else:
            loss = fused_linear_cross_entropy(hidden_states, self.lm_head.weight, shift_labels, ignore_index=-100,
                                              vocab_parallel_group=vp["group"], vocab_start=vp["vocab_start"],
                                              shard_tokens=True, grad_hidden_scale=vp["grad_hidden_scale"],
                                              vocab_size=vp["vocab_size"])
    else:
        keep = slice(-logits_to_keep, None) if isinstance(logits_to_keep, int) else logits_to_keep
        logits = self.lm_head(hidden_states[:, keep, :])
        if labels is not None:
            loss = self.loss_function(logits=logits, labels=labels, vocab_size=cfg.vocab_size, **kwargs)

    if not return_dict:
        out = (logits,) + tuple(outputs[1:])
        return ((loss,) + out) if loss is not None else out
    return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=outputs.past_key_values,
                                  hidden_states=outputs.hidden_states, attentions=outputs.attentions)


def warmup_fused_lce(hidden_size: int = 4096, vocab_size: int = 151936, dtype: torch.dtype = torch.bfloat16,
                     device: str = "cuda"):
    """One tiny forward+backward at the model's (hidden, vocab) (:517-529)."""
    x = torch.randn(8, hidden_size, dtype=dtype, device=device, requires_grad=True)
    w = torch.randn(vocab_size, hidden_size, dtype=dtype, device=device, requires_grad=True)
    t = torch.randint(0, vocab_size, (8,), device=device)
    fused_linear_cross_entropy(x, w, t).backward()
    torch.cuda.synchronize()
