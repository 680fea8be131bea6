"""numpy restatement of the reference ops (fp32 storage, float64 reductions).

Every function cites the lines of the reference it follows
(paths are relative to the aghilann/bastile source tree).  Inputs are numpy
arrays (any float dtype); results are float32 unless stated.  Rounding to a
16-bit storage type is the caller's business: this is the *unrounded* fp32
answer that bf16 results are compared with at rtol = atol = 2e-2.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32
F64 = np.float64


# --------------------------------------------------------------------- RMSNorm
def rms_norm_fwd(x, w, eps=1e-6):
    """y = x * rsqrt(mean(x^2) + eps) * w; returns (y, rstd).

    src/bastile/ops/rms_norm.py:15-34 (_rms_fwd): fp32 math, one rounding at the store."""
    x = np.asarray(x, F64)
    n = x.shape[-1]
    rstd = 1.0 / np.sqrt((x * x).sum(-1, keepdims=True) / n + eps)
    y = x * rstd * np.asarray(w, F64)
    return y.astype(F32), rstd[..., 0].astype(F32)


def rms_norm_bwd(dy, x, w, rstd=None, eps=1e-6):
    """dx = (dy*w - xhat*mean(xhat*dy*w))*rstd, dw = sum_rows dy*xhat.

    src/bastile/ops/rms_norm.py:37-68 (_rms_bwd) and :150-153 (partial sums -> dw)."""
    x = np.asarray(x, F64)
    dy = np.asarray(dy, F64)
    w = np.asarray(w, F64)
    n = x.shape[-1]
    if rstd is None:
        rstd = 1.0 / np.sqrt((x * x).sum(-1) / n + eps)
    r = np.asarray(rstd, F64)[..., None]
    xhat = x * r
    wdy = dy * w
    c = (xhat * wdy).sum(-1, keepdims=True) / n
    dx = (wdy - xhat * c) * r
    dw = (dy * xhat).reshape(-1, n).sum(0)
    return dx.astype(F32), dw.astype(F32)


# ------------------------------------------------------------------------ RoPE
def rope(q, k, cos, sin, negate_sin=False):
    """Rotate-half RoPE of q [B,Hq,T,D] and k [B,Hk,T,D] with cos/sin [1|B, T, D or D/2].

    src/bastile/ops/rope.py:44-90 (_rope_kernel): o1 = x1*cos - x2*sin, o2 = x2*cos + x1*sin
    on the two halves of head_dim; :93-122: only the first D/2 columns of cos/sin are used;
    :132-136: the backward is the same rotation with -sin."""
    q = np.asarray(q, F64)
    k = np.asarray(k, F64)
    half = q.shape[-1] // 2
    c = np.asarray(cos, F64)[..., :half][:, None, :, :]
    s = np.asarray(sin, F64)[..., :half][:, None, :, :]
    if negate_sin:
        s = -s

    def rot(t):
        t1, t2 = t[..., :half], t[..., half:]
        return np.concatenate((t1 * c - t2 * s, t2 * c + t1 * s), axis=-1).astype(F32)

    return rot(q), rot(k)


# ------------------------------------------------- fusions across op boundaries
def add_rms_norm_fwd(x, residual, w, eps=1e-6, round_to=None):
    """stream = x + residual, y = rms_norm(stream) * w; returns (y, stream, rstd).

    The residual add of Qwen3DecoderLayer.forward (transformers modeling_qwen3.py:326 / :335)
    followed by the reference's norm (src/bastile/ops/rms_norm.py:15-34).  ``round_to`` is a
    callable that rounds the stream to its storage type before it is normalised, as the
    separate torch add does; None keeps it exact."""
    stream = np.asarray(x, F64) + np.asarray(residual, F64)
    if round_to is not None:
        stream = np.asarray(round_to(stream.astype(F32)), F64)
    y, rstd = rms_norm_fwd(stream, w, eps)
    return y, stream.astype(F32), rstd


def add_rms_norm_bwd(dy, dstream, stream, w, rstd=None, eps=1e-6):
    """Gradient of add_rms_norm_fwd with respect to the stream (= to x = to residual), and dw:
    the norm's input gradient (rms_norm.py:37-68) plus what arrives along the residual path."""
    dx, dw = rms_norm_bwd(dy, stream, w, rstd, eps)
    return (np.asarray(dx, F64) + np.asarray(dstream, F64)).astype(F32), dw


def head_norm_rope_fwd(x, w, cos, sin, eps=1e-6, round_to=None):
    """q_norm / k_norm then RoPE for x [B,T,H,D] (a projection output viewed per head), as
    Qwen3Attention.forward chains them (modeling_qwen3.py:256-261): the reference's norm
    (rms_norm.py:15-34) on head_dim-wide rows, then its rotation (rope.py:44-90).  Returns
    (out [B,T,H,D], rstd [B,T,H]).  ``round_to`` rounds the normalised heads to the storage
    type before the rotation, as two separate kernels do."""
    y, rstd = rms_norm_fwd(x, w, eps)
    if round_to is not None:
        y = round_to(y)
    yt = np.transpose(np.asarray(y, F64), (0, 2, 1, 3))
    out, _ = rope(yt, yt[:, :1], cos, sin)
    return np.transpose(out, (0, 2, 1, 3)), rstd


def head_norm_rope_bwd(dout, x, w, cos, sin, eps=1e-6, round_to=None):
    """Gradients of head_norm_rope_fwd: un-rotate with -sin (rope.py:132-136), then the norm's
    backward (rms_norm.py:37-68, 150-153).  Returns (dx [B,T,H,D], dw [D])."""
    gt = np.transpose(np.asarray(dout, F64), (0, 2, 1, 3))
    dy, _ = rope(gt, gt[:, :1], cos, sin, negate_sin=True)
    dy = np.transpose(dy, (0, 2, 1, 3))
    if round_to is not None:
        dy = round_to(dy)
    return rms_norm_bwd(dy, x, w, None, eps)


# ---------------------------------------------------------------------- SwiGLU
def _sigmoid(g):
    return 1.0 / (1.0 + np.exp(-g))


def swiglu_fwd(gate, up):
    """silu(gate) * up.  src/bastile/ops/swiglu.py:35-50 (swiglu_forward_kernel)."""
    g = np.asarray(gate, F64)
    return (g * _sigmoid(g) * np.asarray(up, F64)).astype(F32)


def swiglu_bwd(dy, gate, up):
    """dgate = dy*up*sig(g)*(1+g*(1-sig(g))), dup = dy*g*sig(g).

    src/bastile/ops/swiglu.py:67-90 (swiglu_backward_kernel)."""
    d = np.asarray(dy, F64)
    g = np.asarray(gate, F64)
    u = np.asarray(up, F64)
    sg = _sigmoid(g)
    return (d * sg * (1.0 + g * (1.0 - sg)) * u).astype(F32), (d * g * sg).astype(F32)


def mlp_fwd(x, wg, wu, wd):
    """down(silu(gate(x)) * up(x)); returns (y, gate, up, h).

    src/bastile/ops/swiglu.py:179-187 (CuTileSwiGLUMLP): three bias-free linears."""
    x = np.asarray(x, F64)
    gate = x @ np.asarray(wg, F64).T
    up = x @ np.asarray(wu, F64).T
    h = gate * _sigmoid(gate) * up
    y = h @ np.asarray(wd, F64).T
    return y.astype(F32), gate.astype(F32), up.astype(F32), h.astype(F32)


def mlp_bwd(dy, x, wg, wu, wd):
    """Gradients of mlp_fwd: returns (dx, dwg, dwu, dwd) - autograd of swiglu.py:186-187."""
    x = np.asarray(x, F64)
    dy = np.asarray(dy, F64)
    wg, wu, wd = (np.asarray(t, F64) for t in (wg, wu, wd))
    gate = x @ wg.T
    up = x @ wu.T
    sg = _sigmoid(gate)
    h = gate * sg * up
    dh = dy @ wd
    dgate = dh * sg * (1.0 + gate * (1.0 - sg)) * up
    dup = dh * gate * sg
    dx = dgate @ wg + dup @ wu
    return (dx.astype(F32), (dgate.T @ x).astype(F32), (dup.T @ x).astype(F32), (dy.T @ h).astype(F32))


# ------------------------------------------------- fused linear + cross-entropy
def lce_shard_stats(x, w, target, ignore_index=-100, v_offset=0, tile_v=4096):
    """Per-row (max, sum exp(logit - max), target logit) over one vocabulary shard.

    Online update over column tiles as in _ce_online_kernel pass 1
    (src/bastile/ops/fused_linear_cross_entropy.py:62-85); the target logit is the
    gather of :108-114 (0 for ignored rows; here also 0 when the label lies outside
    the shard [v_offset, v_offset + V))."""
    logits = np.asarray(x, F64) @ np.asarray(w, F64).T
    rows, v = logits.shape
    row_max = np.full(rows, -1e30, F64)
    sum_exp = np.zeros(rows, F64)
    for c0 in range(0, v, tile_v):
        tile = logits[:, c0:c0 + tile_v]
        new_max = np.maximum(row_max, tile.max(1))
        sum_exp = sum_exp * np.exp(row_max - new_max) + np.exp(tile - new_max[:, None]).sum(1)
        row_max = new_max
    t = np.asarray(target).reshape(-1)
    loc = t - v_offset
    owned = (t != ignore_index) & (loc >= 0) & (loc < v)
    tgt = np.where(owned, logits[np.arange(rows), np.clip(loc, 0, v - 1)], 0.0)
    return np.stack((row_max, sum_exp, tgt), -1), logits


def merge_shard_stats(stats):
    """[n_shards, rows, 3] -> [rows, 3]: log-sum-exp merge of vocabulary shards."""
    stats = np.asarray(stats, F64)
    gmax = stats[..., 0].max(0)
    gsum = (stats[..., 1] * np.exp(stats[..., 0] - gmax)).sum(0)
    return np.stack((gmax, gsum, stats[..., 2].sum(0)), -1)


def lce_fwd_bwd(x, w, target, ignore_index=-100, reduction="mean", n_shards=1):
    """loss, d hidden, d weight of cross_entropy(x @ w.T, target) with upstream grad 1.

    Follows ChunkedLinearCrossEntropyFunction (:304-399): loss_row = max + log(sum) -
    target logit (:88-91), dlogits = softmax - onehot with ignored rows zeroed (:93-100,
    126-130), dx = dlogits @ W (:173), dW = dlogits^T @ x (:181-185), mean = / n_valid
    with 0 when nothing is valid (:334-343).  With n_shards > 1 the vocabulary is split
    into equal slices whose statistics are merged by merge_shard_stats - the result
    must not depend on n_shards."""
    x = np.asarray(x, F64)
    w = np.asarray(w, F64)
    t = np.asarray(target).reshape(-1)
    rows, v = x.shape[0], w.shape[0]
    assert v % n_shards == 0
    vs = v // n_shards
    parts = [lce_shard_stats(x, w[r * vs:(r + 1) * vs], t, ignore_index, r * vs) for r in range(n_shards)]
    stats = merge_shard_stats(np.stack([p[0] for p in parts]))
    logits = np.concatenate([p[1] for p in parts], axis=1)
    valid = t != ignore_index
    n_valid = int(valid.sum())
    loss_row = np.where(valid, stats[:, 0] + np.log(stats[:, 1]) - stats[:, 2], 0.0)
    if reduction == "mean":
        scale = 1.0 / n_valid if n_valid > 0 else 0.0
    else:
        scale = 1.0
    loss = loss_row.sum() * scale
    probs = np.exp(logits - stats[:, :1]) / stats[:, 1:2]
    probs[np.arange(rows)[valid], t[valid]] -= 1.0
    probs[~valid] = 0.0
    dlogits = probs * scale
    return F32(loss), (dlogits @ w).astype(F32), (dlogits.T @ x).astype(F32)


# ----------------------------------------------------------------------- AdamW
def adamw_step(p, g, m, v, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-2):
    """One AdamW step in float64; returns (p, m, v).  The update rule of torch.optim.AdamW, which
    the reference's benchmark loop runs (tests/benchmarks/e2e/qwen_8b_seqlen.py:122-125, 154-158):
    decoupled decay, bias-corrected moments, eps added after the square root."""
    p, g, m, v = (np.asarray(t, F64) for t in (p, g, m, v))
    p = p * (1.0 - lr * weight_decay)
    m = beta1 * m + (1.0 - beta1) * g
    v = beta2 * v + (1.0 - beta2) * g * g
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    p = p - (lr / bc1) * m / (np.sqrt(v) / np.sqrt(bc2) + eps)
    return p, m, v
