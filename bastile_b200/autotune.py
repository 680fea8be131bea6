"""Warm-up and cache management (src/bastile/autotune.py:7-59 of the reference).

The kernels are compiled ahead of time, so "warm-up" means loading the shared
library and launching the small kernels once (which also creates the CUDA
context state they need); the tensor-core kernels are touched as well so that
their tensor-map driver entry point is resolved before the first training step.
"""

from __future__ import annotations

import logging
from pathlib import Path

import torch

_CACHE_DIR = Path.home() / ".cache" / "bastile"


def clear_cache() -> None:
    """Delete ``~/.cache/bastile/*.json`` (kept for API parity; nothing writes there)."""
    if not _CACHE_DIR.exists():
        return
    for f in _CACHE_DIR.glob("*.json"):
        try:
            f.unlink()
        except OSError:
            pass


def warmup_all_kernels(batch_size: int = 4, seq_len: int = 512, hidden_size: int = 2048,
                       intermediate_size: int = 5504, dtype: torch.dtype = torch.bfloat16,
                       device: str = "cuda") -> None:
    """Run each kernel family once on small tensors; returns silently without CUDA."""
    if not torch.cuda.is_available():
        return
    try:
        from .ops.rms_norm import rms_norm
        from .ops.swiglu import swiglu

        bt = batch_size * seq_len
        x = torch.randn(bt, hidden_size, dtype=dtype, device=device)
        w = torch.ones(hidden_size, dtype=dtype, device=device)
        for _ in range(3):
            rms_norm(x, w, eps=1e-6)
        torch.cuda.synchronize()
        gate = torch.randn(bt, intermediate_size, dtype=dtype, device=device)
        up = torch.randn(bt, intermediate_size, dtype=dtype, device=device)
        for _ in range(3):
            swiglu(gate, up)
        torch.cuda.synchronize()
        if dtype in (torch.bfloat16, torch.float16):
            # one small launch of the tensor-core kernels: resolves the tensor-map driver entry
            # point and sets the shared-memory attributes before the first training step
            from .ops.fused_linear_cross_entropy import fused_linear_cross_entropy
            from .ops.swiglu import SwiGLUMLPFunction

            xs = torch.randn(256, 256, dtype=dtype, device=device)
            wg = torch.randn(512, 256, dtype=dtype, device=device)
            wd = torch.randn(256, 512, dtype=dtype, device=device)
            SwiGLUMLPFunction.apply(xs, wg, wg, wd)
            fused_linear_cross_entropy(xs, wg, torch.zeros(256, dtype=torch.int64, device=device))
            torch.cuda.synchronize()
    except Exception as exc:
        logging.getLogger(__name__).debug("Warmup skipped: %s", exc)
