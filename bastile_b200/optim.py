"""AdamW on the sm_100a streaming kernel (``bt_adamw_step``).

Same hyper-parameters, state names (``exp_avg``, ``exp_avg_sq``, ``step``) and update rule as
``torch.optim.AdamW`` (decoupled weight decay, bias correction, ``eps`` added after the square
root), so a ``state_dict`` moves between the two.  Moments are kept in the parameter's dtype,
the arithmetic is fp32.  The reference has no optimizer; its benchmark runs the torch one
inside the timed step (tests/benchmarks/e2e/qwen_8b_seqlen.py:122-125).
"""

from __future__ import annotations

import ctypes
from collections import defaultdict

import torch

from . import _lib


class AdamW(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2):
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("AdamW: invalid hyper-parameter")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        lib = _lib.get_lib()
        for group in self.param_groups:
            buckets = defaultdict(list)  # (device, dtype) -> [(p, g, m, v)]
            step_no = None
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("bastile_b200 AdamW does not take sparse gradients")
                _lib.require_cuda(p, p.grad)
                if not p.is_contiguous():
                    raise RuntimeError("bastile_b200 AdamW needs contiguous parameters")
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
                st["step"] = int(st["step"]) + 1
                step_no = st["step"] if step_no is None else step_no
                g = p.grad
                if g.dtype != p.dtype:
                    g = g.to(p.dtype)
                if not g.is_contiguous():
                    g = g.contiguous()
                buckets[(p.device, p.dtype, st["step"])].append((p, g, st["exp_avg"], st["exp_avg_sq"]))
            for (dev, dtype, step), items in buckets.items():
                n = len(items)
                arr = ctypes.c_void_p * n
                ps = arr(*[t[0].data_ptr() for t in items])
                gs = arr(*[t[1].data_ptr() for t in items])
                ms = arr(*[t[2].data_ptr() for t in items])
                vs = arr(*[t[3].data_ptr() for t in items])
                ns = (ctypes.c_int64 * n)(*[t[0].numel() for t in items])
                b1, b2 = group["betas"]
                small = sum(1 for t in items if t[0].numel() <= 65536)
                launches = (n - small) + (small + 47) // 48  # one per large tensor, 48 small ones per launch
                with _lib.device_of(dev), _lib.timed("adamw", launches, dev):
                    rc = lib.bt_adamw_step(ps, gs, ms, vs, ns, n, float(group["lr"]), float(b1), float(b2),
                                           float(group["eps"]), float(group["weight_decay"]), int(step),
                                           _lib.dtype_code(dtype), _lib.stream_ptr(dev))
                _lib.check(rc, "bt_adamw_step")
        return loss
