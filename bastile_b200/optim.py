"""AdamW on the sm_100a streaming kernel (``bt_adamw_step``).

Same hyper-parameters, state names (``exp_avg``, ``exp_avg_sq``, ``step``) and update rule as
``torch.optim.AdamW`` (decoupled weight decay, bias correction, ``eps`` added after the square
root), so a ``state_dict`` moves between the two.  Moments are kept in the parameter's dtype,
the arithmetic is fp32.  The reference has no optimizer; its benchmark runs the torch one
inside the timed step (tests/benchmarks/e2e/qwen_8b_seqlen.py:122-125).

``overlap_backward=True`` moves the update of every large parameter to the moment its gradient
is complete: a post-accumulate-grad hook queues the kernel on a side stream that waits for the
backward work launched so far, so the bandwidth-bound update runs underneath the (tensor-core
bound) rest of the backward pass instead of after it.  ``step()`` then only updates what is
left (small tensors, parameters whose hook did not fire) and makes the current stream wait for
the side stream.  The result is bit-identical to the plain mode.  It assumes the training loop
of the reference's benchmark - exactly one ``backward()`` per ``step()``, no gradient clipping
or other use of the gradients between the two - and gradients that are final when they are
accumulated, so it must stay off under DistributedDataParallel / FSDP (they reduce gradients
after accumulation) and with gradient accumulation over several backward passes.
"""

from __future__ import annotations

import ctypes
from collections import defaultdict

import torch

from . import _lib


# parameters below this many elements are left to step(): their launches are too short to be
# worth a stream hand-over each
_OVERLAP_MIN_NUMEL = 1 << 20


class AdamW(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2,
                 overlap_backward: bool = False, background_ctas_per_sm: int = 0):
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("AdamW: invalid hyper-parameter")
        self.overlap_backward = bool(overlap_backward)
        # Resident CTAs per SM of an update that runs underneath the backward pass (0 = the kernel's
        # default).  Measured on a B200 inside a Qwen3-8B step: throttling the update to 1-2 CTAs per
        # SM stretches it past the end of the backward pass and loses more than it hides; the step is
        # power-capped, so what overlap gains is idle gaps, not free bandwidth.
        self.background_ctas_per_sm = int(background_ctas_per_sm)
        self._side_streams: dict = {}   # device -> side stream of the early updates
        self._early: set = set()        # parameters already updated during the current backward
        self._group_of: dict = {}       # parameter -> its param group
        self._hooks: list = []
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    def add_param_group(self, param_group):
        super().add_param_group(param_group)
        group = self.param_groups[-1]
        for p in group["params"]:
            self._group_of[p] = group
            if p.requires_grad and hasattr(p, "register_post_accumulate_grad_hook"):
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad_ready))

    @torch.no_grad()
    def _on_grad_ready(self, p):
        if (not self.overlap_backward or p.grad is None or not p.is_cuda or p.numel() < _OVERLAP_MIN_NUMEL
                or p in self._early or p.grad.is_sparse):
            return
        dev = p.device
        side = self._side_streams.get(dev)
        if side is None:
            side = self._side_streams[dev] = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))  # the gradient's kernels are queued there
        with torch.cuda.stream(side):
            self._update(self._group_of[p], [p], ctas_per_sm=self.background_ctas_per_sm)
        self._early.add(p)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            if self.overlap_backward:
                raise RuntimeError("AdamW(overlap_backward=True) cannot re-evaluate a closure")
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            self._update(group, [p for p in group["params"] if p not in self._early])
        for dev, side in self._side_streams.items():
            torch.cuda.current_stream(dev).wait_stream(side)
        self._early.clear()
        return loss

    def _update(self, group, params, ctas_per_sm: int = 0):
        """One AdamW step for ``params`` (members of ``group``) on the current stream."""
        lib = _lib.get_lib()
        buckets = defaultdict(list)  # (device, dtype, step) -> [(p, g, m, v)]
        for p in params:
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
                                       int(ctas_per_sm), _lib.dtype_code(dtype), _lib.stream_ptr(dev))
            _lib.check(rc, "bt_adamw_step")
