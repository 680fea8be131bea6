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
after accumulation) and with gradient accumulation over several backward passes (a second
gradient for a parameter that was already updated raises).  A parameter that is used in several
places of the graph (tied embeddings) is fine: autograd sums the contributions before the one
accumulation that fires the hook, and every kernel that reads the weight in the backward pass
has been queued by then.

``master_weights=True`` keeps an fp32 copy of every parameter and fp32 moments (state names
``master``, ``exp_avg``, ``exp_avg_sq``) and writes the rounded parameter back in its own dtype
(``bt_adamw_master_step``): "bf16 parameters / fp32 master".

:class:`ShardedAdamW` is the multi-GPU form: gradient reduction, the update of this rank's
1/N of every bucket and the re-assembly of the parameters, all queued underneath the backward
pass as the gradients arrive.
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
                 overlap_backward: bool = False, background_ctas_per_sm: int = 0, master_weights: bool = False,
                 check_device_status: bool = False):
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("AdamW: invalid hyper-parameter")
        self.overlap_backward = bool(overlap_backward)
        self.master_weights = bool(master_weights)
        # step() ends with a synchronising read of the device status words (bounded waits that ran
        # out, labels outside the vocabulary) and raises if any is set; off by default because the
        # ops themselves never synchronise
        self.check_device_status = bool(check_device_status)
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
            if self.overlap_backward and p.requires_grad and hasattr(p, "register_post_accumulate_grad_hook"):
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad_ready))

    def close(self):
        """Remove the gradient hooks.  A hook ties parameter -> optimizer -> parameter through a
        reference that Python's cycle collector cannot see, so an optimizer created with
        ``overlap_backward=True`` (and its model and state) is only freed after ``close()``."""
        for h in self._hooks:
            h.remove()
        self._hooks.clear()

    @torch.no_grad()
    def _on_grad_ready(self, p):
        if (not self.overlap_backward or p.grad is None or not p.is_cuda or p.numel() < _OVERLAP_MIN_NUMEL
                or p.grad.is_sparse):
            return
        if p in self._early:
            raise RuntimeError("AdamW(overlap_backward=True): a second gradient arrived for a parameter that was "
                               "already updated in this step (several backward passes per step are not supported)")
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
        if self.check_device_status:
            _lib.check_all_status()
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
                sdt = torch.float32 if self.master_weights else p.dtype
                st["exp_avg"] = torch.zeros_like(p, dtype=sdt, memory_format=torch.contiguous_format)
                st["exp_avg_sq"] = torch.zeros_like(p, dtype=sdt, memory_format=torch.contiguous_format)
                if self.master_weights:
                    st["master"] = p.detach().to(torch.float32, memory_format=torch.contiguous_format, copy=True)
            st["step"] = int(st["step"]) + 1
            g = p.grad
            if g.dtype != p.dtype:
                g = g.to(p.dtype)
            if not g.is_contiguous():
                g = g.contiguous()
            if self.master_weights:
                b1, b2 = group["betas"]
                with _lib.device_of(p.device), _lib.timed("adamw", 1, p.device):
                    rc = lib.bt_adamw_master_step(st["master"].data_ptr(), st["exp_avg"].data_ptr(),
                                                  st["exp_avg_sq"].data_ptr(), g.data_ptr(), p.data_ptr(), p.numel(),
                                                  float(group["lr"]), float(b1), float(b2), float(group["eps"]),
                                                  float(group["weight_decay"]), int(st["step"]), 1.0,
                                                  int(ctas_per_sm), _lib.dtype_code(p.dtype), _lib.stream_ptr(p.device))
                _lib.check(rc, "bt_adamw_master_step")
                continue
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


# ------------------------------------------------------------------------------------------
class _Bucket:
    __slots__ = ("params", "offsets", "numel", "flat_p", "flat_g", "lo", "hi", "state", "pending", "arrived",
                 "launched", "device", "dtype", "sinks")


def _cuda_update(bucket, step, hyper, master_weights):
    """This rank's slice of a bucket through the streaming kernels, on the current stream."""
    lib = _lib.get_lib()
    dev, n = bucket.device, bucket.hi - bucket.lo
    p, g, st = bucket.flat_p[bucket.lo:bucket.hi], bucket.flat_g[bucket.lo:bucket.hi], bucket.state
    lr, (b1, b2), eps, wd = hyper["lr"], hyper["betas"], hyper["eps"], hyper["weight_decay"]
    code, stream = _lib.dtype_code(bucket.dtype), _lib.stream_ptr(dev)
    with _lib.device_of(dev), _lib.timed("adamw", 1, dev):
        if master_weights:
            rc = lib.bt_adamw_master_step(st["master"].data_ptr(), st["exp_avg"].data_ptr(),
                                          st["exp_avg_sq"].data_ptr(), g.data_ptr(), p.data_ptr(), n, float(lr),
                                          float(b1), float(b2), float(eps), float(wd), int(step), 1.0, 0, code, stream)
        else:
            one = ctypes.c_void_p * 1
            rc = lib.bt_adamw_step(one(p.data_ptr()), one(g.data_ptr()), one(st["exp_avg"].data_ptr()),
                                   one(st["exp_avg_sq"].data_ptr()), (ctypes.c_int64 * 1)(n), 1, float(lr), float(b1),
                                   float(b2), float(eps), float(wd), int(step), 0, code, stream)
    _lib.check(rc, "sharded AdamW update")


class ShardedAdamW:
    """Data-parallel gradient averaging and AdamW as ONE object, for one process per GPU.

    The reference scales out with FSDP FULL_SHARD around its patched model
    (tests/benchmarks/e2e/qwen_8b_fsdp.py:161-168); this is the part of that recipe that costs
    time when the model fits one GPU - reduce-scatter of the gradients, a sharded optimizer,
    all-gather of the parameters - without re-sharding the weights for every layer:

    * parameters are re-laid as views into flat buckets (``bucket_mb`` each, filled in reverse
      registration order, the order in which gradients become final; 1 GiB measured best on a
      Qwen3-8B step on two B200: 416 ms against 420 ms with 256 MiB and 429 ms with 64 MiB; the
      parameters whose gradients arrive last go into smaller buckets of ``last_bucket_mb``,
      a quarter of ``bucket_mb`` unless given, because their collectives are what a step exposes);
    * a post-accumulate-grad hook copies each gradient into its bucket on a side stream - unless
      the op that produced it (the MLP block, the fused loss) found the bucket view registered as
      the weight's gradient destination and wrote it there in the first place; when a
      bucket is complete the side stream reduce-scatters it (NCCL, average), runs the AdamW
      kernel on this rank's 1/N slice of the bucket (moments - and the fp32 master copy with
      ``master_weights=True`` - exist only for that slice) and all-gathers the bucket's
      parameters in place - all underneath the rest of the backward pass;
    * ``step()`` handles buckets whose gradients never all arrived (missing ones count as zero)
      and makes the current stream wait for the side stream: what the step leaves exposed is the
      last bucket's reduction, update and all-gather.

    One ``backward()`` per ``step()``; no gradient clipping or other use of ``.grad`` (gradients
    are consumed by the hook and ``.grad`` is left ``None``).  ``zero_grad()`` exists for loop
    compatibility.  With a group of one rank (or no process group) it is a flat, overlapped AdamW.
    ``update_fn(bucket, step, hyper, master_weights)`` replaces the CUDA kernels (tests on CPU ranks).
    """

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2,
                 group=None, bucket_mb: int = 1024, master_weights: bool = False, update_fn=None,
                 last_bucket_mb: int | None = None):
        import torch.distributed as dist

        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("ShardedAdamW: invalid hyper-parameter")
        self.hyper = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        self.master_weights = bool(master_weights)
        self._update_fn = update_fn or _cuda_update
        self._dist = dist if (dist.is_available() and dist.is_initialized()) else None
        self.group = group
        self.world = self._dist.get_world_size(group) if self._dist else 1
        self.rank = self._dist.get_rank(group) if self._dist else 0
        self._nccl = bool(self._dist) and self._dist.get_backend(group) == "nccl"
        self.step_count = 0
        self.buckets: list[_Bucket] = []
        self._where: dict = {}
        self._streams: dict = {}
        self._hooks = []
        last_mb = max(1, int(bucket_mb) // 4) if last_bucket_mb is None else int(last_bucket_mb)
        self._build([p for p in params if p.requires_grad], int(bucket_mb) << 20, min(last_mb, int(bucket_mb)) << 20)

    # -- layout
    def _build(self, params, bucket_bytes, last_bucket_bytes):
        align = 128  # elements: every parameter view starts on a 256-byte (16-bit) boundary
        quantum = align * self.world
        open_buckets: dict = {}

        def close(key):
            units = open_buckets.pop(key, None)
            if not units:
                return
            dev, dtype = key
            b = _Bucket()
            b.params, b.offsets, off = [], [], 0
            for unit in reversed(units):  # registration order inside the bucket (gate | up stay adjacent)
                off = (off + align - 1) // align * align
                for p in unit:  # members of a unit stay back to back, as they were
                    b.params.append(p)
                    b.offsets.append(off)
                    off += p.numel()
            b.numel = (off + quantum - 1) // quantum * quantum
            b.device, b.dtype = dev, dtype
            b.flat_p = torch.zeros(b.numel, dtype=dtype, device=dev)
            b.flat_g = torch.zeros(b.numel, dtype=dtype, device=dev)
            with torch.no_grad():
                for p, o in zip(b.params, b.offsets):
                    view = b.flat_p[o:o + p.numel()].view(p.shape)
                    view.copy_(p.detach())
                    p.data = view
            shard = b.numel // self.world
            b.lo, b.hi = self.rank * shard, (self.rank + 1) * shard
            sdt = torch.float32 if self.master_weights else dtype
            b.state = {"exp_avg": torch.zeros(shard, dtype=sdt, device=dev),
                       "exp_avg_sq": torch.zeros(shard, dtype=sdt, device=dev)}
            if self.master_weights:
                b.state["master"] = b.flat_p[b.lo:b.hi].to(torch.float32, copy=True)
            b.pending, b.arrived, b.launched = len(b.params), set(), False
            b.sinks = []
            for i, p in enumerate(b.params):
                self._where[p] = (b, i)
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))
                if dev.type == "cuda":
                    # ops that allocate this weight's gradient themselves write it here directly
                    o = b.offsets[i]
                    dest = b.flat_g[o:o + p.numel()].view(p.shape)
                    _lib.register_grad_sink(p.data, dest)
                    b.sinks.append(dest)
            self.buckets.append(b)

        # Units: runs of parameters that already lie one after the other in memory, in registration
        # order (q/k/v weights stacked for the one-product projections, for instance).  A unit keeps
        # its order and stays in one bucket, so whatever relies on that layout still finds it.
        units: list = []
        for p in params:
            if not p.is_contiguous():
                raise RuntimeError("ShardedAdamW needs contiguous parameters")
            prev = units[-1][-1] if units else None
            if (prev is not None and prev.device == p.device and prev.dtype == p.dtype
                    and p.data_ptr() == prev.data_ptr() + prev.numel() * prev.element_size()
                    and (prev.numel() * prev.element_size()) % 16 == 0):
                units[-1].append(p)
            else:
                units.append([p])
        def nbytes(unit):
            return sum(p.numel() * p.element_size() for p in unit)

        # Buckets are filled in reverse registration order: the order in which gradients become final.
        # What a step leaves exposed is the collectives of the buckets that complete last, so the last
        # 2 x bucket_bytes of parameters go into buckets of last_bucket_bytes: their reductions start
        # while the first layers' backward still runs.  A tensor as large as a bucket (embedding,
        # lm_head) gets a bucket of its own instead of holding its neighbours back, and two neighbours
        # of the same shape (gate | up, k | v) are never separated, so that an op which writes both
        # gradients as one stacked result finds their destinations side by side.
        order = list(reversed(units))
        remaining: dict = {}
        for unit in order:
            key = (unit[0].device, unit[0].dtype)
            remaining[key] = remaining.get(key, 0) + nbytes(unit)
        def twins(a, b):
            return (a is not None and b is not None and len(a) == 1 and len(b) == 1 and a[0].dim() >= 2
                    and a[0].shape == b[0].shape and a[0].device == b[0].device and a[0].dtype == b[0].dtype)

        sizes: dict = {}
        for i, unit in enumerate(order):
            key = (unit[0].device, unit[0].dtype)
            limit = bucket_bytes if remaining[key] > 2 * bucket_bytes else last_bucket_bytes
            size = nbytes(unit)
            held = open_buckets.get(key)
            if size >= limit and held and not twins(held[-1], unit):
                close(key)
                sizes[key] = 0
            open_buckets.setdefault(key, []).append(unit)
            sizes[key] = sizes.get(key, 0) + size
            remaining[key] -= size
            nxt = order[i + 1] if i + 1 < len(order) else None
            # a pair stays together; a run of three or more same-shaped tensors may still be cut after a pair
            pair_open = twins(unit, nxt) and not (len(open_buckets[key]) > 1 and twins(open_buckets[key][-2], unit))
            if sizes[key] >= limit and not pair_open:
                close(key)
                sizes[key] = 0
        for key in list(open_buckets):
            close(key)

    # -- streams (none on CPU tensors)
    def _side(self, dev):
        if dev.type != "cuda":
            return None
        s = self._streams.get(dev)
        if s is None:
            s = self._streams[dev] = torch.cuda.Stream(device=dev)
        return s

    class _On:
        def __init__(self, stream):
            self.ctx = torch.cuda.stream(stream) if stream is not None else None

        def __enter__(self):
            if self.ctx is not None:
                self.ctx.__enter__()

        def __exit__(self, *exc):
            if self.ctx is not None:
                self.ctx.__exit__(*exc)
            return False

    # -- backward-time work
    @torch.no_grad()
    def _on_grad(self, p):
        g = p.grad
        if g is None:
            return
        b, i = self._where[p]
        if i in b.arrived:
            raise RuntimeError("ShardedAdamW: a second gradient arrived for a parameter within one step "
                               "(several backward passes per step are not supported)")
        side = self._side(b.device)
        if side is not None:
            side.wait_stream(torch.cuda.current_stream(b.device))  # the gradient's kernels are queued there
        o = b.offsets[i]
        dest = b.flat_g[o:o + p.numel()]
        if g.data_ptr() != dest.data_ptr():  # (an op that knew the destination wrote it there already)
            with self._On(side):
                dest.view(p.shape).copy_(g)
            if side is not None:
                g.record_stream(side)
        p.grad = None
        b.arrived.add(i)
        b.pending -= 1
        if b.pending == 0:
            self._launch(b)

    def _launch(self, b):
        """Reduce, update this rank's slice, re-assemble: queued on the side stream."""
        side = self._side(b.device)
        with self._On(side):
            if self.world > 1:
                shard_g = b.flat_g[b.lo:b.hi]
                if self._nccl:
                    self._dist.reduce_scatter_tensor(shard_g, b.flat_g, op=self._dist.ReduceOp.AVG, group=self.group)
                else:  # backends without reduce-scatter / average (gloo on CPU ranks)
                    self._dist.all_reduce(b.flat_g, group=self.group)
                    shard_g.div_(self.world)
            self._update_fn(b, self.step_count + 1, self.hyper, self.master_weights)
            if self.world > 1:
                self._dist.all_gather_into_tensor(b.flat_p, b.flat_p[b.lo:b.hi], group=self.group)
        b.launched = True

    # -- loop surface
    def zero_grad(self, set_to_none: bool = True):
        for b in self.buckets:
            for p in b.params:
                p.grad = None

    @torch.no_grad()
    def step(self):
        for b in self.buckets:
            if not b.launched:
                if b.arrived:  # some parameters of the bucket got no gradient: they count as zero
                    side = self._side(b.device)
                    with self._On(side):
                        for i, (p, o) in enumerate(zip(b.params, b.offsets)):
                            if i not in b.arrived:
                                b.flat_g[o:o + p.numel()].zero_()
                    self._launch(b)
                # a bucket none of whose parameters received a gradient is left alone, as
                # torch.optim skips parameters without .grad
            b.pending, b.launched = len(b.params), False
            b.arrived = set()
        for dev, side in self._streams.items():
            torch.cuda.current_stream(dev).wait_stream(side)
        self.step_count += 1

    def close(self):
        """Remove the gradient hooks (they tie parameters and this object together through a
        reference the cycle collector cannot see: without this call neither is ever freed)."""
        for h in self._hooks:
            h.remove()
        self._hooks.clear()
        for b in self.buckets:
            _lib.unregister_grad_sinks(b.sinks)
            b.sinks = []

    def state_bytes(self) -> int:
        """Bytes of optimizer state (moments, master copy) this rank holds."""
        return sum(t.numel() * t.element_size() for b in self.buckets for t in b.state.values())
